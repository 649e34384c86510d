"""ctypes binding of libb200attn.so (C ABI: include/b200attn.h).

There is deliberately no fallback: if the shared library is missing the import of any op
fails with a clear message (run `python -c "import __graft_entry__ as g; g.build()"` or
`make -C vllm-backend-public_b200/csrc`).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent          # vllm-backend-public_b200/
_DEFAULT_LIB_PATH = PKG_ROOT / "lib" / "libb200attn.so"
LIB_PATH = Path(os.environ.get("B200ATTN_LIB", _DEFAULT_LIB_PATH))
# `make core`: the host runtime, sampling and the kernels of csrc/Makefile's SRCS_MIX only -- what a model without
# paged-decode / tcgen05-prefill attention needs.  Used when the full library is not built (a first start compiles
# this part alone); the entry points it lacks raise B2Error when called.
CORE_LIB_PATH = PKG_ROOT / "lib" / "libb200core.so"

B2_OK, B2_EINVAL, B2_EUNSUPPORTED, B2_ECUDA, B2_ENOMEM, B2_ENOTFOUND, B2_EEXISTS = 0, -1, -2, -3, -4, -5, -6
KV_BF16, KV_FP8_E4M3 = 0, 1
ABI_VERSION = 5
ACT_BF16, ACT_F32 = 0, 1
NORM_LAYER, NORM_RMS = 0, 1
ROUTE_TOPK_SOFTMAX, ROUTE_SOFTMAX_ALL, ROUTE_SIGMOID_GROUPED = 0, 1, 2
GLU_SILU, GLU_CLAMPED, GLU_GELU_TANH, FF_RELU_SQ = 0, 1, 2, 3
DECAY_HEAD_SOFTPLUS, DECAY_CHANNEL_SOFTPLUS, DECAY_CHANNEL_SIGMOID_POW, DECAY_HEAD_CONST = 0, 1, 2, 3
GATE_SILU, GATE_SIGMOID = 0, 1

_ERRNAMES = {-1: "B2_EINVAL", -2: "B2_EUNSUPPORTED", -3: "B2_ECUDA", -4: "B2_ENOMEM",
             -5: "B2_ENOTFOUND", -6: "B2_EEXISTS"}


class B2Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{_ERRNAMES.get(code, code)}: {msg}")
        self.code = code


vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes): one entry per declaration in include/b200attn.h
SIGNATURES = {
    "b2_version": (i32, []),
    "b2_last_error": (C.c_char_p, []),
    "b2_reshape_and_cache": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i64, i64, i64, i64, i32, vp, vp, vp]),
    "b2_reshape_and_cache_decode": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i64, i32,
                                          vp, vp, vp]),
    "b2_paged_decode_workspace_bytes": (sz, [i32, i32, i32, i32, i32, i32, i32]),
    "b2_paged_decode_auto_splits": (i32, [i32, i32, i32, i32, i32, i32, i32]),
    "b2_paged_decode_plan_splits": (i32, [vp, i32, i32, i32, i32, i32, i32]),
    "b2_paged_decode": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64,
                              f32, i32, vp, vp, vp, sz, i32, vp]),
    "b2_paged_decode_append_fused": (i32, [i32, i32, i32]),
    "b2_paged_decode_append": (i32, [vp, vp, vp, vp, vp, i64, i64, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64,
                                     i64, i64, i64, i64, f32, i32, vp, vp, vp, sz, i32, vp]),
    "b2_paged_decode_static": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64,
                                     f32, i32, vp, vp, i32, vp]),
    "b2_decode_plan_create": (vp, [vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, f32, i32, vp, vp, vp, sz, vp]),
    "b2_decode_plan_destroy": (None, [vp]),
    "b2_decode_plan_run": (i32, [vp, vp, vp, vp, vp, i32, i64, i64, i32, vp]),
    "b2_decode_plan_run_append": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, vp, vp, i32, i64, i64, i32, vp]),
    "b2_paged_decode_simt": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64,
                                   f32, i32, vp, vp, vp]),
    "b2_prefill_attention": (i32, [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i64, i64, i64,
                                   i64, i64, f32, i32, vp, vp, vp]),
    "b2_dequant_kv_blocks": (i32, [vp, vp, vp, vp, vp, i64, i32, i32, i32, i64, i64, vp]),
    "b2_rms_norm": (i32, [vp, vp, vp, vp, i32, i32, i64, i64, i64, f32, vp]),
    "b2_silu_and_mul": (i32, [vp, vp, i32, i32, i64, i64, vp]),
    "b2_rope_and_cache": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, vp, vp, vp]),
    "b2_rope_and_cache_ex": (i32, [vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i64, i64, i64, i32, vp, vp, i32, vp]),
    "b2_skinny_gemm": (i32, [vp, vp, vp, i32, i32, i32, i64, i64, vp]),
    "b2_sample": (i32, [vp, vp, i32, i32, i64, vp, vp, vp]),
    "b2_sample_filtered": (i32, [vp, vp, i32, i32, i64, vp, vp, vp, vp, vp]),
    "b2_bm_create": (vp, [i64, i32]),
    "b2_bm_destroy": (None, [vp]),
    "b2_bm_num_free": (i64, [vp]),
    "b2_bm_num_seqs": (i64, [vp]),
    "b2_bm_seq_len": (i64, [vp, i64]),
    "b2_bm_can_append": (i32, [vp, i64, i64]),
    "b2_bm_alloc_seq": (i32, [vp, i64, i64]),
    "b2_bm_append": (i32, [vp, i64, i64, vp]),
    "b2_bm_free_seq": (i32, [vp, i64]),
    "b2_bm_fill_tables": (i32, [vp, vp, i32, vp, i32, vp]),
    "b2_bm_plan_decode": (i32, [vp, vp, i32, vp, i32, vp, vp]),
    "b2_sched_create": (vp, [i64, i32, i32, i32, i32]),
    "b2_sched_destroy": (None, [vp]),
    "b2_sched_add_request": (i32, [vp, i64, i32, i32]),
    "b2_sched_finish": (i32, [vp, i64]),
    "b2_sched_step": (i32, [vp, vp]),
    "b2_sched_step_explicit": (i32, [vp, vp, vp, i32, vp]),
    "b2_sched_num_waiting": (i64, [vp]),
    "b2_sched_num_running": (i64, [vp]),
    "b2_sched_num_free_blocks": (i64, [vp]),
    "b2_sched_generated": (i64, [vp, i64]),
    "b2_comm_alloc": (i32, [sz, vp, vp]),
    "b2_comm_open": (i32, [vp, vp]),
    "b2_comm_close": (i32, [vp]),
    "b2_comm_free": (i32, [vp]),
    "b2_comm_region_bytes": (sz, [i32, i32, i32, i32, i32]),
    "b2_comm_create": (vp, [i32, i32, vp, sz, i32, i32, i32, i32]),
    "b2_comm_destroy": (None, [vp]),
    "b2_comm_input": (vp, [vp, i32]),
    "b2_comm_gathered": (vp, [vp]),
    "b2_comm_debug_stamps": (i32, [vp, vp]),
    "b2_comm_allreduce_rms_norm": (i32, [vp, i32, vp, vp, vp, i32, i64, i64, f32, vp]),
    "b2_comm_push_allreduce_rms_norm": (i32, [vp, vp, i64, vp, vp, vp, i32, i64, i64, f32, vp]),
    "b2_comm_allgather_cols": (i32, [vp, vp, i64, i32, i32, vp]),
    "b2_embed_streams": (i32, [vp, vp, i32, vp, i32, i32, i32, f32, vp]),
    "b2_hc_step": (i32, [vp, i32, i32, i32, vp, i64, vp, vp, vp, vp, f32, i32, vp, i64, i32, vp]),
    "b2_delta_prep": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp,
                            vp, vp]),
    "b2_delta_scan": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, i32, vp, vp, vp]),
    "b2_delta_out": (i32, [vp, vp, i64, i32, i32, i32, i32, i32, vp, f32, vp, i64, vp]),
    "b2_recur_prep": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, i32, vp, i32, i32, f32, f32, i32, i32, i32, vp, i64, vp, vp, f32,
                            vp, vp, vp, i32, vp, vp, vp, vp, vp]),
    "b2_channel_scan": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, i32, vp, vp, vp]),
    "b2_gated_head_norm": (i32, [vp, vp, i64, i32, i32, i32, i32, i32, vp, f32, f32, vp, i64, vp]),
    "b2_qk_prep_cache": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, i32, vp, vp, f32, vp, f32, i32, vp, i32, vp, vp, vp, vp]),
    "b2_qknorm_cache": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, vp, vp, f32, vp, i32, vp, vp, vp, vp]),
    "b2_chunk_attention": (i32, [vp, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, f32,
                                 f32, vp]),
    "b2_masked_attention": (i32, [vp, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32,
                                  f32, f32, vp, vp, i64, vp]),
    "b2_qk_rope_cache": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp, vp, vp, vp]),
    "b2_moe_tile_rows": (i32, []),
    "b2_moe_capacity": (i32, [i32, i32]),
    "b2_moe_route": (i32, [vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp]),
    "b2_moe_select": (i32, [vp, i64, vp, i32, i32, i32, i32, vp, vp, vp]),
    "b2_moe_route_ex": (i32, [vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp]),
    "b2_moe_select_ex": (i32, [vp, i64, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp]),
    "b2_moe_align": (i32, [vp, i32, i32, i32, vp, vp, vp, vp, vp]),
    "b2_moe_gather": (i32, [vp, i64, i32, vp, i32, i32, i32, vp, vp]),
    "b2_moe_combine": (i32, [vp, i32, vp, vp, i32, i32, i32, vp, i64, i32, vp]),
    "b2_moe_experts": (i32, [vp, i64, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp, i64, i32, f32,
                             f32, vp]),
    "b2_sandwich_norm": (i32, [vp, i32, i32, vp, i64, vp, vp, vp, vp, f32, i32, vp, i64, i32, vp]),
    "b2_row_norm": (i32, [vp, i64, vp, i64, i32, i32, i32, vp, f32, vp]),
    "b2_relu_sq": (i32, [vp, i64, vp, i64, i32, i32, i32, vp]),
    "b2_glu_and_mul": (i32, [vp, i64, vp, i64, i32, i32, i32, i32, f32, f32, vp]),
    "b2_gate_mul": (i32, [vp, i64, vp, i64, vp, i64, i32, i32, i32, i32, f32, vp]),
    "b2_embed_sinusoid_norm": (i32, [vp, vp, i32, vp, vp, i32, i32, vp, vp, i32, f32, vp]),
    "b2_group_norm_step": (i32, [vp, vp, i32, i32, vp, i64, vp, vp, vp, i32, f32, vp, vp, vp, vp, vp, i32, vp, i64, i32, i32, vp]),
    "b2_shift_state": (i32, [vp, i32, vp, i32, f32, vp, vp, vp, i32, vp, vp]),
    "b2_softcap": (i32, [vp, i64, i32, i32, i32, f32, vp]),
    "b2_latent_prep": (i32, [vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, f32, vp, vp, i32, vp, i32, vp, vp, vp]),
    "b2_latent_prep_rows": (i32, [vp, i64, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, f32, vp, vp, i32, vp, i32, vp,
                                  vp, vp]),
    "b2_latent_attention": (i32, [vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp, i64, vp, i64,
                                  vp]),
    "b2_latent_gather": (i32, [vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, vp]),
    "b2_window_attention": (i32, [vp, vp, i64, i32, vp, i64, i32, vp, vp, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                  f32, i32, vp, i64, vp]),
    "b2_latent_attention_workspace": (i64, [i32, i32, i32, i32, i32, i32, i32, i32, i32]),
}

_lib = None
_partial = False


def _not_built(name: str, path: Path):
    def stub(*_a, **_k):
        raise B2Error(B2_EUNSUPPORTED, f"{name} is not part of {path.name}: build the full library "
                                       f"(`make -C {PKG_ROOT / 'csrc'}`)")
    return stub


def load() -> C.CDLL:
    """Load the library once; raise loudly when it is absent or its ABI differs."""
    global _lib, _partial
    if _lib is not None:
        return _lib
    path, partial = LIB_PATH, False
    if not path.exists() and path == _DEFAULT_LIB_PATH and CORE_LIB_PATH.exists():
        path, partial = CORE_LIB_PATH, True
    if not path.exists():
        raise ImportError(
            f"{LIB_PATH} not found: the sm_100a extension is not built. b200attn has no CPU or "
            f"PyTorch fallback; build it with `make -C {PKG_ROOT / 'csrc'}`.")
    lib = C.CDLL(str(path))
    partial = partial or path.name == CORE_LIB_PATH.name
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)      # AttributeError if the symbol is missing
        except AttributeError:
            if not partial:
                raise
            setattr(lib, name, _not_built(name, path))
            continue
        fn.restype = res
        fn.argtypes = args
    v = lib.b2_version()
    if v != ABI_VERSION:
        raise ImportError(f"{LIB_PATH}: ABI version {v}, binding expects {ABI_VERSION}")
    _lib, _partial = lib, partial
    return lib


def is_full() -> bool:
    """True when the loaded library holds every entry point (the paged-decode and tcgen05 prompt kernels too)."""
    load()
    return not _partial


def check(rc: int) -> None:
    if rc != B2_OK:
        raise B2Error(rc, load().b2_last_error().decode("utf-8", "replace"))
