"""Torch-tensor front end of the C ABI: the two device ops on the hot path.

Mirrors the call shape of vLLM's `ops.reshape_and_cache` / `ops.paged_attention_v1/v2` (the ops
the engine launched by reference benchmark-vllm/vllm_manager.py:371-374 runs each decode step),
but every argument is checked here and handed to libb200attn.so as raw pointers + sizes on the
current CUDA stream.  CUDA tensors only: there is no CPU path.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import _lib
from ._lib import KV_BF16, KV_FP8_E4M3


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# step inputs that may also live in PINNED host memory: the kernels then read them over PCIe (unified addressing),
# which replaces the H2D copy of an engine step (b200attn.step.DecodeStep(zero_copy_inputs=True))
_PINNED_OK = ("q", "k_new", "v_new")


def _need_cuda(**tensors) -> torch.device:
    dev = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda and name in _PINNED_OK and t.is_pinned():
            continue
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor (b200attn has no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"{name} is on {t.device}, expected {dev}")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _kv_dtype_of(cache: torch.Tensor) -> int:
    if cache.dtype == torch.bfloat16:
        return KV_BF16
    if cache.dtype in (torch.uint8, torch.float8_e4m3fn):
        return KV_FP8_E4M3
    raise ValueError(f"KV cache dtype {cache.dtype} unsupported (bf16 or uint8/float8_e4m3fn)")


def _check_cache(k_cache: torch.Tensor, v_cache: torch.Tensor):
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape or k_cache.dtype != v_cache.dtype:
        raise ValueError("k_cache / v_cache must both be [num_blocks, Hkv, bs, d] of one dtype")
    if k_cache.stride() != v_cache.stride():
        raise ValueError("k_cache / v_cache must share strides")
    nb, Hkv, bs, d = k_cache.shape
    s = k_cache.stride()
    if s[3] != 1 or s[2] != d:
        raise ValueError("each (block, head) tile of the KV cache must be contiguous [bs, d]")
    return nb, Hkv, bs, d, s[0], s[1]


def reshape_and_cache(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      slot_mapping: torch.Tensor, k_scale: Optional[torch.Tensor] = None,
                      v_scale: Optional[torch.Tensor] = None) -> None:
    """k_cache[slot // bs, h, slot % bs, :] = k_new[t, h, :] (same for v); slot < 0 skips the token.

    k_new / v_new: [T, Hkv, d] bf16 (the last two dims contiguous; a token stride is allowed so a
    fused QKV projection can be written without a copy).  fp8 caches need 1-element fp32 device
    tensors k_scale / v_scale."""
    lib = _lib.load()
    dev = _need_cuda(k_new=k_new, v_new=v_new, k_cache=k_cache, v_cache=v_cache, slot_mapping=slot_mapping,
                     k_scale=k_scale, v_scale=v_scale)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    if k_new.dtype != torch.bfloat16 or v_new.dtype != torch.bfloat16:
        raise ValueError("k_new / v_new must be bf16")
    if k_new.dim() != 3 or k_new.shape != v_new.shape or k_new.shape[1:] != (Hkv, d):
        raise ValueError(f"k_new / v_new must be [T, {Hkv}, {d}]")
    for t in (k_new, v_new):
        if t.stride(2) != 1 or t.stride(1) != d:
            raise ValueError("k_new / v_new: head and dim axes must be contiguous")
    T = k_new.shape[0]
    if slot_mapping.dtype != torch.int64 or slot_mapping.shape != (T,) or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 [T]")
    if kvd == KV_FP8_E4M3:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
    _lib.check(lib.b2_reshape_and_cache(
        _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping),
        T, Hkv, d, bs, k_new.stride(0) if T else Hkv * d, v_new.stride(0) if T else Hkv * d,
        bstride, hstride, kvd, _ptr(k_scale), _ptr(v_scale), _stream(dev)))


def reshape_and_cache_decode(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                             slot_mapping: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                             k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> None:
    """Decode-step KV write over DEVICE-RESIDENT block tables (b2_reshape_and_cache_decode): token b is the newest
    token of batch row b, and its slot also names the block of table column (seq_lens[b] - 1) // bs, which is
    written in the same pass -- so a step uploads seq_lens + slots instead of the [B, max_nb] table."""
    lib = _lib.load()
    dev = _need_cuda(k_new=k_new, v_new=v_new, k_cache=k_cache, v_cache=v_cache, slot_mapping=slot_mapping,
                     block_tables=block_tables, seq_lens=seq_lens, k_scale=k_scale, v_scale=v_scale)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    if k_new.dtype != torch.bfloat16 or v_new.dtype != torch.bfloat16:
        raise ValueError("k_new / v_new must be bf16")
    if k_new.dim() != 3 or k_new.shape != v_new.shape or k_new.shape[1:] != (Hkv, d):
        raise ValueError(f"k_new / v_new must be [B, {Hkv}, {d}]")
    for t in (k_new, v_new):
        if t.stride(2) != 1 or t.stride(1) != d:
            raise ValueError("k_new / v_new: head and dim axes must be contiguous")
    B = k_new.shape[0]
    if slot_mapping.dtype != torch.int64 or slot_mapping.shape != (B,) or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 [B]")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != B \
            or block_tables.stride(1) != 1 or (B > 1 and block_tables.stride(0) != block_tables.shape[1]):
        raise ValueError("block_tables must be a contiguous int32 [B, max_nb]")
    if seq_lens.dtype != torch.int32 or seq_lens.shape != (B,) or not seq_lens.is_contiguous():
        raise ValueError("seq_lens must be a contiguous int32 [B]")
    if kvd == KV_FP8_E4M3:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
    _lib.check(lib.b2_reshape_and_cache_decode(
        _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(slot_mapping), _ptr(block_tables), _ptr(seq_lens),
        B, Hkv, d, bs, block_tables.shape[1], k_new.stride(0) if B else Hkv * d, v_new.stride(0) if B else Hkv * d,
        bstride, hstride, kvd, _ptr(k_scale), _ptr(v_scale), _stream(dev)))


def decode_workspace_bytes(B: int, Hq: int, Hkv: int, d: int, bs: int, max_nb: int, num_splits: int = 0) -> int:
    return int(_lib.load().b2_paged_decode_workspace_bytes(B, Hq, Hkv, d, bs, max_nb, num_splits))


def decode_auto_splits(B: int, Hq: int, Hkv: int, d: int, bs: int, max_nb: int, kv_dtype: int = KV_BF16) -> int:
    return int(_lib.load().b2_paged_decode_auto_splits(B, Hq, Hkv, d, bs, max_nb, kv_dtype))


def plan_num_splits(seq_lens_host: torch.Tensor, Hq: int, Hkv: int, d: int = 128, bs: int = 16,
                    kv_dtype: int = KV_BF16) -> int:
    """Schedule choice from the scheduler's HOST copy of seq_lens (int32 CPU tensor): 1 = single-pass grid,
    0 = dynamic persistent schedule.  Pure host arithmetic (b2_paged_decode_plan_splits)."""
    if seq_lens_host.is_cuda or seq_lens_host.dtype != torch.int32 or not seq_lens_host.is_contiguous():
        raise ValueError("seq_lens_host must be a contiguous int32 CPU tensor")
    rc = _lib.load().b2_paged_decode_plan_splits(seq_lens_host.data_ptr(), seq_lens_host.numel(), Hq, Hkv, d, bs, kv_dtype)
    if rc < 0:
        _lib.check(rc)
    return int(rc)


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                 seq_lens: torch.Tensor, scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                 v_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 workspace: Optional[torch.Tensor] = None, num_splits: int = 0, impl: str = "tma") -> torch.Tensor:
    """out[b, hq] = softmax(scale * q[b, hq] . K[b, :seq_lens[b], hq // G]) . V[...]  -> bf16 [B, Hq, d].

    `workspace` is a uint8 device tensor of at least decode_workspace_bytes(...) bytes; one is
    allocated per call when omitted (the engine passes a persistent one).  `out` may be a pinned host tensor.  impl="simt" selects
    the CUDA-core A/B kernel."""
    lib = _lib.load()
    # `out` may also be a PINNED host tensor: the kernels then store the result rows straight into host memory
    # (unified addressing), which replaces the D2H copy of an engine step (b200attn.step.DecodeStep)
    out_on_host = out is not None and not out.is_cuda
    if out_on_host and not out.is_pinned():
        raise ValueError("out must be a CUDA tensor or a pinned host tensor (b200attn has no CPU path)")
    dev = _need_cuda(q=q, k_cache=k_cache, v_cache=v_cache, block_tables=block_tables, seq_lens=seq_lens,
                     k_scale=k_scale, v_scale=v_scale, out=None if out_on_host else out, workspace=workspace)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    if q.dtype != torch.bfloat16 or q.dim() != 3 or q.shape[2] != d:
        raise ValueError(f"q must be bf16 [B, Hq, {d}]")
    B, Hq, _ = q.shape
    if q.stride(2) != 1 or q.stride(1) != d:
        raise ValueError("q: head and dim axes must be contiguous")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != B \
            or not block_tables.is_contiguous():
        raise ValueError("block_tables must be a contiguous int32 [B, max_nb]")
    if seq_lens.dtype != torch.int32 or seq_lens.shape != (B,) or not seq_lens.is_contiguous():
        raise ValueError("seq_lens must be a contiguous int32 [B]")
    max_nb = block_tables.shape[1]
    if out is None:
        out = torch.empty(B, Hq, d, dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or out.shape != (B, Hq, d) or out.stride(2) != 1 or out.stride(1) != d:
        raise ValueError("out must be bf16 [B, Hq, d] with contiguous head/dim axes")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if kvd == KV_FP8_E4M3:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
    if B == 0:
        return out
    qs = q.stride(0) if B > 1 else Hq * d
    os_ = out.stride(0) if B > 1 else Hq * d
    if impl == "simt":
        _lib.check(lib.b2_paged_decode_simt(
            _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(seq_lens),
            B, Hq, Hkv, d, bs, max_nb, qs, os_, bstride, hstride, float(scale), kvd,
            _ptr(k_scale), _ptr(v_scale), _stream(dev)))
        return out
    if impl != "tma":
        raise ValueError(f"impl {impl!r}")
    need = lib.b2_paged_decode_workspace_bytes(B, Hq, Hkv, d, bs, max_nb, num_splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        if workspace is not None:
            raise ValueError(f"workspace holds {workspace.numel() * workspace.element_size()} bytes, {need} required")
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    wbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _lib.check(lib.b2_paged_decode(
        _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(seq_lens),
        B, Hq, Hkv, d, bs, max_nb, nb, qs, os_, bstride, hstride, float(scale), kvd,
        _ptr(k_scale), _ptr(v_scale), _ptr(workspace), wbytes, num_splits, _stream(dev)))
    return out


def paged_decode_append(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, slot_mapping: torch.Tensor,
                        k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                        scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                        v_scale: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                        workspace: Optional[torch.Tensor] = None, num_splits: int = 0) -> torch.Tensor:
    """One decode step of one layer in one call (b2_paged_decode_append): reshape_and_cache(k_new, v_new, ...,
    slot_mapping) of the step's new token per row, then paged_decode over seq_lens (which count that token) -- same
    bits in `out` and in the caches as the two calls.  With num_splits = 1 and Hq / Hkv <= 16 it is ONE launch: the CTA
    that owns (row, kv head) writes the row's new K/V itself before it streams the row (append_is_fused)."""
    lib = _lib.load()
    dev = _need_cuda(q=q, k_new=k_new, v_new=v_new, slot_mapping=slot_mapping, k_cache=k_cache, v_cache=v_cache,
                     block_tables=block_tables, seq_lens=seq_lens, k_scale=k_scale, v_scale=v_scale, out=out,
                     workspace=workspace)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    if q.dtype != torch.bfloat16 or q.dim() != 3 or q.shape[2] != d:
        raise ValueError(f"q must be bf16 [B, Hq, {d}]")
    B, Hq, _ = q.shape
    if q.stride(2) != 1 or q.stride(1) != d:
        raise ValueError("q: head and dim axes must be contiguous")
    if k_new.dtype != torch.bfloat16 or v_new.dtype != torch.bfloat16:
        raise ValueError("k_new / v_new must be bf16")
    if k_new.shape != (B, Hkv, d) or v_new.shape != (B, Hkv, d):
        raise ValueError(f"k_new / v_new must be [{B}, {Hkv}, {d}] (one new token per row)")
    for t in (k_new, v_new):
        if t.stride(2) != 1 or t.stride(1) != d:
            raise ValueError("k_new / v_new: head and dim axes must be contiguous")
    if slot_mapping.dtype != torch.int64 or slot_mapping.shape != (B,) or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 [B]")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != B \
            or not block_tables.is_contiguous():
        raise ValueError("block_tables must be a contiguous int32 [B, max_nb]")
    if seq_lens.dtype != torch.int32 or seq_lens.shape != (B,) or not seq_lens.is_contiguous():
        raise ValueError("seq_lens must be a contiguous int32 [B]")
    max_nb = block_tables.shape[1]
    if out is None:
        out = torch.empty(B, Hq, d, dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or out.shape != (B, Hq, d) or out.stride(2) != 1 or out.stride(1) != d:
        raise ValueError("out must be bf16 [B, Hq, d] with contiguous head/dim axes")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if kvd == KV_FP8_E4M3:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
    if B == 0:
        return out
    need = lib.b2_paged_decode_workspace_bytes(B, Hq, Hkv, d, bs, max_nb, num_splits)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        if workspace is not None:
            raise ValueError(f"workspace holds {workspace.numel() * workspace.element_size()} bytes, {need} required")
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    wbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    one = Hkv * d
    _lib.check(lib.b2_paged_decode_append(
        _ptr(out), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(slot_mapping),
        k_new.stride(0) if B > 1 else one, v_new.stride(0) if B > 1 else one,
        _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(seq_lens),
        B, Hq, Hkv, d, bs, max_nb, nb, q.stride(0) if B > 1 else Hq * d, out.stride(0) if B > 1 else Hq * d,
        bstride, hstride, float(scale), kvd, _ptr(k_scale), _ptr(v_scale), _ptr(workspace), wbytes, num_splits,
        _stream(dev)))
    return out


def append_is_fused(Hq: int, Hkv: int, num_splits: int) -> bool:
    """True when paged_decode_append runs as one launch for these heads and this schedule (b2_paged_decode_append_fused)."""
    rc = _lib.load().b2_paged_decode_append_fused(Hq, Hkv, num_splits)
    if rc < 0:
        _lib.check(rc)
    return rc == 1


class DecodePlan:
    """Per-engine decode handle (b2_decode_plan_*): caches, geometry, scales and workspace are fixed at creation, where
    the two TMA descriptors are encoded and the workspace header is zeroed; run() is then argument checks + launches
    (no driver call, no getenv; two launches for the dynamic schedule).  The caller keeps caches and workspace alive."""

    def __init__(self, k_cache: torch.Tensor, v_cache: torch.Tensor, max_batch: int, Hq: int, max_nb: int,
                 scale: Optional[float] = None, k_scale: Optional[torch.Tensor] = None,
                 v_scale: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None):
        self._lib = _lib.load()
        self._h = None
        dev = _need_cuda(k_cache=k_cache, v_cache=v_cache, k_scale=k_scale, v_scale=v_scale, workspace=workspace)
        nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
        kvd = _kv_dtype_of(k_cache)
        need = max(int(self._lib.b2_paged_decode_workspace_bytes(max_batch, Hq, Hkv, d, bs, max_nb, 0)), 256)
        if workspace is None:
            workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        elif workspace.numel() * workspace.element_size() < need:
            raise ValueError(f"workspace holds {workspace.numel() * workspace.element_size()} bytes, {need} required")
        self.dev, self.Hq, self.Hkv, self.d, self.bs, self.max_nb, self.max_batch = dev, Hq, Hkv, d, bs, max_nb, max_batch
        # the handle stores raw pointers: keep every tensor behind them alive
        self._keep = (k_cache, v_cache, k_scale, v_scale, workspace)
        self.workspace = workspace
        if scale is None:
            scale = 1.0 / math.sqrt(d)
        h = self._lib.b2_decode_plan_create(
            _ptr(k_cache), _ptr(v_cache), max_batch, Hq, Hkv, d, bs, max_nb, nb, bstride, hstride, float(scale), kvd,
            _ptr(k_scale), _ptr(v_scale), _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(dev))
        if not h:
            raise _lib.B2Error(_lib.B2_EINVAL, self._lib.b2_last_error().decode("utf-8", "replace"))
        self._h = h
        self._run = self._lib.b2_decode_plan_run

    def run(self, q: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor, out: torch.Tensor,
            num_splits: int = 0) -> torch.Tensor:
        """q / out: bf16 [B, Hq, d] (row stride allowed; pinned host memory allowed); block_tables int32 [B, max_nb]
        and seq_lens int32 [B] on the device.  Shapes are the creator's; only the cheap checks are repeated here."""
        B = q.shape[0]
        if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or q.shape[1:] != (self.Hq, self.d) \
                or out.shape != q.shape or q.stride(1) != self.d or out.stride(1) != self.d:
            raise ValueError(f"q / out must be bf16 [B, {self.Hq}, {self.d}] with contiguous head/dim axes")
        if block_tables.dtype != torch.int32 or block_tables.shape != (B, self.max_nb) or not block_tables.is_cuda \
                or block_tables.stride(1) != 1 or (B > 1 and block_tables.stride(0) != self.max_nb):
            raise ValueError(f"block_tables must be a device int32 [B, {self.max_nb}]")
        if seq_lens.dtype != torch.int32 or seq_lens.shape != (B,) or not seq_lens.is_cuda:
            raise ValueError("seq_lens must be a device int32 [B]")
        for name, t in (("q", q), ("out", out)):
            if not t.is_cuda and not t.is_pinned():
                raise ValueError(f"{name} must be a CUDA tensor or a pinned host tensor (b200attn has no CPU path)")
        qs = q.stride(0) if B > 1 else self.Hq * self.d
        os_ = out.stride(0) if B > 1 else self.Hq * self.d
        _lib.check(self._run(self._h, out.data_ptr(), q.data_ptr(), block_tables.data_ptr(), seq_lens.data_ptr(), B,
                             qs, os_, num_splits, _stream(self.dev)))
        return out

    def run_append(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, slot_mapping: torch.Tensor,
                   block_tables: torch.Tensor, seq_lens: torch.Tensor, out: torch.Tensor,
                   num_splits: int = 0) -> torch.Tensor:
        """reshape_and_cache_decode(k_new, v_new, ..., slot_mapping, block_tables, seq_lens) + run(...) in one call
        (b2_decode_plan_run_append): one launch for the single-pass grid.  k_new / v_new: bf16 [B, Hkv, d] rows (strided
        views and pinned host memory allowed); slot_mapping int64 [B] and the RESIDENT block_tables int32 [B, max_nb]
        (updated in place) on the device."""
        B = q.shape[0]
        if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or q.shape[1:] != (self.Hq, self.d) \
                or out.shape != q.shape or q.stride(1) != self.d or out.stride(1) != self.d:
            raise ValueError(f"q / out must be bf16 [B, {self.Hq}, {self.d}] with contiguous head/dim axes")
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            if t.dtype != torch.bfloat16 or t.shape != (B, self.Hkv, self.d) or t.stride(2) != 1 or t.stride(1) != self.d:
                raise ValueError(f"{name} must be bf16 [B, {self.Hkv}, {self.d}] with contiguous head/dim axes")
        if slot_mapping.dtype != torch.int64 or slot_mapping.shape != (B,) or not slot_mapping.is_cuda \
                or not slot_mapping.is_contiguous():
            raise ValueError("slot_mapping must be a contiguous device int64 [B]")
        if block_tables.dtype != torch.int32 or block_tables.shape != (B, self.max_nb) or not block_tables.is_cuda \
                or block_tables.stride(1) != 1 or (B > 1 and block_tables.stride(0) != self.max_nb):
            raise ValueError(f"block_tables must be a device int32 [B, {self.max_nb}]")
        if seq_lens.dtype != torch.int32 or seq_lens.shape != (B,) or not seq_lens.is_cuda:
            raise ValueError("seq_lens must be a device int32 [B]")
        for name, t in (("q", q), ("out", out), ("k_new", k_new), ("v_new", v_new)):
            if not t.is_cuda and not t.is_pinned():
                raise ValueError(f"{name} must be a CUDA tensor or a pinned host tensor (b200attn has no CPU path)")
        one = self.Hkv * self.d
        _lib.check(self._lib.b2_decode_plan_run_append(
            self._h, out.data_ptr(), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), slot_mapping.data_ptr(),
            k_new.stride(0) if B > 1 else one, v_new.stride(0) if B > 1 else one, block_tables.data_ptr(),
            seq_lens.data_ptr(), B, q.stride(0) if B > 1 else self.Hq * self.d,
            out.stride(0) if B > 1 else self.Hq * self.d, num_splits, _stream(self.dev)))
        return out

    def close(self) -> None:
        if self._h:
            self._lib.b2_decode_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------
# prompt-chunk attention and the element-wise ops of a decoder layer
# ------------------------------------------------------------------------------------------------
def dequant_kv_blocks(k_cache: torch.Tensor, v_cache: torch.Tensor, src_blocks: torch.Tensor,
                      k_out: Optional[torch.Tensor] = None, v_out: Optional[torch.Tensor] = None):
    """bf16 copies of the fp8-e4m3 cache blocks `src_blocks` (device int32 [n]): out block i = float(e4m3) of block
    src_blocks[i], exact in bf16 and still unscaled (b2_dequant_kv_blocks).  Returns (k_out, v_out),
    bf16 [n, Hkv, bs, d]; pass the cache's k_scale / v_scale to prefill_attention together with them."""
    lib = _lib.load()
    dev = _need_cuda(k_cache=k_cache, v_cache=v_cache, src_blocks=src_blocks, k_out=k_out, v_out=v_out)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    if _kv_dtype_of(k_cache) != KV_FP8_E4M3:
        raise ValueError("dequant_kv_blocks needs an fp8 (uint8) cache")
    if src_blocks.dtype != torch.int32 or src_blocks.dim() != 1 or not src_blocks.is_contiguous():
        raise ValueError("src_blocks must be a contiguous int32 [n]")
    n = src_blocks.numel()
    shape = (n, Hkv, bs, d)
    outs = []
    for o in (k_out, v_out):
        if o is None:
            o = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        elif o.dtype != torch.bfloat16 or tuple(o.shape) != shape or not o.is_contiguous():
            raise ValueError(f"k_out / v_out must be contiguous bf16 {list(shape)}")
        outs.append(o)
    _lib.check(lib.b2_dequant_kv_blocks(_ptr(outs[0]), _ptr(outs[1]), _ptr(k_cache), _ptr(v_cache), _ptr(src_blocks),
                                        n, Hkv, d, bs, bstride, hstride, _stream(dev)))
    return outs[0], outs[1]


def fp8_prefill_plan(block_tables: torch.Tensor, kv_lens_host, bs: int):
    """For prompt chunks over an fp8 cache: which cache blocks to dequantise and the block table of the scratch
    cache they land in.  kv_lens_host[c] = ctx_start[c] + len_c (host ints: the scheduler knows them).
    Returns (src_blocks device int32 [n], scratch_block_tables device int32 [n_chunks, max nb_c])."""
    n_chunks = block_tables.shape[0]
    nbs = [(int(L) + bs - 1) // bs for L in kv_lens_host]
    if len(nbs) != n_chunks or max(nbs, default=0) > block_tables.shape[1]:
        raise ValueError("kv_lens_host does not match the chunks / block_tables")
    dev = block_tables.device
    rows = torch.repeat_interleave(torch.arange(n_chunks), torch.tensor(nbs, dtype=torch.int64))
    cols = torch.cat([torch.arange(n) for n in nbs]) if nbs else torch.zeros(0, dtype=torch.int64)
    src = block_tables[rows.to(dev), cols.to(dev)].contiguous()
    bt = torch.zeros(n_chunks, max(max(nbs, default=1), 1), dtype=torch.int32)
    off = 0
    for c, n in enumerate(nbs):
        bt[c, :n] = torch.arange(off, off + n, dtype=torch.int32)
        off += n
    return src, bt.to(dev)


def _prefill_over_fp8(q, k_cache, v_cache, block_tables, cu_q, ctx_start, total_tokens, scale, out, k_scale, v_scale,
                      kv_lens_host):
    """fp8 cache: gather + dequantise the blocks each chunk can see into a bf16 scratch cache, then the bf16 kernel.
    Without kv_lens_host one device read sizes the scratch."""
    if kv_lens_host is None:
        kv_lens_host = (ctx_start.to(torch.int64) + (cu_q[1:] - cu_q[:-1]).to(torch.int64)).cpu().tolist()
    src, bt = fp8_prefill_plan(block_tables, kv_lens_host, k_cache.shape[2])
    ks, vs = dequant_kv_blocks(k_cache, v_cache, src)
    return prefill_attention(q, ks, vs, bt, cu_q, ctx_start, total_tokens, scale, out, k_scale, v_scale)


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                      cu_q: torch.Tensor, ctx_start: torch.Tensor, total_tokens: Optional[int] = None,
                      scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                      k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
                      kv_lens_host=None) -> torch.Tensor:
    """Causal attention of prompt chunks over the paged cache (b2_prefill_attention).

    q / out: bf16 [T, Hq, d] (token stride allowed); chunk c = rows cu_q[c]:cu_q[c+1], positions
    ctx_start[c] + i, blocks block_tables[c].  The chunk's K/V must already be in the cache.
    `total_tokens` = cu_q[-1] as a host int (defaults to q.shape[0]; it sizes the grid without a device sync).
    fp8 caches (uint8 + k_scale / v_scale): the visible blocks are dequantised into a bf16 scratch cache first
    (b2_dequant_kv_blocks); pass kv_lens_host = [ctx_start[c] + len_c] to size it without a device read.
    bf16 caches with k_scale / v_scale: the cache is taken to hold K / k_scale and V / v_scale (that scratch)."""
    lib = _lib.load()
    dev = _need_cuda(q=q, k_cache=k_cache, v_cache=v_cache, block_tables=block_tables, cu_q=cu_q,
                     ctx_start=ctx_start, out=out, k_scale=k_scale, v_scale=v_scale)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    if kvd == KV_FP8_E4M3:
        if k_scale is None or v_scale is None:
            raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
        if ctx_start.numel() == 0 or q.shape[0] == 0:
            return out if out is not None else torch.empty_like(q)
        return _prefill_over_fp8(q, k_cache, v_cache, block_tables, cu_q, ctx_start, total_tokens, scale, out,
                                 k_scale, v_scale, kv_lens_host)
    if q.dtype != torch.bfloat16 or q.dim() != 3 or q.shape[2] != d or q.stride(2) != 1 or q.stride(1) != d:
        raise ValueError(f"q must be bf16 [T, Hq, {d}] with contiguous head/dim axes")
    T, Hq, _ = q.shape
    n_chunks = ctx_start.numel()
    for name, t, n in (("cu_q", cu_q, n_chunks + 1), ("ctx_start", ctx_start, n_chunks)):
        if t.dtype != torch.int32 or t.shape != (n,) or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous int32 [{n}]")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != n_chunks \
            or not block_tables.is_contiguous():
        raise ValueError("block_tables must be a contiguous int32 [n_chunks, max_nb]")
    if out is None:
        out = torch.empty(T, Hq, d, dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or out.shape != (T, Hq, d) or out.stride(2) != 1 or out.stride(1) != d:
        raise ValueError("out must be bf16 [T, Hq, d] with contiguous head/dim axes")
    if total_tokens is None:
        total_tokens = T
    if not 0 <= total_tokens <= T:
        raise ValueError(f"total_tokens={total_tokens} outside [0, {T}]")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if n_chunks == 0 or total_tokens == 0:
        return out
    _lib.check(lib.b2_prefill_attention(
        _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(cu_q), _ptr(ctx_start),
        n_chunks, total_tokens, Hq, Hkv, d, bs, block_tables.shape[1], nb,
        q.stride(0) if T > 1 else Hq * d, out.stride(0) if T > 1 else Hq * d, bstride, hstride,
        float(scale), kvd, _ptr(k_scale), _ptr(v_scale), _stream(dev)))
    return out


def _rows(t: torch.Tensor, name: str):
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be bf16 [T, H] with a contiguous last axis")
    return t.shape[0], t.shape[1], (t.stride(0) if t.shape[0] > 1 else t.shape[1])


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = bf16(w * h * rsqrt(mean(h^2) + eps)); with `residual`, h = bf16(x + residual) is stored back into
    residual first (fused add).  b2_rms_norm."""
    lib = _lib.load()
    dev = _need_cuda(x=x, weight=weight, residual=residual, out=out)
    T, H, xs = _rows(x, "x")
    if weight.dtype != torch.bfloat16 or weight.shape != (H,) or not weight.is_contiguous():
        raise ValueError(f"weight must be a contiguous bf16 [{H}]")
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    To, Ho, os_ = _rows(out, "out")
    if (To, Ho) != (T, H):
        raise ValueError("out shape differs from x")
    rs = 0
    if residual is not None:
        Tr, Hr, rs = _rows(residual, "residual")
        if (Tr, Hr) != (T, H):
            raise ValueError("residual shape differs from x")
    _lib.check(lib.b2_rms_norm(_ptr(out), _ptr(x), _ptr(residual), _ptr(weight), T, H, xs, os_, rs, float(eps),
                               _stream(dev)))
    return out


def silu_and_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]  (b2_silu_and_mul)."""
    lib = _lib.load()
    dev = _need_cuda(gate_up=gate_up, out=out)
    T, H2, is_ = _rows(gate_up, "gate_up")
    if H2 % 2:
        raise ValueError("gate_up must be [T, 2*I]")
    I = H2 // 2
    if out is None:
        out = torch.empty(T, I, dtype=torch.bfloat16, device=dev)
    To, Io, os_ = _rows(out, "out")
    if (To, Io) != (T, I):
        raise ValueError("out must be [T, I]")
    _lib.check(lib.b2_silu_and_mul(_ptr(out), _ptr(gate_up), T, I, is_, os_, _stream(dev)))
    return out


def rope_and_cache(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: torch.Tensor, slot_mapping: torch.Tensor, Hq: int,
                   k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
                   write_k: bool = True) -> None:
    """Neox rotary on the q and k parts of qkv [T, (Hq + 2 Hkv) * d] in place, then K', V into the paged cache
    through slot_mapping (b2_rope_and_cache_ex).  cos_sin: fp32 [max_pos, d] = cos | sin halves per position.
    write_k=False leaves the k part of qkv unrotated (the rotated rows go to the cache only)."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, positions=positions, cos_sin=cos_sin, k_cache=k_cache, v_cache=v_cache,
                     slot_mapping=slot_mapping, k_scale=k_scale, v_scale=v_scale)
    nb, Hkv, bs, d, bstride, hstride = _check_cache(k_cache, v_cache)
    kvd = _kv_dtype_of(k_cache)
    T, W, ts = _rows(qkv, "qkv")
    if W != (Hq + 2 * Hkv) * d:
        raise ValueError(f"qkv rows must hold (Hq + 2 Hkv) * d = {(Hq + 2 * Hkv) * d} elements, got {W}")
    if positions.dtype != torch.int32 or positions.shape != (T,) or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int32 [T]")
    if slot_mapping.dtype != torch.int64 or slot_mapping.shape != (T,) or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 [T]")
    if cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or cos_sin.shape[1] != d or not cos_sin.is_contiguous():
        raise ValueError(f"cos_sin must be a contiguous fp32 [max_pos, {d}]")
    if kvd == KV_FP8_E4M3:
        for s in (k_scale, v_scale):
            if s is None or s.dtype != torch.float32 or s.numel() != 1:
                raise ValueError("fp8 KV cache needs 1-element fp32 device tensors k_scale / v_scale")
    _lib.check(lib.b2_rope_and_cache_ex(_ptr(qkv), _ptr(positions), _ptr(cos_sin), cos_sin.shape[0], _ptr(k_cache),
                                        _ptr(v_cache), _ptr(slot_mapping), T, Hq, Hkv, d, bs, ts, bstride, hstride, kvd,
                                        _ptr(k_scale), _ptr(v_scale), 1 if write_k else 0, _stream(dev)))


SKINNY_GEMM_MAX_M = 256


def skinny_gemm(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for the rows of a decode step (M <= 256): the weight-streaming tcgen05 kernel
    b2_skinny_gemm.  x bf16 [M, K] (row stride allowed), w bf16 [N, K] contiguous, out bf16 [M, N] (row stride allowed)."""
    lib = _lib.load()
    dev = _need_cuda(x=x, w=w, out=out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError("skinny_gemm: x [M, K] and w [N, K] must be bf16 with the same K")
    if x.stride(1) != 1 or not w.is_contiguous():
        raise ValueError("skinny_gemm: x rows and w must be contiguous")
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or out.shape != (M, N) or out.stride(1) != 1:
        raise ValueError(f"skinny_gemm: out must be bf16 [{M}, {N}] with contiguous rows")
    _lib.check(lib.b2_skinny_gemm(_ptr(out), _ptr(x), _ptr(w), M, N, K, x.stride(0) if M > 1 else K,
                                  out.stride(0) if M > 1 else N, _stream(dev)))
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token per row of bf16 logits [B, V]: greedy where temperature <= 0 (or None), else one Gumbel-max draw from
    softmax(logits / T) keyed by seeds[b], restricted to the top_k[b] largest logits (int32 [B]; <= 0: no limit) and then
    to the smallest top set holding top_p[b] of that mass (fp32 [B]; >= 1: no limit) -- b2_sample_filtered.
    Returns int64 [B]."""
    lib = _lib.load()
    dev = _need_cuda(logits=logits, temperature=temperature, seeds=seeds, out=out, top_k=top_k, top_p=top_p)
    B, V, st = _rows(logits, "logits")
    if B == 1:
        st = (V + 7) // 8 * 8            # one row: the stride is never used, only checked
    if temperature is not None and (temperature.dtype != torch.float32 or temperature.shape != (B,)
                                    or not temperature.is_contiguous()):
        raise ValueError("temperature must be a contiguous fp32 [B]")
    if seeds is not None and (seeds.dtype != torch.int64 or seeds.shape != (B,) or not seeds.is_contiguous()):
        raise ValueError("seeds must be a contiguous int64 [B]")
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=dev)
    elif out.dtype != torch.int64 or out.shape != (B,) or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 [B]")
    if top_k is not None and (top_k.dtype != torch.int32 or top_k.shape != (B,) or not top_k.is_contiguous()):
        raise ValueError("top_k must be a contiguous int32 [B]")
    if top_p is not None and (top_p.dtype != torch.float32 or top_p.shape != (B,) or not top_p.is_contiguous()):
        raise ValueError("top_p must be a contiguous fp32 [B]")
    _lib.check(lib.b2_sample_filtered(_ptr(out), _ptr(logits), B, V, st, _ptr(temperature), _ptr(seeds), _ptr(top_k),
                                      _ptr(top_p), _stream(dev)))
    return out


# ======================================================================================================================
# Building blocks beyond the Llama layer (csrc/hyper_norm.cu, delta_rule.cu, chunk_attention.cu, moe.cu).
# Activations / weights / caches are bf16 or fp32 (one type per call); residual streams, statistics and recurrent state
# are fp32 in both.  Small parameter vectors are fp32.
# ======================================================================================================================
from dataclasses import dataclass  # noqa: E402

from ._lib import (ACT_BF16, ACT_F32, DECAY_CHANNEL_SIGMOID_POW, DECAY_CHANNEL_SOFTPLUS,  # noqa: E402,F401
                   DECAY_HEAD_CONST, DECAY_HEAD_SOFTPLUS, FF_RELU_SQ, GATE_SIGMOID, GATE_SILU, GLU_CLAMPED, GLU_GELU_TANH, GLU_SILU, NORM_LAYER,
                   NORM_RMS, ROUTE_SIGMOID_GROUPED, ROUTE_SOFTMAX_ALL, ROUTE_TOPK_SOFTMAX)


def _act(t: torch.Tensor, name: str) -> int:
    if t.dtype == torch.bfloat16:
        return ACT_BF16
    if t.dtype == torch.float32:
        return ACT_F32
    raise ValueError(f"{name} must be bf16 or fp32, not {t.dtype}")


def _f32(t: Optional[torch.Tensor], name: str, shape=None) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or (shape is not None and tuple(t.shape) != tuple(shape)):
        raise ValueError(f"{name} must be a contiguous fp32 tensor" + (f" of shape {tuple(shape)}" if shape else ""))
    return t


def _mat(t: torch.Tensor, name: str):
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{name} must be [rows, cols] with a contiguous last axis")
    return t.shape[0], t.shape[1], (t.stride(0) if t.shape[0] > 1 else t.shape[1])


@dataclass
class SeqBatch:
    """The sequences of one step, as every varlen op of this section reads them (all int32, on the device).
    Sequence i owns batch rows cu_q[i] .. cu_q[i+1]-1 and has ctx_start[i] tokens in the cache before them; a negative
    ctx_start marks padding rows (CUDA-graph buckets).  A decode row is a sequence with one row."""
    cu_q: torch.Tensor                       # [n + 1]
    ctx_start: torch.Tensor                  # [n]
    block_tables: Optional[torch.Tensor]     # [n, max_nb]
    state_slots: Optional[torch.Tensor]      # [n]; < 0: the sequence keeps no recurrent state
    n_seq: int
    rows: int


def step_batch(arange: torch.Tensor, n_decode: int, dec_bt, dec_sl, dec_state, prefill) -> SeqBatch:
    """[decode rows | prompt chunks] of one engine step as one list of sequences.  arange: int32 [>= n_decode + 1] =
    0, 1, 2, ...; dec_sl: the decode rows' sequence lengths INCLUDING the new token (0 = padding row); prefill: the step's
    PrefillBatch or None."""
    npf = prefill.cu_q.shape[0] - 1 if prefill is not None and prefill.total_tokens else 0
    if not npf:
        return SeqBatch(arange[:n_decode + 1], dec_sl - 1, dec_bt, dec_state, n_decode, n_decode)
    rows = n_decode + prefill.total_tokens
    if not n_decode:
        return SeqBatch(prefill.cu_q, prefill.ctx_start, prefill.block_tables, prefill.state_slots, npf, rows)
    state = None if dec_state is None or prefill.state_slots is None else torch.cat([dec_state, prefill.state_slots])
    return SeqBatch(torch.cat([arange[:n_decode], prefill.cu_q + n_decode]), torch.cat([dec_sl - 1, prefill.ctx_start]),
                    torch.cat([dec_bt, prefill.block_tables]).contiguous(), state, n_decode + npf, rows)


def embed_streams(embed: torch.Tensor, tokens: torch.Tensor, streams: int, scale: float) -> torch.Tensor:
    """x[t, s, :] = embed[tokens[t]] * scale for s < streams: fp32 [T, streams, D]  (b2_embed_streams)."""
    lib = _lib.load()
    dev = _need_cuda(embed=embed, tokens=tokens)
    if tokens.dtype != torch.int64 or not tokens.is_contiguous() or not embed.is_contiguous():
        raise ValueError("tokens must be contiguous int64, embed contiguous")
    T, D = tokens.shape[0], embed.shape[1]
    x = torch.empty(T, streams, D, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_embed_streams(_ptr(x), _ptr(embed), _act(embed, "embed"), _ptr(tokens), T, D, streams, float(scale),
                                    _stream(dev)))
    return x


def hc_step(x: torch.Tensor, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
            out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None,
            norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6, norm_kind: int = NORM_LAYER,
            h_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """One pass over the fp32 residual streams x [T, S, D] (updated in place):
    with y [T, D]:      x[:, j] <- sum_s mix[s, j] * x[:, s] + out_w[j] * y      (mix / out_w None = identity / ones)
    with norm_w [D]:    returns h = norm(sum_s in_w[s] * x[:, s]) * norm_w as h_dtype (in_w None = ones).
    S = 1 with the defaults is residual add + norm.  b2_hc_step."""
    lib = _lib.load()
    dev = _need_cuda(x=x, y=y, mix=mix, out_w=out_w, in_w=in_w, norm_w=norm_w)
    if x.dtype != torch.float32 or x.dim() != 3 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32 [T, S, D]")
    T, S, D = x.shape
    ys = 0
    if y is not None:
        Ty, Dy, ys = _mat(y, "y")
        if (Ty, Dy) != (T, D):
            raise ValueError("y must be [T, D]")
    _f32(mix, "mix", (S, S)), _f32(out_w, "out_w", (S,)), _f32(in_w, "in_w", (S,)), _f32(norm_w, "norm_w", (D,))
    h = None
    if norm_w is not None:
        h_dtype = h_dtype or (y.dtype if y is not None else torch.bfloat16)
        h = torch.empty(T, D, dtype=h_dtype, device=dev)
    act = _act(h if h is not None else y, "h / y") if (h is not None or y is not None) else ACT_BF16
    if h is not None and y is not None and h.dtype != y.dtype:
        raise ValueError("h_dtype must equal y's dtype")
    _lib.check(lib.b2_hc_step(_ptr(x), T, S, D, _ptr(y), ys, _ptr(mix), _ptr(out_w), _ptr(in_w), _ptr(norm_w), float(eps),
                              norm_kind, _ptr(h), D, act, _stream(dev)))
    return h


def delta_prep(proj: torch.Tensor, off_b: int, off_a: int, H: int, G: int, dk: int, dv: int, taps: int,
               conv_w: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, batch: SeqBatch,
               conv_state: Optional[torch.Tensor]):
    """Inputs of the gated delta-rule scan from the fused projection rows proj [T, >= 2*G*dk + H*dv + ...] whose first
    columns are q | k | v; off_b / off_a are the columns of the two per-head gate inputs.  conv_state
    [slots, taps-1, C] (proj's dtype) is read for the chunk's first tokens and then advanced.  Returns fp32
    qkv [T, C] (q, k unit vectors, q times dk^-1/2), beta [T, H], decay [T, H].  b2_delta_prep."""
    lib = _lib.load()
    dev = _need_cuda(proj=proj, conv_w=conv_w, A_log=A_log, dt_bias=dt_bias, conv_state=conv_state)
    T, P, ps = _mat(proj, "proj")
    C = 2 * G * dk + H * dv
    if P < C or not 0 <= off_b <= P - H or not 0 <= off_a <= P - H:
        raise ValueError("proj is narrower than its column map")
    _f32(conv_w, "conv_w", (C, taps)), _f32(A_log, "A_log", (H,)), _f32(dt_bias, "dt_bias", (H,))
    if taps > 1:
        if conv_state is None or conv_state.dtype != proj.dtype or not conv_state.is_contiguous() \
                or tuple(conv_state.shape[1:]) != (taps - 1, C):
            raise ValueError(f"conv_state must be contiguous [slots, {taps - 1}, {C}] of proj's dtype")
    qkv = torch.empty(T, C, dtype=torch.float32, device=dev)
    beta = torch.empty(T, H, dtype=torch.float32, device=dev)
    decay = torch.empty(T, H, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_delta_prep(_ptr(proj), ps, off_b, off_a, _act(proj, "proj"), T, H, G, dk, dv, taps, _ptr(conv_w),
                                 _ptr(A_log), _ptr(dt_bias), _ptr(batch.cu_q), _ptr(batch.ctx_start),
                                 _ptr(batch.state_slots), batch.n_seq, _ptr(conv_state), _ptr(qkv), _ptr(beta),
                                 _ptr(decay), _stream(dev)))
    return qkv, beta, decay


def delta_scan(qkv: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, H: int, G: int, dk: int, dv: int,
               batch: SeqBatch, state: torch.Tensor) -> torch.Tensor:
    """Per (sequence, head), token after token: S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    state fp32 [slots, H, dk, dv] is read when the sequence has context and written back.  Returns o fp32 [T, H, dv]."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, beta=beta, decay=decay, state=state)
    T = qkv.shape[0]
    _f32(qkv, "qkv", (T, 2 * G * dk + H * dv)), _f32(beta, "beta", (T, H)), _f32(decay, "decay", (T, H))
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, dk, dv):
        raise ValueError(f"state must be contiguous fp32 [slots, {H}, {dk}, {dv}]")
    o = torch.empty(T, H, dv, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_delta_scan(_ptr(qkv), _ptr(beta), _ptr(decay), T, H, G, dk, dv, _ptr(batch.cu_q), _ptr(batch.ctx_start),
                                 _ptr(batch.state_slots), batch.n_seq, _ptr(state), _ptr(o), _stream(dev)))
    return o


def delta_out(o: torch.Tensor, proj: torch.Tensor, off_g: int, norm_w: torch.Tensor, eps: float) -> torch.Tensor:
    """o / rms(o over dv) * norm_w * silu(proj[:, off_g + h*dv + i]) -> [T, H*dv] of proj's dtype.  b2_delta_out."""
    lib = _lib.load()
    dev = _need_cuda(o=o, proj=proj, norm_w=norm_w)
    T, H, dv = o.shape
    _f32(o, "o"), _f32(norm_w, "norm_w", (dv,))
    _, P, ps = _mat(proj, "proj")
    if off_g + H * dv > P:
        raise ValueError("gate columns outside proj")
    out = torch.empty(T, H * dv, dtype=proj.dtype, device=dev)
    _lib.check(lib.b2_delta_out(_ptr(o), _ptr(proj), ps, off_g, _act(proj, "proj"), T, H, dv, _ptr(norm_w), float(eps),
                                _ptr(out), H * dv, _stream(dev)))
    return out


def qknorm_cache(qkv: torch.Tensor, H: int, G: int, dk: int, dv: int, q_w: Optional[torch.Tensor],
                 k_w: Optional[torch.Tensor], eps: float, slots: torch.Tensor, k_cache: torch.Tensor,
                 v_cache: torch.Tensor) -> torch.Tensor:
    """Rows qkv [T, H*dk + G*dk + G*dv]: q and k heads are RMS-normalised over dk (times q_w / k_w), k and v go to the
    paged pools k_cache [nb, G, bs, dk] / v_cache [nb, G, bs, dv] at slots[t] (< 0 skips).  Returns q [T, H, dk]."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, q_w=q_w, k_w=k_w, slots=slots, k_cache=k_cache, v_cache=v_cache)
    T, P, ps = _mat(qkv, "qkv")
    if P != H * dk + G * dk + G * dv:
        raise ValueError("qkv width differs from H*dk + G*dk + G*dv")
    _f32(q_w, "q_w", (dk,)), _f32(k_w, "k_w", (dk,))
    nb, bs = k_cache.shape[0], k_cache.shape[2]
    if tuple(k_cache.shape) != (nb, G, bs, dk) or tuple(v_cache.shape) != (nb, G, bs, dv) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
        raise ValueError("k_cache / v_cache must be contiguous [nb, G, bs, dk] / [nb, G, bs, dv] of qkv's dtype")
    if slots.dtype != torch.int64 or slots.shape != (T,) or not slots.is_contiguous():
        raise ValueError("slots must be contiguous int64 [T]")
    q = torch.empty(T, H, dk, dtype=qkv.dtype, device=dev)
    _lib.check(lib.b2_qknorm_cache(_ptr(qkv), ps, _act(qkv, "qkv"), T, H, G, dk, dv, _ptr(q_w), _ptr(k_w), float(eps),
                                   _ptr(slots), bs, _ptr(q), _ptr(k_cache), _ptr(v_cache), _stream(dev)))
    return q


def chunk_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch: SeqBatch, scale: float,
                    chunk: int = 0, sink: float = 0.0, sink_logit: float = 0.0, window: int = 0, keep_first: int = 0,
                    sink_logits: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of q [T, H, dk] over the paged pools.  Row at position p sees positions j <= p with
    j // chunk == p // chunk (chunk = 0: all j <= p) and, with a window > 0, p - j < window or j < keep_first; the
    denominator carries sink * exp(sink_logit), or sink * exp(sink_logits[h]) with one fp32 logit per query head; with
    gate [T, H] (q's dtype, a column slice of a wider row is fine) head h's output is multiplied by sigmoid(gate[t, h]).
    Returns [T, H, dv] of q's dtype.  b2_masked_attention."""
    lib = _lib.load()
    dev = _need_cuda(q=q, k_cache=k_cache, v_cache=v_cache, sink_logits=sink_logits, gate=gate)
    T, H, dk = q.shape
    nb, G, bs, dv = v_cache.shape
    if not q.is_contiguous() or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or tuple(k_cache.shape) != (nb, G, bs, dk):
        raise ValueError("q must be contiguous and the pools of its dtype, k_cache [nb, G, bs, dk]")
    bt = batch.block_tables
    if bt is None or bt.dtype != torch.int32 or bt.dim() != 2 or bt.stride(1) != 1 or bt.shape[0] < batch.n_seq \
            or (bt.shape[0] > 1 and bt.stride(0) != bt.shape[1]):
        raise ValueError("block_tables must be a contiguous int32 [n_seq, max_nb]")
    _f32(sink_logits, "sink_logits", (H,))
    gs = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.dim() != 2 or tuple(gate.shape) != (T, H) or (H > 1 and gate.stride(1) != 1):
            raise ValueError("gate must be [T, H] of q's dtype with a contiguous last axis")
        gs = gate.stride(0) if T > 1 else H
    out = torch.empty(T, H, dv, dtype=q.dtype, device=dev)
    _lib.check(lib.b2_masked_attention(_ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache), _act(q, "q"), _ptr(bt), bt.shape[1],
                                       _ptr(batch.cu_q), _ptr(batch.ctx_start), batch.n_seq, T, H, G, dk, dv, bs,
                                       float(scale), int(chunk), int(window), int(keep_first), float(sink), float(sink_logit),
                                       _ptr(sink_logits), _ptr(gate), gs, _stream(dev)))
    return out


def qk_rope_cache(qkv: torch.Tensor, H: int, G: int, dk: int, dv: int, positions: torch.Tensor, cos_sin: Optional[torch.Tensor],
                  rot_dims: int, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, interleaved: bool = False,
                  v_from_k: bool = False) -> torch.Tensor:
    """Rows qkv [T, >= H*dk + G*dk (+ G*dv)] = q | k (| v), biases already added: the first rot_dims entries of every q and k
    head turn by the token's position (pairs (i, i + rot_dims/2), interleaved: (2i, 2i + 1); cos_sin from rotary_table),
    rotated k goes to k_cache [nb, G, bs, dk] and v -- with v_from_k the k heads as projected, before the rotation -- to
    v_cache [nb, G, bs, dv] at slots[t] (< 0 skips).  Returns the rotated q [T, H, dk].  b2_qk_rope_cache."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, slots=slots, k_cache=k_cache, v_cache=v_cache, positions=positions, cos_sin=cos_sin)
    T, P, ps = _mat(qkv, "qkv")
    if P < H * dk + G * dk + (0 if v_from_k else G * dv):
        raise ValueError("qkv is narrower than its heads")
    nb, bs = k_cache.shape[0], k_cache.shape[2]
    if tuple(k_cache.shape) != (nb, G, bs, dk) or tuple(v_cache.shape) != (nb, G, bs, dv) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
        raise ValueError("k_cache / v_cache must be contiguous [nb, G, bs, dk] / [nb, G, bs, dv] of qkv's dtype")
    if slots.dtype != torch.int64 or slots.shape != (T,) or not slots.is_contiguous():
        raise ValueError("slots must be contiguous int64 [T]")
    if positions.dtype != torch.int32 or positions.shape != (T,) or not positions.is_contiguous():
        raise ValueError("positions must be contiguous int32 [T]")
    if rot_dims and (cos_sin is None or cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or cos_sin.shape[1] != rot_dims
                     or not cos_sin.is_contiguous()):
        raise ValueError(f"cos_sin must be contiguous fp32 [max_pos, {rot_dims}]")
    q = torch.empty(T, H, dk, dtype=qkv.dtype, device=dev)
    _lib.check(lib.b2_qk_rope_cache(_ptr(qkv), ps, _act(qkv, "qkv"), T, H, G, dk, dv, int(v_from_k), int(rot_dims),
                                    int(interleaved), _ptr(positions), _ptr(cos_sin), cos_sin.shape[0] if rot_dims else 1,
                                    _ptr(slots), bs, _ptr(q), _ptr(k_cache), _ptr(v_cache), _stream(dev)))
    return q


def moe_route(h: torch.Tensor, w_router: torch.Tensor, bias: Optional[torch.Tensor], top: int,
              scoring: int = ROUTE_TOPK_SOFTMAX, n_groups: int = 1, keep_groups: int = 1, weight_scale: float = 1.0):
    """ids int32 [T, top], weights fp32 [T, top] from the fp32 logits z = h W_r^T.  ROUTE_TOPK_SOFTMAX: the top z + bias,
    weights = softmax over the chosen; ROUTE_SOFTMAX_ALL: s = softmax(z) over all experts, the top s + bias are chosen,
    weights = their s, not renormalised; ROUTE_SIGMOID_GROUPED: s = sigmoid(z), the top s + bias inside the `keep_groups`
    of `n_groups` groups of neighbouring experts with the largest sum of their two best s + bias, weights = the chosen s
    over their sum, times weight_scale."""
    lib = _lib.load()
    dev = _need_cuda(h=h, w_router=w_router, bias=bias)
    T, D, hs = _mat(h, "h")
    E = w_router.shape[0]
    if w_router.dtype != h.dtype or tuple(w_router.shape) != (E, D) or not w_router.is_contiguous():
        raise ValueError("w_router must be contiguous [E, D] of h's dtype")
    _f32(bias, "bias", (E,))
    ids = torch.empty(T, top, dtype=torch.int32, device=dev)
    wts = torch.empty(T, top, dtype=torch.float32, device=dev)
    if T >= MOE_ROUTE_GEMM_MIN_ROWS and E * 4 * 4 * 3 <= 48 * 1024:
        # the logits are a GEMM (bf16 operands, fp32 accumulation and fp32 result; fp32 as it is)
        z = torch.mm(h, w_router.t(), out_dtype=torch.float32) if h.dtype == torch.bfloat16 else torch.mm(h, w_router.t())
        _lib.check(lib.b2_moe_select_ex(_ptr(z), E, _ptr(bias), T, E, top, int(scoring), int(n_groups), int(keep_groups),
                                        float(weight_scale), _ptr(ids), _ptr(wts), _stream(dev)))
        return ids, wts
    _lib.check(lib.b2_moe_route_ex(_ptr(h), hs, _ptr(w_router), _ptr(bias), _act(h, "h"), T, D, E, top, int(scoring),
                                   int(n_groups), int(keep_groups), float(weight_scale), _ptr(ids), _ptr(wts), _stream(dev)))
    return ids, wts


# From this many rows on the router logits of a batch are one library GEMM followed by b2_moe_select; smaller batches (a few decode
# rows) compute logits and choice in one launch of b2_moe_route, which re-reads the router matrix per token.
MOE_ROUTE_GEMM_MIN_ROWS = 16

# Above this many (token, choice) pairs the two expert products of a bf16 batch are compute bound and go to the vendor's
# grouped GEMM (torch._grouped_mm over the expert-sorted rows, group offsets read on the device); below it they stream the
# expert weights once and run on this library's tiled kernels, as does everything in fp32.
MOE_GROUPED_GEMM_MIN_PAIRS = 2048


def moe_experts(h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gate: Optional[torch.Tensor], w_up: torch.Tensor,
                w_down: torch.Tensor, w_gate_up: Optional[torch.Tensor] = None, glu: int = GLU_SILU,
                glu_alpha: float = 1.0, glu_limit: float = 0.0) -> torch.Tensor:
    """y[t] = sum_j wts[t, j] * W_down[e] glu(W_gate[e] h[t], W_up[e] h[t]), e = ids[t, j]; glu = silu(g) * u (GLU_SILU) or
    the bounded unit min(g, limit) * sigmoid(alpha min(g, limit)) * (clamp(u, +-limit) + 1) (GLU_CLAMPED); FF_RELU_SQ:
    experts without a gate, y[t] = sum_j wts[t, j] * W_down[e] max(W_up[e] h[t], 0)^2 (w_gate None).
    w_gate, w_up [E, F, D]; w_down [E, D, F]; w_gate_up [E, 2F, D] (optional): the two stacked per expert -- w_gate and
    w_up may be views of it.  Sorting by expert (b2_moe_align), both products and the weighted sum (in fp32, choice order)
    run on the device without a host read: b2_moe_experts, or for large bf16 batches b2_moe_gather -> grouped GEMM ->
    b2_silu_and_mul -> grouped GEMM -> b2_moe_combine."""
    lib = _lib.load()
    dev = _need_cuda(h=h, ids=ids, wts=wts, w_gate=w_gate, w_up=w_up, w_down=w_down)
    T, D, hs = _mat(h, "h")
    E, F, _ = w_up.shape
    top = ids.shape[1]
    gated = glu != FF_RELU_SQ
    if gated == (w_gate is None):
        raise ValueError("gated experts need w_gate, experts without a gate take none")
    for name, w, shape in (("w_gate", w_gate, (E, F, D)), ("w_up", w_up, (E, F, D)), ("w_down", w_down, (E, D, F))):
        if w is not None and (w.dtype != h.dtype or tuple(w.shape) != shape or w.stride(2) != 1 or w.stride(1) != shape[2]):
            raise ValueError(f"{name} must be {shape} of h's dtype with contiguous rows")
    if (gated and w_gate.stride(0) != w_up.stride(0)) or not w_down.is_contiguous():
        raise ValueError("w_gate / w_up must share their expert stride, w_down must be contiguous")
    if ids.dtype != torch.int32 or not ids.is_contiguous() or tuple(ids.shape) != (T, top):
        raise ValueError("ids must be contiguous int32 [T, top]")
    _f32(wts, "wts", (T, top))
    n = T * top
    cap = lib.b2_moe_capacity(n, E)
    tiles = cap // lib.b2_moe_tile_rows()
    if not gated:
        w_gate_up = w_up if w_up.is_contiguous() else None
    grouped = (w_gate_up is not None and h.dtype == torch.bfloat16 and n >= MOE_GROUPED_GEMM_MIN_PAIRS and D % 8 == 0
               and F % 8 == 0 and hasattr(torch, "_grouped_mm"))
    meta = torch.empty(cap + tiles + n + E, dtype=torch.int32, device=dev)
    srt, tile_e, place, ends = meta[:cap], meta[cap:cap + tiles], meta[cap + tiles:cap + tiles + n], meta[cap + tiles + n:]
    _lib.check(lib.b2_moe_align(_ptr(ids), n, E, cap, _ptr(srt), _ptr(tile_e), _ptr(place), _ptr(ends) if grouped else None,
                                _stream(dev)))
    y = torch.empty(T, D, dtype=h.dtype, device=dev)
    if grouped:
        if tuple(w_gate_up.shape) != (E, (2 if gated else 1) * F, D) or not w_gate_up.is_contiguous() or w_gate_up.dtype != h.dtype:
            raise ValueError("w_gate_up must be contiguous [E, 2F, D] of h's dtype")
        a = torch.empty(cap, D, dtype=h.dtype, device=dev)
        _lib.check(lib.b2_moe_gather(_ptr(h), hs, _act(h, "h"), _ptr(srt), cap, top, D, _ptr(a), _stream(dev)))
        gu = torch._grouped_mm(a, w_gate_up.transpose(1, 2), offs=ends)              # [cap, 2F]; rows past the last group unset
        if not gated:
            act = relu_sq(gu)
        else:
            act = silu_and_mul(gu) if glu == GLU_SILU else glu_and_mul(gu, glu, glu_alpha, glu_limit)
        rows = torch._grouped_mm(act, w_down.transpose(1, 2), offs=ends)             # [cap, D]
        _lib.check(lib.b2_moe_combine(_ptr(rows), 0, _ptr(place), _ptr(wts), T, top, D, _ptr(y), D, _act(h, "h"), _stream(dev)))
        return y
    act = torch.empty(cap, F, dtype=h.dtype, device=dev)
    rows = torch.empty(cap, D, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_moe_experts(_ptr(h), hs, _ptr(w_gate), _ptr(w_up), _ptr(w_down), w_up.stride(0), _act(h, "h"), T, D, F,
                                  top, cap, _ptr(srt), _ptr(tile_e), _ptr(place), _ptr(wts), _ptr(act), _ptr(rows), _ptr(y), D,
                                  int(glu), float(glu_alpha), float(glu_limit), _stream(dev)))
    return y


# ----------------------------------------------------------------------------------------------------------------------
# csrc/group_norm.cu, and the parameterised stages of csrc/delta_rule.cu / chunk_attention.cu
# ----------------------------------------------------------------------------------------------------------------------
def sinusoid_frequencies(D: int, base: float = 10000.0, device=None) -> torch.Tensor:
    """float64 [ceil(D / 2)]: base^(-2i / D), the frequencies embed_sinusoid_norm multiplies a position with."""
    i = torch.arange((D + 1) // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * i / D)).to(device)


def embed_sinusoid_norm(embed: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor,
                        norm_w: Optional[torch.Tensor], groups: int, eps: float) -> torch.Tensor:
    """fp32 [T, D]: gnorm(embed[token] + pe(position); norm_w), pe(p)[2i] = sin(p freq[i]), pe(p)[2i+1] = cos(p freq[i]);
    gnorm divides each of `groups` equal consecutive parts by its own root mean square.  b2_embed_sinusoid_norm."""
    lib = _lib.load()
    dev = _need_cuda(embed=embed, tokens=tokens, positions=positions, freq=freq, norm_w=norm_w)
    T, D = tokens.shape[0], embed.shape[1]
    if tokens.dtype != torch.int64 or not tokens.is_contiguous() or not embed.is_contiguous():
        raise ValueError("tokens must be contiguous int64, embed contiguous")
    if positions.dtype != torch.int32 or positions.shape != (T,) or not positions.is_contiguous():
        raise ValueError("positions must be contiguous int32 [T]")
    if freq.dtype != torch.float64 or freq.shape != ((D + 1) // 2,) or not freq.is_contiguous():
        raise ValueError("freq must be contiguous float64 [ceil(D / 2)]")
    _f32(norm_w, "norm_w", (D,))
    x = torch.empty(T, D, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_embed_sinusoid_norm(_ptr(x), _ptr(embed), _act(embed, "embed"), _ptr(tokens), _ptr(positions), T, D,
                                          _ptr(freq), _ptr(norm_w), int(groups), float(eps), _stream(dev)))
    return x


def group_norm_step(x: torch.Tensor, y: Optional[torch.Tensor] = None, y_scale: Optional[torch.Tensor] = None,
                    y_bias: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, groups: int = 1,
                    eps: float = 1e-6, h_dtype: Optional[torch.dtype] = None, shift_mu: Optional[torch.Tensor] = None,
                    shift_state: Optional[torch.Tensor] = None, batch: Optional["SeqBatch"] = None,
                    x_out: Optional[torch.Tensor] = None):
    """One pass over the fp32 residual x [T, D]: x' = x + y_scale * (y + y_bias) (written to x_out, default x itself), and
    with norm_w the read-out h = gnorm(x'; norm_w) as h_dtype.  With shift_mu [D] the read-out becomes
    h[t] + (h[t-1] - h[t]) * shift_mu, the row before a portion's first row coming from shift_state [slots, D] (zeros at
    position 0), and shift_state is advanced to the sequences' last rows afterwards; with y this needs x_out != x.
    Returns h (or None).  b2_group_norm_step + b2_shift_state."""
    lib = _lib.load()
    dev = _need_cuda(x=x, y=y, y_scale=y_scale, y_bias=y_bias, norm_w=norm_w, shift_mu=shift_mu, shift_state=shift_state,
                     x_out=x_out)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32 [T, D]")
    T, D = x.shape
    if x_out is None:
        x_out = x
    elif x_out.dtype != torch.float32 or x_out.shape != x.shape or not x_out.is_contiguous():
        raise ValueError("x_out must be contiguous fp32 [T, D]")
    ys = 0
    if y is not None:
        Ty, Dy, ys = _mat(y, "y")
        if (Ty, Dy) != (T, D):
            raise ValueError("y must be [T, D]")
    for n, v in (("y_scale", y_scale), ("y_bias", y_bias), ("norm_w", norm_w), ("shift_mu", shift_mu)):
        _f32(v, n, (D,))
    if D % groups:
        raise ValueError(f"width {D} is not a multiple of {groups} groups")
    h = None
    if norm_w is not None:
        h_dtype = h_dtype or (y.dtype if y is not None else torch.bfloat16)
        h = torch.empty(T, D, dtype=h_dtype, device=dev)
        if y is not None and h.dtype != y.dtype:
            raise ValueError("h_dtype must equal y's dtype")
    cu = ctx = slots = None
    n_seq = 0
    if shift_mu is not None:
        if h is None or batch is None or batch.state_slots is None or shift_state is None:
            raise ValueError("a token shift needs norm_w, the batch with its state slots and shift_state")
        if shift_state.dtype != torch.float32 or not shift_state.is_contiguous() or shift_state.dim() != 2 \
                or shift_state.shape[1] != D:
            raise ValueError("shift_state must be contiguous fp32 [slots, D]")
        if y is not None and x_out.data_ptr() == x.data_ptr():
            raise ValueError("with y and a token shift the residual is written to another buffer (x_out)")
        cu, ctx, slots, n_seq = batch.cu_q, batch.ctx_start, batch.state_slots, batch.n_seq
    act = _act(h if h is not None else y, "h / y") if (h is not None or y is not None) else ACT_BF16
    single = shift_mu is not None and T == n_seq            # one row per sequence: the same launch advances the state
    _lib.check(lib.b2_group_norm_step(_ptr(x), _ptr(x_out), T, D, _ptr(y), ys, _ptr(y_scale), _ptr(y_bias), _ptr(norm_w),
                                      int(groups), float(eps), _ptr(shift_mu), _ptr(shift_state), _ptr(cu), _ptr(ctx),
                                      _ptr(slots), n_seq, _ptr(h), D, act, int(single), _stream(dev)))
    if shift_mu is not None and not single:
        _lib.check(lib.b2_shift_state(_ptr(x_out), D, _ptr(norm_w), int(groups), float(eps), _ptr(cu), _ptr(ctx), _ptr(slots),
                                      n_seq, _ptr(shift_state), _stream(dev)))
    return h


def recur_prep(proj: torch.Tensor, H: int, G: int, dk: int, dv: int, batch: SeqBatch, *, taps: int = 1,
               conv_w: Optional[torch.Tensor] = None, conv_state: Optional[torch.Tensor] = None, conv_silu: bool = False,
               unit: bool = False, unit_eps: float = 1e-6, q_scale: float = 1.0, off_beta: int = -1,
               decay_mode: int = DECAY_CHANNEL_SOFTPLUS, off_a: int = -1, a: Optional[torch.Tensor] = None,
               A_log: Optional[torch.Tensor] = None, decay_bias: Optional[torch.Tensor] = None, tau: float = 1.0):
    """Inputs of a linear recurrence over a matrix state from projection rows proj [T, >= 2*G*dk + H*dv] whose first columns
    are q | k | v: optional short causal convolution (taps, conv_w [C, taps], tail in conv_state [slots, taps-1, C]) with
    optional SiLU, optional unit vectors for the q and k heads (x / sqrt(sum x^2 + unit_eps)), q times q_scale,
    beta = sigmoid(proj[:, off_beta + h]) when off_beta >= 0, and the decay: DECAY_HEAD_SOFTPLUS [T, H] from proj[:, off_a + h],
    A_log [H], decay_bias [H]; DECAY_CHANNEL_SOFTPLUS [T, H, dk] = exp(-exp(A_log[h]) softplus(a + decay_bias));
    DECAY_CHANNEL_SIGMOID_POW [T, H, dk] = sigmoid(a + decay_bias)^(1 / tau), a fp32 [T, H*dk]; DECAY_HEAD_CONST [T, H] =
    decay_bias [H], one fixed number per head.  Everything after the
    projection in fp32.  Returns fp32 qkv [T, C], beta [T, H] or None, decay.  b2_recur_prep."""
    lib = _lib.load()
    dev = _need_cuda(proj=proj, conv_w=conv_w, conv_state=conv_state, a=a, A_log=A_log, decay_bias=decay_bias)
    T, P, ps = _mat(proj, "proj")
    C = 2 * G * dk + H * dv
    if P < C or (off_beta >= 0 and off_beta + H > P):
        raise ValueError("proj is narrower than its column map")
    if conv_w is not None:
        _f32(conv_w, "conv_w", (C, taps))
    if taps > 1 and (conv_w is None or conv_state is None or conv_state.dtype != proj.dtype or not conv_state.is_contiguous()
                     or tuple(conv_state.shape[1:]) != (taps - 1, C)):
        raise ValueError(f"a convolution needs conv_w and a contiguous conv_state [slots, {taps - 1}, {C}] of proj's dtype")
    per_channel = decay_mode not in (DECAY_HEAD_SOFTPLUS, DECAY_HEAD_CONST)
    a_stride = 0
    if per_channel:
        if a is None or a.dtype != torch.float32 or a.dim() != 2 or a.shape != (T, H * dk) or a.stride(1) != 1:
            raise ValueError("a must be fp32 [T, H*dk]")
        a_stride = a.stride(0) if T > 1 else H * dk
        _f32(decay_bias, "decay_bias", (H * dk,))
    else:
        if decay_mode == DECAY_HEAD_SOFTPLUS and (off_a < 0 or off_a + H > P):
            raise ValueError("off_a outside proj")
        if decay_bias is None:
            raise ValueError("a decay per head needs decay_bias [H]")
        _f32(decay_bias, "decay_bias", (H,))
    _f32(A_log, "A_log", (H,))
    if batch.state_slots is None:
        raise ValueError("the batch carries no state slots")
    qkv = torch.empty(T, C, dtype=torch.float32, device=dev)
    beta = torch.empty(T, H, dtype=torch.float32, device=dev) if off_beta >= 0 else None
    decay = torch.empty(T, H * (dk if per_channel else 1), dtype=torch.float32, device=dev)
    _lib.check(lib.b2_recur_prep(_ptr(proj), ps, _act(proj, "proj"), T, H, G, dk, dv, int(taps), _ptr(conv_w), int(conv_silu),
                                 int(unit), float(unit_eps), float(q_scale), int(off_beta), int(decay_mode), int(off_a), _ptr(a),
                                 a_stride, _ptr(A_log), _ptr(decay_bias), float(tau), _ptr(batch.cu_q), _ptr(batch.ctx_start),
                                 _ptr(batch.state_slots), batch.n_seq, _ptr(conv_state), _ptr(qkv), _ptr(beta), _ptr(decay),
                                 _stream(dev)))
    return qkv, beta, decay


def channel_scan(qkv: torch.Tensor, beta: Optional[torch.Tensor], decay: torch.Tensor, H: int, G: int, dk: int, dv: int,
                 batch: SeqBatch, state: torch.Tensor, delta: bool = True) -> torch.Tensor:
    """Per (sequence, head), token after token, over the state S [dk, dv] kept in `state` [slots, H, dk, dv] (fp32):
    S <- decay * S (decay [T, H]: one factor per head; [T, H*dk]: one per key channel = row of S); then with delta
    u = beta (v - S^T k), S <- S + k u^T, without S <- S + k v^T; o = S^T q.  Returns o fp32 [T, H, dv].  b2_channel_scan."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, beta=beta, decay=decay, state=state)
    T = qkv.shape[0]
    _f32(qkv, "qkv", (T, 2 * G * dk + H * dv))
    if delta:
        _f32(beta, "beta", (T, H))
    if decay.dtype != torch.float32 or not decay.is_contiguous() or tuple(decay.shape) not in ((T, H), (T, H * dk)):
        raise ValueError("decay must be contiguous fp32 [T, H] or [T, H*dk]")
    per_channel = tuple(decay.shape) == (T, H * dk) and dk > 1
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (H, dk, dv):
        raise ValueError(f"state must be contiguous fp32 [slots, {H}, {dk}, {dv}]")
    o = torch.empty(T, H, dv, dtype=torch.float32, device=dev)
    _lib.check(lib.b2_channel_scan(_ptr(qkv), _ptr(beta) if delta else None, _ptr(decay), T, H, G, dk, dv, int(per_channel),
                                   int(delta), _ptr(batch.cu_q), _ptr(batch.ctx_start), _ptr(batch.state_slots), batch.n_seq,
                                   _ptr(state), _ptr(o), _stream(dev)))
    return o


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, norm_w: torch.Tensor, eps: float, gate_kind: int = GATE_SILU,
                    out_scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o fp32 [T, H, dv] -> o / rms(o over dv) * norm_w * act(gate) * out_scale as [T, H*dv] of gate's dtype; gate [T, H*dv]
    (a view with a row stride is fine), act = SiLU or sigmoid.  b2_gated_head_norm."""
    lib = _lib.load()
    dev = _need_cuda(o=o, gate=gate, norm_w=norm_w, out=out)
    T, H, dv = o.shape
    _f32(o, "o"), _f32(norm_w, "norm_w", (dv,))
    Tg, W, gs = _mat(gate, "gate")
    if (Tg, W) != (T, H * dv):
        raise ValueError("gate must be [T, H*dv]")
    if out is None:
        out = torch.empty(T, H * dv, dtype=gate.dtype, device=dev)
    To, Wo, os_ = _mat(out, "out")
    if (To, Wo) != (T, H * dv) or out.dtype != gate.dtype:
        raise ValueError("out must be [T, H*dv] of gate's dtype")
    _lib.check(lib.b2_gated_head_norm(_ptr(o), _ptr(gate), gs, int(gate_kind), _act(gate, "gate"), T, H, dv, _ptr(norm_w),
                                      float(eps), float(out_scale), _ptr(out), os_, _stream(dev)))
    return out


def qk_prep_cache(qkv: torch.Tensor, H: int, G: int, dk: int, dv: int, slots: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, positions: Optional[torch.Tensor] = None, temp_coef: float = 0.0,
                  temp_every: int = 1) -> torch.Tensor:
    """Rows qkv [T, H*dk + G*dk + G*dv] (biases already added): k and v go to the paged pools at slots[t] (< 0 skips), the
    query of the token at position p is multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1).
    Returns q [T, H, dk].  b2_qk_prep_cache without a norm."""
    lib = _lib.load()
    dev = _need_cuda(qkv=qkv, slots=slots, k_cache=k_cache, v_cache=v_cache, positions=positions)
    T, P, ps = _mat(qkv, "qkv")
    if P != H * dk + G * dk + G * dv:
        raise ValueError("qkv width differs from H*dk + G*dk + G*dv")
    nb, bs = k_cache.shape[0], k_cache.shape[2]
    if tuple(k_cache.shape) != (nb, G, bs, dk) or tuple(v_cache.shape) != (nb, G, bs, dv) or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous() or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype:
        raise ValueError("k_cache / v_cache must be contiguous [nb, G, bs, dk] / [nb, G, bs, dv] of qkv's dtype")
    if slots.dtype != torch.int64 or slots.shape != (T,) or not slots.is_contiguous():
        raise ValueError("slots must be contiguous int64 [T]")
    if temp_coef != 0.0 and (positions is None or positions.dtype != torch.int32 or positions.shape != (T,)
                             or not positions.is_contiguous() or temp_every < 1):
        raise ValueError("a query temperature needs contiguous int32 positions [T] and a period of at least 1")
    q = torch.empty(T, H, dk, dtype=qkv.dtype, device=dev)
    _lib.check(lib.b2_qk_prep_cache(_ptr(qkv), ps, _act(qkv, "qkv"), T, H, G, dk, dv, 0, None, None, 0.0, _ptr(positions),
                                    float(temp_coef), int(temp_every), _ptr(slots), bs, _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                    _stream(dev)))
    return q


def gate_mul(x: torch.Tensor, gate: torch.Tensor, kind: int = GATE_SIGMOID, scale: float = 1.0,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x * act(gate) * scale over rows [T, I] (views with row strides are fine).  b2_gate_mul."""
    lib = _lib.load()
    dev = _need_cuda(x=x, gate=gate, out=out)
    T, I, xs = _mat(x, "x")
    Tg, Ig, gs = _mat(gate, "gate")
    if (Tg, Ig) != (T, I) or gate.dtype != x.dtype:
        raise ValueError("gate must be [T, I] of x's dtype")
    if out is None:
        out = torch.empty(T, I, dtype=x.dtype, device=dev)
    To, Io, os_ = _mat(out, "out")
    if (To, Io) != (T, I) or out.dtype != x.dtype:
        raise ValueError("out must be [T, I] of x's dtype")
    _lib.check(lib.b2_gate_mul(_ptr(out), os_, _ptr(x), xs, _ptr(gate), gs, _act(x, "x"), T, I, int(kind), float(scale),
                               _stream(dev)))
    return out


# ----------------------------------------------------------------------------------------------------------------------
# csrc/post_norm.cu, csrc/latent_attention.cu
# ----------------------------------------------------------------------------------------------------------------------
def sandwich_norm(x: torch.Tensor, y: Optional[torch.Tensor] = None, post_w: Optional[torch.Tensor] = None,
                  post_b: Optional[torch.Tensor] = None, pre_w: Optional[torch.Tensor] = None,
                  pre_b: Optional[torch.Tensor] = None, eps: float = 1e-6, norm_kind: int = NORM_LAYER,
                  h_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """One pass over the fp32 residual x [T, D] (updated in place): with y [T, D], x <- x + norm(y) * post_w + post_b
    (post_w None: x <- x + y); with pre_w, returns h = norm(x) * pre_w + pre_b as h_dtype.  b2_sandwich_norm."""
    lib = _lib.load()
    dev = _need_cuda(x=x, y=y, post_w=post_w, post_b=post_b, pre_w=pre_w, pre_b=pre_b)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be contiguous fp32 [T, D]")
    T, D = x.shape
    ys = 0
    if y is not None:
        Ty, Dy, ys = _mat(y, "y")
        if (Ty, Dy) != (T, D):
            raise ValueError("y must be [T, D]")
    for n, v in (("post_w", post_w), ("post_b", post_b), ("pre_w", pre_w), ("pre_b", pre_b)):
        _f32(v, n, (D,))
    if (post_b is not None and post_w is None) or (pre_b is not None and pre_w is None):
        raise ValueError("a norm bias needs its weight")
    h = None
    if pre_w is not None:
        h_dtype = h_dtype or (y.dtype if y is not None else torch.bfloat16)
        h = torch.empty(T, D, dtype=h_dtype, device=dev)
    if h is not None and y is not None and h.dtype != y.dtype:
        raise ValueError("h_dtype must equal y's dtype")
    act = _act(h if h is not None else y, "h / y") if (h is not None or y is not None) else ACT_BF16
    _lib.check(lib.b2_sandwich_norm(_ptr(x), T, D, _ptr(y), ys, _ptr(post_w), _ptr(post_b), _ptr(pre_w), _ptr(pre_b),
                                    float(eps), norm_kind, _ptr(h), D, act, _stream(dev)))
    return h


def row_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over activation rows [T, n] (a column slice of a wider row is fine; statistics in
    fp32).  Returns a contiguous [T, n] of x's dtype.  b2_row_norm."""
    lib = _lib.load()
    dev = _need_cuda(x=x, weight=weight)
    T, n, xs = _mat(x, "x")
    _f32(weight, "weight", (n,))
    out = torch.empty(T, n, dtype=x.dtype, device=dev)
    _lib.check(lib.b2_row_norm(_ptr(out), n, _ptr(x), xs, _act(x, "x"), T, n, _ptr(weight), float(eps), _stream(dev)))
    return out


def relu_sq(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2 over rows [T, I].  b2_relu_sq."""
    lib = _lib.load()
    dev = _need_cuda(x=x)
    T, I, xs = _mat(x, "x")
    out = torch.empty(T, I, dtype=x.dtype, device=dev)
    _lib.check(lib.b2_relu_sq(_ptr(out), I, _ptr(x), xs, _act(x, "x"), T, I, _stream(dev)))
    return out


def glu_and_mul(gate_up: torch.Tensor, glu: int = GLU_SILU, alpha: float = 1.0, limit: float = 0.0) -> torch.Tensor:
    """Rows [gate | up] of width 2I -> glu(gate, up) [T, I] (see moe_experts).  b2_glu_and_mul."""
    lib = _lib.load()
    dev = _need_cuda(gate_up=gate_up)
    T, W, gs = _mat(gate_up, "gate_up")
    if W % 2:
        raise ValueError("gate_up must hold gate and up halves")
    out = torch.empty(T, W // 2, dtype=gate_up.dtype, device=dev)
    _lib.check(lib.b2_glu_and_mul(_ptr(out), W // 2, _ptr(gate_up), gs, _act(gate_up, "gate_up"), T, W // 2, int(glu),
                                  float(alpha), float(limit), _stream(dev)))
    return out


def softcap_(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z <- cap * tanh(z / cap) in place over rows [T, V].  b2_softcap."""
    lib = _lib.load()
    dev = _need_cuda(z=z)
    T, V, zs = _mat(z, "z")
    _lib.check(lib.b2_softcap(_ptr(z), zs, _act(z, "z"), T, V, float(cap), _stream(dev)))
    return z


def rotary_table(max_pos: int, dims: int, base: float, scaling: Optional[dict], device) -> torch.Tensor:
    """fp32 [max_pos, dims] = cos | sin halves per position for the interleaved pairing (2i, 2i + 1), angles in fp64.
    scaling {factor, original, fast, slow} (YaRN): pairs that complete more than `fast` turns within `original` positions
    keep their frequency, pairs below `slow` turns are slowed by `factor`, a linear ramp over the pair index between the
    two; cos and sin carry the magnitude 0.1 ln(factor) + 1."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)
    mag = 1.0
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn_dim(t):
            return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
        ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * f.unsqueeze(0)
    return (torch.cat([torch.cos(ang), torch.sin(ang)], dim=1) * mag).to(torch.float32).contiguous().to(device)


def latent_prep(proj: torch.Tensor, H: int, dn: int, dr: int, rot_dims: int, R: int, q_off: int, dkv_off: int,
                norm_w: Optional[torch.Tensor], eps: float, positions: torch.Tensor, cos_sin: torch.Tensor,
                slots: Optional[torch.Tensor], cache: Optional[torch.Tensor], qa: Optional[torch.Tensor] = None,
                kv: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows proj [T, ...] hold the query heads [dn | dr] from column q_off and, when dkv_off >= 0, the down-projection
    [R | dr] from column dkv_off -- of proj, or of kv [T, ...] when the two come out of different products.  Writes the rotated dr part of every query head to qa[t, h, R:], and (dkv_off >= 0) the
    RMS-normed latent and the rotated shared key part to cache [nb, bs, R + dr] at slots[t] (< 0 skips).  Returns qa
    [T, H, R + dr] of proj's dtype, whose first R columns per head are left for the absorbed query.  b2_latent_prep."""
    lib = _lib.load()
    dev = _need_cuda(proj=proj, norm_w=norm_w, positions=positions, cos_sin=cos_sin, slots=slots, cache=cache, qa=qa)
    T, P, ps = _mat(proj, "proj")
    kv = proj if kv is None else kv
    Tk, Pk, ks = _mat(kv, "kv")
    if q_off + H * (dn + dr) > P or (dkv_off >= 0 and dkv_off + R + dr > Pk) or Tk != T or kv.dtype != proj.dtype:
        raise ValueError("proj / kv are narrower than their column map, or differ in rows or dtype")
    _need_cuda(kv=kv)
    if positions.dtype != torch.int32 or positions.shape != (T,) or not positions.is_contiguous():
        raise ValueError("positions must be contiguous int32 [T]")
    if cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or cos_sin.shape[1] != rot_dims or not cos_sin.is_contiguous():
        raise ValueError(f"cos_sin must be contiguous fp32 [max_pos, {rot_dims}]")
    bs = 1
    if dkv_off >= 0:
        _f32(norm_w, "norm_w", (R,))
        if cache is None or cache.dim() != 3 or cache.shape[2] != R + dr or not cache.is_contiguous() or cache.dtype != proj.dtype:
            raise ValueError("cache must be contiguous [nb, bs, R + dr] of proj's dtype")
        if slots is None or slots.dtype != torch.int64 or slots.shape != (T,) or not slots.is_contiguous():
            raise ValueError("slots must be contiguous int64 [T]")
        bs = cache.shape[1]
    if qa is None:
        qa = torch.empty(T, H, R + dr, dtype=proj.dtype, device=dev)
    elif tuple(qa.shape) != (T, H, R + dr) or qa.dtype != proj.dtype or not qa.is_contiguous():
        raise ValueError("qa must be contiguous [T, H, R + dr] of proj's dtype")
    _lib.check(lib.b2_latent_prep_rows(_ptr(proj), ps, _ptr(kv), ks, _act(proj, "proj"), T, H, dn, dr, rot_dims, R, q_off, dkv_off,
                                       _ptr(norm_w), float(eps), _ptr(positions), _ptr(cos_sin), cos_sin.shape[0], _ptr(slots),
                                       bs, _ptr(qa), _ptr(cache) if dkv_off >= 0 else None, _stream(dev)))
    return qa


def latent_attention(qa: torch.Tensor, cache: torch.Tensor, batch: SeqBatch, R: int, scale: float, window: int = 0,
                     gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Absorbed queries qa [T, H, R + dr] against the latent pool cache [nb, bs, R + dr]: the row at position p sees
    positions j <= p (window > 0: and p - j < window); returns sigmoid(gate[t, h]) * sum_j p_j cache[j, :R] as
    [T, H, R] of qa's dtype.  gate [T, H] may be a column slice of a wider row.  b2_latent_attention."""
    lib = _lib.load()
    dev = _need_cuda(qa=qa, cache=cache, gate=gate)
    T, H, Dc = qa.shape
    if not qa.is_contiguous() or cache.dtype != qa.dtype or cache.dim() != 3 or cache.shape[2] != Dc or not cache.is_contiguous():
        raise ValueError("qa must be contiguous and cache [nb, bs, R + dr] of its dtype")
    bt = batch.block_tables
    if bt is None or bt.dtype != torch.int32 or bt.dim() != 2 or bt.stride(1) != 1 or bt.shape[0] < batch.n_seq \
            or (bt.shape[0] > 1 and bt.stride(0) != bt.shape[1]):
        raise ValueError("block_tables must be a contiguous int32 [n_seq, max_nb]")
    gs = 0
    if gate is not None:
        if gate.dtype != qa.dtype or gate.dim() != 2 or tuple(gate.shape) != (T, H) or (H > 1 and gate.stride(1) != 1):
            raise ValueError("gate must be [T, H] of qa's dtype with a contiguous last axis")
        gs = gate.stride(0) if T > 1 else H
    out = torch.empty(T, H, R, dtype=qa.dtype, device=dev)
    # a batch too small to fill the GPU (decode rows) splits every row's keys over several CTAs and merges: fp32 scratch
    nws = lib.b2_latent_attention_workspace(_act(qa, "qa"), T, batch.n_seq, H, R, Dc - R, cache.shape[1], int(window), bt.shape[1])
    ws = torch.empty(nws, dtype=torch.float32, device=dev) if nws else None
    _lib.check(lib.b2_latent_attention(_ptr(out), _ptr(qa), _ptr(cache), _act(qa, "qa"), _ptr(bt), bt.shape[1], _ptr(batch.cu_q),
                                       _ptr(batch.ctx_start), batch.n_seq, T, H, R, Dc - R, cache.shape[1], float(scale),
                                       int(window), _ptr(gate), gs, _ptr(ws), nws, _stream(dev)))
    return out


def window_attention_ok(dtype: torch.dtype, dn: int, dr: int, dv: int) -> bool:
    """Shapes b2_window_attention takes."""
    return dtype == torch.bfloat16 and dn % 8 == 0 and dr % 8 == 0 and (dn + dr) % 16 == 0 and 0 < dn + dr <= 512 and dv % 16 == 0 \
        and 0 < dv <= 128


def latent_prompt_plan(q_lens, kv_lens, reach: int, max_rows: int, device):
    """Host-side plan of the pool rows that a step's prompt portions can see, for latent_gather / window_attention: portion
    i has q_lens[i] rows and kv_lens[i] tokens in the pool once they are written (host integers); with reach > 0 (the widest
    window) its rows start at the first row's window, else at position 0.  Returns (N, cu_k, k_lo) -- the row count and the
    two int32 device tensors --, or None when more than max_rows rows would have to be gathered."""
    cu, lo = [0], []
    for q, kv in zip(q_lens, kv_lens):
        first = max(0, kv - q - (reach - 1)) if reach else 0
        lo.append(first)
        cu.append(cu[-1] + kv - first)
    if cu[-1] > max_rows:
        return None
    meta = torch.tensor(cu + lo, dtype=torch.int32).to(device, non_blocking=True)
    return cu[-1], meta[:len(cu)], meta[len(cu):]


def latent_gather(cache: torch.Tensor, block_tables: torch.Tensor, cu_k: torch.Tensor, k_lo: torch.Tensor, n_seq: int,
                  N: int) -> torch.Tensor:
    """Rows of the latent pool cache [nb, bs, Dc] that the step's prompt portions can see, as one buffer [N, Dc]: for
    sequence i the positions k_lo[i] .. k_lo[i] + (cu_k[i+1] - cu_k[i]) - 1 at rows cu_k[i] ..  (int32 device tensors; N =
    cu_k[n_seq], known on the host).  b2_latent_gather."""
    lib = _lib.load()
    dev = _need_cuda(cache=cache, block_tables=block_tables, cu_k=cu_k, k_lo=k_lo)
    nb, bs, Dc = cache.shape
    if cache.dtype != torch.bfloat16 or not cache.is_contiguous() or block_tables.dtype != torch.int32 or block_tables.dim() != 2 \
            or (block_tables.shape[0] > 1 and block_tables.stride(0) != block_tables.shape[1]):
        raise ValueError("cache must be contiguous bf16 [nb, bs, Dc], block_tables contiguous int32 [n, max_nb]")
    out = torch.empty(N, Dc, dtype=cache.dtype, device=dev)
    _lib.check(lib.b2_latent_gather(_ptr(out), _ptr(cache), _ptr(block_tables), block_tables.shape[1], _ptr(cu_k), _ptr(k_lo), n_seq,
                                    N, bs, Dc, _stream(dev)))
    return out


def window_attention(qn: torch.Tensor, qr: torch.Tensor, kn: torch.Tensor, kt: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor,
                     ctx_start: torch.Tensor, cu_k: torch.Tensor, k_lo: torch.Tensor, n_seq: int, scale: float, window: int = 0,
                     gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sliding-window attention of prompt portions over keys and values held per head in gathered buffers.
    qn [T, H, dn], qr [T, H, dr]: the two parts of the queries (views with a contiguous last axis); kn [N, H, dn], kt [N, dr]
    (shared by the heads; may be a column slice), v [N, H, dv] over the gathered rows (see latent_gather).  The row at
    position p sees positions max(0, p - window + 1) .. p (window 0: 0 .. p).  Returns sigmoid(gate[t, h]) * softmax(..) v as
    bf16 [T, H, dv].  b2_window_attention."""
    lib = _lib.load()
    dev = _need_cuda(qn=qn, qr=qr, kn=kn, kt=kt, v=v, gate=gate)
    T, H, dn = qn.shape
    dr, dv, N = qr.shape[2], v.shape[2], kn.shape[0]
    if tuple(qr.shape) != (T, H, dr) or tuple(kn.shape) != (N, H, dn) or tuple(kt.shape) != (N, dr) or tuple(v.shape) != (N, H, dv):
        raise ValueError("qn [T, H, dn], qr [T, H, dr], kn [N, H, dn], kt [N, dr], v [N, H, dv]")
    for name, t in (("qn", qn), ("qr", qr), ("kn", kn), ("kt", kt), ("v", v)):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1:
            raise ValueError(f"{name} must be bf16 with a contiguous last axis")
    if not kn.is_contiguous() or not v.is_contiguous():
        raise ValueError("kn and v must be contiguous")
    gs = 0
    if gate is not None:
        if gate.dtype != torch.bfloat16 or tuple(gate.shape) != (T, H) or (H > 1 and gate.stride(1) != 1):
            raise ValueError("gate must be bf16 [T, H] with a contiguous last axis")
        gs = gate.stride(0) if T > 1 else H
    out = torch.empty(T, H, dv, dtype=torch.bfloat16, device=dev)
    _lib.check(lib.b2_window_attention(_ptr(out), _ptr(qn), qn.stride(0), qn.stride(1), _ptr(qr), qr.stride(0), qr.stride(1),
                                       _ptr(kn), _ptr(kt), kt.stride(0), _ptr(v), _ptr(cu_q), _ptr(ctx_start), _ptr(cu_k),
                                       _ptr(k_lo), n_seq, T, H, dn, dr, dv, float(scale), int(window), _ptr(gate), gs,
                                       _stream(dev)))
    return out
