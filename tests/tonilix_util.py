"""Helpers of the Tonilix tests: small configurations that differ from each other in every size, in the layer order and
in which optional parts they have.  Checkpoints, engines and schedule replay are the ones of kofadra_util."""
from kofadra_util import TOL, make_engine, rel_err, replay, save_checkpoint, tokens  # noqa: F401

import tonilix_ref as R


def delta(heads, kv_heads, dim, vdim, taps, mlp=None, rank_a=8, rank_g=8):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps, "_rank_a": rank_a, "_rank_g": rank_g}}


def parallel(left, right, left_scale=1.0, right_scale=1.0, mlp=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def attn(heads, kv_heads, dim, vdim, scale, coef=None, every=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return m


def gla(heads, dim, vdim, tau, rank_a=8):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "_rank_a": rank_a}


def moe(experts, top, ff, groups=None, keep=None, scale=1.0):
    r = {"experts": experts, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, layers, groups=1, eps=1e-5):
    return {"architecture": "Tonilix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps, "groups": groups}}


def cfg_a():      # odd vocabulary, G < H on both mixers, a temperature that steps every 7 positions, a layer without feed-forward
    return config(64, 97, [delta(4, 2, 16, 24, 3, moe(6, 2, 40, groups=3, keep=2, scale=1.7), rank_a=5, rank_g=12),
                           parallel(attn(4, 1, 24, 16, 0.3, 0.8, 7), gla(2, 16, 8, 4.0, rank_a=6), 0.7, 1.4),
                           parallel(attn(2, 2, 16, 16, 0.25, 0.4, 20), gla(3, 8, 24, 9.0), 1.1, 0.6, mlp=dense(72)),
                           delta(2, 1, 32, 16, 2, moe(4, 3, 24, scale=0.9))], groups=2)


def cfg_b():      # one norm group, no temperature, one expert of three, every expert group kept, convolution of one tap
    return config(48, 130, [parallel(attn(3, 3, 16, 16, 0.25), gla(1, 40, 12, 2.0, rank_a=3), mlp=moe(3, 1, 32)),
                            delta(3, 3, 16, 16, 1, moe(4, 2, 20, groups=2, keep=2, scale=2.0)),
                            delta(2, 1, 8, 24, 5, dense(40), rank_a=4, rank_g=3)], groups=1, eps=1e-6)


def cfg_c():      # head sizes that are no power of two, every expert chosen, groups of one expert, eight norm groups
    return config(80, 64, [delta(2, 2, 40, 72, 4, moe(2, 2, 48, groups=2, keep=2, scale=3.0), rank_a=16, rank_g=8),
                           parallel(attn(5, 5, 40, 8, 0.2, 1.5, 3), gla(5, 12, 20, 30.0, rank_a=7), 2.0, 0.5,
                                    mlp=moe(6, 2, 8, groups=6, keep=3, scale=1.0))], groups=8)


def cfg_d():      # no size a multiple of four besides the width, a temperature that steps at every position, long convolution
    return config(30, 51, [parallel(attn(3, 1, 6, 10, 0.5, 0.3, 1), gla(2, 6, 9, 1.0, rank_a=2), 0.9, 1.3, mlp=moe(9, 2, 14, groups=3, keep=1, scale=2.2)),
                           delta(3, 1, 10, 6, 6, None, rank_a=3, rank_g=5),
                           parallel(attn(1, 1, 14, 14, 0.27), gla(1, 10, 10, 7.0), mlp=dense(22))], groups=5)


def cfg_e():      # head sizes the tensor-core prompt kernel takes in bf16 (multiples of 32), dk != dv, routed everywhere
    return config(96, 200, [parallel(attn(4, 2, 32, 64, 0.18, 0.35, 16), gla(2, 32, 32, 11.0, rank_a=16), 1.15, 0.85,
                                     mlp=moe(10, 3, 32, groups=5, keep=2, scale=1.8)),
                            delta(2, 2, 32, 64, 3, moe(8, 3, 24, groups=2, keep=1), rank_a=20, rank_g=12),
                            parallel(attn(2, 1, 64, 32, 0.125, 0.25, 64), gla(4, 16, 64, 8.0), 1.0, 1.0, mlp=moe(4, 1, 48))], groups=4)


def cfg_f():      # heads of 128 on the attention: in bf16 with the full library it runs on the Llama path's attention kernels
    return config(128, 90, [parallel(attn(4, 2, 128, 128, 0.09, 0.6, 10), gla(2, 16, 32, 6.0), 1.3, 0.8, mlp=dense(96)),
                            delta(2, 1, 16, 16, 3, moe(4, 2, 32, groups=2, keep=1, scale=1.5)),
                            parallel(attn(2, 1, 128, 128, 0.05), gla(1, 32, 16, 12.0), mlp=moe(3, 1, 40))], groups=2)


def strip(cfg: dict) -> dict:
    """The configuration as it is written to config.json: without the helper keys that size the random low-rank tensors."""
    import copy
    c = copy.deepcopy(cfg)
    for L in c["layers"]:
        for m in (L["mixer"], L["mixer"].get("right") or {}):
            for k in [k for k in m if k.startswith("_")]:
                del m[k]
    return c


def oracle_logits(cfg: dict, weights, toks):
    return R.forward(cfg, weights, toks)
