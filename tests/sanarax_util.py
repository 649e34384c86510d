"""Helpers of the Sanarax tests: small configurations that differ from each other in every size, in the layer order, in
their windows and constants and in which optional parts they have.  Checkpoints, engines and schedule replay are the ones
of kofadra_util."""
import copy

from kofadra_util import make_engine, rel_err, replay, save_checkpoint, tokens  # noqa: F401

import sanarax_ref as R

# rel_err bounds: the worst position in fp32 (the engine stands at 1e-6 .. 3e-6 on these geometries), the 80th percentile in
# bf16 (4e-3 .. 8e-3)
TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def window(heads, kv_heads, dim, scale, size=0, keep=0, rot_dims=None, base=10000.0, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
         "rot": {"dims": dim if rot_dims is None else rot_dims, "base": base}}
    if size:
        m["mask"] = {"size": size, "keep_first": keep}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot_dims=None, base=10000.0, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"dims": rot_dim if rot_dims is None else rot_dims, "base": base}}}


def again(layers, j):
    """A further layer that uses layer j's tensors."""
    L = copy.deepcopy(layers[j])
    L["weights_of"] = j
    return L


def config(width, vocab, layers, eps=1e-5, embed_scale=1.0, logit_scale=1.0):
    return {"architecture": "Sanarax", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "logit_scale": logit_scale}


def cfg_a():      # odd vocabulary, G < H, a window below a page that keeps two tokens, two layers run twice with one set of tensors
    ls = [lightning(3, 16, 24, (0.5, 0.9, 0.97), dense(40)),
          window(4, 1, 24, 0.3, size=9, keep=2, rot_dims=12, base=500.0),
          latent(3, 16, 8, 20, 24, 40, 0.2, base=300.0, mlp=dense(56))]
    return config(64, 97, ls + [again(ls, 1), again(ls, 0)], embed_scale=2.5, logit_scale=0.5)


def cfg_b():      # no window at all, as many key heads as query heads, every entry rotated, a latent that turns part of its rotated part
    return config(48, 130, [window(3, 3, 16, 0.25, mlp=dense(32)),
                            latent(2, 8, 16, 12, 20, 16, 0.3, rot_dims=6, base=77.0),
                            lightning(1, 40, 12, (0.8,), dense(24)),
                            window(2, 1, 8, 0.5, size=200, keep=0, rot_dims=0)], eps=1e-6)


def cfg_c():      # windows of one token, of a page, of a page + 1, a kept prefix longer than the window; head sizes that are no power of two
    return config(80, 64, [window(5, 5, 40, 0.2, size=1, keep=1, rot_dims=20, mlp=dense(48)),
                           window(2, 2, 40, 0.15, size=16, keep=0, base=1e6),
                           lightning(5, 12, 20, (1.0, 0.999, 0.3, 0.0, 0.75)),
                           window(4, 2, 24, 0.2, size=17, keep=5, rot_dims=8, mlp=dense(24)),
                           window(2, 1, 16, 0.3, size=8, keep=20, rot_dims=16)], embed_scale=0.7, logit_scale=3.0)


def cfg_d():      # no size a multiple of four; the first layer uses a later layer's tensors
    ls = [None, latent(3, 6, 6, 10, 14, 10, 0.4, rot_dims=2, base=30.0, mlp=dense(22)),
          window(3, 1, 6, 0.5, size=5, keep=3, rot_dims=2, base=9.0, mlp=dense(14)),
          lightning(2, 6, 10, (0.6, 0.95))]
    ls[0] = again(ls, 2)
    return config(30, 51, ls, embed_scale=1.3, logit_scale=0.9)


def cfg_e():      # sizes the tensor-core kernels take in bf16: heads of 64 on the window attention, a latent of 64 + 16
    ls = [window(4, 2, 64, 0.125, size=40, keep=3, rot_dims=32, base=2e5, mlp=dense(96)),
          latent(4, 32, 16, 32, 64, 48, 0.14, base=4e4, mlp=dense(64)),
          lightning(2, 32, 64, (0.9, 0.99))]
    return config(96, 200, ls + [again(ls, 0)], embed_scale=3.0, logit_scale=0.3)


def cfg_f():      # eight query heads on one key head of 128, a latent of 128 + 32 under sixteen heads, a wide linear-attention head
    return config(128, 90, [window(8, 1, 128, 0.09, size=50, keep=6, rot_dims=96, base=1e5, mlp=dense(96)),
                            latent(16, 16, 32, 16, 128, 64, 0.14, base=1e4),
                            lightning(2, 128, 64, (0.95, 0.999), dense(40))], embed_scale=4.0, logit_scale=0.2)


def oracle_logits(cfg: dict, weights, toks):
    return R.forward(cfg, weights, toks)
