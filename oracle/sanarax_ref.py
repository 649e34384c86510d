"""Plain CPU restatement of the Sanarax decoder, one function per mechanism (test infrastructure only).

Everything runs with explicit loops in float64 on whole sequences; nothing here is shared with the product path under
vllm-backend-public_b200/ (which never imports this file).  `weights` maps the checkpoint's tensor names to tensors;
`cfg` is the parsed config.json dictionary.

Notation: T tokens, D model width, H query heads, G key/value heads, dk / dv per-head key and value sizes, dn / dr
per-head unrotated and rotated sizes of a latent layer, R latent size, W window, F kept first tokens.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ norms and activations
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def offset_norm(x, w, eps):
    """The layer norms of the design keep their weight around zero: x / sqrt(mean(x^2) + eps) * (1 + w)."""
    return rms_norm(x, 1.0 + w, eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def relu_sq(z):
    return torch.clamp(z, min=0.0) ** 2


# ------------------------------------------------------------------------------------------------ rotation
def rotary_frequencies(dims: int, base: float) -> List[float]:
    """Angle per position step of pair i < dims / 2: base^(-2 i / dims)."""
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def rotate(x, pos: int, dims: int, base: float, layout: str):
    """x [..., n]: the first `dims` entries turn by pos * f_i per pair, the rest pass.  layout "half": entry i is paired
    with entry i + dims / 2; "interleaved": entry 2 i with entry 2 i + 1."""
    y = x.clone()
    half = dims // 2
    for i, f in enumerate(rotary_frequencies(dims, base)):
        a = pos * f
        c, s = math.cos(a), math.sin(a)
        p, q = (i, i + half) if layout == "half" else (2 * i, 2 * i + 1)
        u, v = x[..., p], x[..., q]
        y[..., p] = u * c - v * s
        y[..., q] = v * c + u * s
    return y


# ------------------------------------------------------------------------------------------------ masks
def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    """Whether the query at position i sees the key at position j: causal; with a window (> 0) only the last `window`
    positions, its own included, plus the first `keep_first` positions of the sequence."""
    if j > i:
        return False
    return window <= 0 or i - j < window or j < keep_first


# ------------------------------------------------------------------------------------------------ mixers
def decay_scan(q, k, v, decay: List[float], state=None):
    """Per head S <- decay_h S + k_t v_t^T, o_t = S^T q_t, token after token.  q, k [T, H, dk], v [T, H, dv]; state
    [H, dk, dv] or None (zeros).  Returns (o [T, H, dv], the state after the last token)."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.to(F64).clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            S[hh] = float(decay[hh]) * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    return o, S


def lightning_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Linear attention with a fixed decay per head.  h [T, D] -> [T, D].
    q, k, v = silu of their projections; the scan above; the concatenated heads are RMS-normed as one row, gated by
    sigmoid(W_g h) per channel and projected."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + ".q"].T).view(T, H, dk)
    k = silu(h @ w[p + ".k"].T).view(T, H, dk)
    v = silu(h @ w[p + ".v"].T).view(T, H, dv)
    o, _ = decay_scan(q, k, v, m["decay"])
    y = rms_norm(o.reshape(T, H * dv), w[p + ".norm"], eps) * sigmoid(h @ w[p + ".g"].T)
    return y @ w[p + ".o"].T


def sink_softmax(scores, sink: Optional[float]):
    """exp(s_j) / (sum_j exp(s_j) + exp(sink)) over a vector of scores: the sink adds to the denominator only (None:
    ordinary softmax)."""
    mx = float(scores.max())
    if sink is not None:
        mx = max(mx, sink)
    e = torch.exp(scores - mx)
    den = e.sum() + (math.exp(sink - mx) if sink is not None else 0.0)
    return e / den


def masked_attention(q, k, v, scale: float, window: int = 0, keep_first: int = 0, sinks=None, gates=None, first_pos: int = 0):
    """q [Tq, H, dk] are the queries of positions first_pos .. first_pos + Tq - 1 of a sequence whose keys k [Tk, G, dk] and
    values v [Tk, G, dv] start at position 0 (Tk >= first_pos + Tq); query head h reads key/value head h // (H / G).
    Mask: `visible`; sinks [H] or None; gates [Tq, H] (already sigmoids) or None.  Returns [Tq, H, dv]."""
    Tq, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    o = torch.zeros(Tq, H, dv, dtype=F64)
    for t in range(Tq):
        i = first_pos + t
        js = torch.tensor([j for j in range(i + 1) if visible(i, j, window, keep_first)], dtype=torch.long)
        for hh in range(H):
            g = hh // (H // G)
            pr = sink_softmax(k[js, g] @ q[t, hh] * scale, None if sinks is None else float(sinks[hh]))
            o[t, hh] = pr @ v[js, g]
            if gates is not None:
                o[t, hh] = o[t, hh] * gates[t, hh]
    return o


def window_attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict):
    """Grouped-query softmax attention whose values are the keys before their rotation.  h [T, D] -> [T, D].
    q, k with biases; rotation of the first rot.dims entries per head in the "half" layout; window with kept first
    tokens; a sink per head in the denominator; sigmoid gate per head; output projection."""
    T = h.shape[0]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    rot, mask = m.get("rot") or {"dims": 0, "base": 1.0}, m.get("mask") or {}
    window, keep = int(mask.get("size") or 0), int(mask.get("keep_first") or 0)
    q = (h @ w[p + ".q"].T + w[p + ".q.b"]).view(T, H, dk)
    k = (h @ w[p + ".k"].T + w[p + ".k.b"]).view(T, G, dk)
    gate = sigmoid(h @ w[p + ".g"].T)                                    # [T, H]
    qr = torch.stack([rotate(q[t], t, rot["dims"], rot["base"], "half") for t in range(T)])
    kr = torch.stack([rotate(k[t], t, rot["dims"], rot["base"], "half") for t in range(T)])
    o = masked_attention(qr, kr, k, m["scale"], window, keep, w[p + ".sink"], gate)
    return o.reshape(T, H * dk) @ w[p + ".o"].T


def latent_keys_values(c, kt, w_uk, w_uv, H: int):
    """Per head keys [T, H, dn + dr] = [W_uk c | shared rotated part] and values [T, H, dv] = W_uv c from the latent c [T, R]
    and the shared part kt [T, dr]."""
    T = c.shape[0]
    kn = (c @ w_uk.T).view(T, H, -1)
    return torch.cat([kn, kt.unsqueeze(1).expand(T, H, kt.shape[1])], dim=-1), (c @ w_uv.T).view(T, H, -1)


def latent_attention_mixer(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """Causal softmax attention over a shared latent.  h [T, D] -> [T, D].
    Queries: c_q = rms_norm(W_dq h) * w, q = W_uq c_q, per head [dn | dr].  Keys / values: W_dkv h = [R | dr]; the first R,
    RMS-normed, are the latent c, the last dr one rotated key part for all heads; per head k = [W_uk c | rotated part],
    v = W_uv c.  Rotation in the "interleaved" layout on the dr parts; sigmoid gate per head."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {"dims": dr, "base": 10000.0}
    cq = rms_norm(h @ w[p + ".dq"].T, w[p + ".dq.norm"], eps)
    q = (cq @ w[p + ".uq"].T).view(T, H, dn + dr).clone()
    dkv = h @ w[p + ".dkv"].T
    c = rms_norm(dkv[:, :R], w[p + ".dkv.norm"], eps)
    kt = torch.stack([rotate(dkv[t, R:], t, rot["dims"], rot["base"], "interleaved") for t in range(T)])     # [T, dr]
    for t in range(T):
        q[t, :, dn:] = rotate(q[t, :, dn:], t, rot["dims"], rot["base"], "interleaved")
    keys, values = latent_keys_values(c, kt, w[p + ".uk"], w[p + ".uv"], H)
    o = masked_attention(q, keys, values, m["scale"], gates=sigmoid(h @ w[p + ".g"].T))
    return o.reshape(T, H * dv) @ w[p + ".o"].T


def dense_ff(h, w: Dict[str, torch.Tensor], p: str):
    """W_down relu(W_up h)^2."""
    return relu_sq(h @ w[p + ".up"].T) @ w[p + ".down"].T


# ------------------------------------------------------------------------------------------------ the model
def weight_layer(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else int(j)


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """Name -> shape of a checkpoint's tensors (a layer with weights_of has none)."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}", L["mixer"]
        out[p + ".norm1"] = out[p + ".norm1b"] = (D,)
        q = p + ".mix"
        if L["type"] == "lightning":
            n = m["heads"] * m["vdim"]
            out.update({q + ".q": (m["heads"] * m["dim"], D), q + ".k": (m["heads"] * m["dim"], D), q + ".v": (n, D),
                        q + ".g": (n, D), q + ".o": (D, n), q + ".norm": (n,)})
        elif L["type"] == "attention":
            nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            out.update({q + ".q": (nq, D), q + ".q.b": (nq,), q + ".k": (nk, D), q + ".k.b": (nk,), q + ".sink": (m["heads"],),
                        q + ".g": (m["heads"], D), q + ".o": (D, nq)})
        else:
            H, R, Rq = m["heads"], m["kv_rank"], m["q_rank"]
            out.update({q + ".dq": (Rq, D), q + ".dq.norm": (Rq,), q + ".uq": (H * (m["dim"] + m["rot_dim"]), Rq),
                        q + ".dkv": (R + m["rot_dim"], D), q + ".dkv.norm": (R,), q + ".uk": (H * m["dim"], R),
                        q + ".uv": (H * m["vdim"], R), q + ".g": (H, D), q + ".o": (D, H * m["vdim"])})
        if L.get("mlp"):
            out[p + ".norm2"] = out[p + ".norm2b"] = (D,)
            out.update({p + ".mlp.up": (L["mlp"]["ff"], D), p + ".mlp.down": (D, L["mlp"]["ff"])})
    return out


def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16 tensors of a configuration: matrices with unit-variance outputs, layer-norm weights around zero, plain
    norm weights around one, sinks and biases of the order of the scores they sit beside."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(*shape, generator=g, dtype=torch.float32)
        if name.endswith(".b"):
            t = 0.3 * t
        elif name.endswith((".dq.norm", ".dkv.norm", ".mix.norm")):
            t = 1.0 + 0.2 * t
        elif name.endswith(".sink"):
            t = 1.5 * t
        elif len(shape) == 1:
            t = 0.2 * t
        elif name != "embed":
            t = t * shape[-1] ** -0.5
        out[name] = t.to(torch.bfloat16)
    return out


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None):
    """Logits [T, vocab] (float64) of one sequence from position 0; layers_out collects the residual after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, L in enumerate(cfg["layers"]):
        p = f"l{weight_layer(cfg, i)}"
        hin = offset_norm(x, w[p + ".norm1"], eps)
        kind, m = L["type"], L["mixer"]
        if kind == "lightning":
            y = lightning_mixer(hin, w, p + ".mix", m, eps)
        elif kind == "attention":
            y = window_attention_mixer(hin, w, p + ".mix", m)
        elif kind == "latent_attention":
            y = latent_attention_mixer(hin, w, p + ".mix", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer {kind!r}")
        x = x + offset_norm(y, w[p + ".norm1b"], eps)
        if L.get("mlp"):
            if L["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward {L['mlp']['kind']!r}")
            y = dense_ff(offset_norm(x, w[p + ".norm2"], eps), w, p + ".mlp")
            x = x + offset_norm(y, w[p + ".norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T * float(cfg["logit_scale"])
