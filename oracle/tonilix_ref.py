"""Plain CPU restatement of the Tonilix decoder, one function per mechanism (test infrastructure only).

Everything runs token by token or with explicit loops in float64 on whole sequences; nothing here is shared with
the product path under vllm-backend-public_b200/ (which never imports this file).  `weights` maps the checkpoint's
tensor names to tensors; `cfg` is the parsed config.json dictionary.

Notation: T tokens, D model width, H query heads, G key/value heads, dk / dv per-head key and value sizes, E experts.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

F64 = torch.float64


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_div(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_rms_norm(x, w, groups: int, eps: float):
    """The last axis is cut into `groups` equal consecutive parts, each divided by its own root mean square; then * w."""
    D = x.shape[-1]
    parts = x.reshape(*x.shape[:-1], groups, D // groups)
    return rms_div(parts, eps).reshape(x.shape) * w


def sinusoid(positions, D: int, dtype=F64):
    """[T, D]: entry 2i = sin(p * 10000^(-2i / D)), entry 2i + 1 = cos of the same angle."""
    out = torch.zeros(len(positions), D, dtype=dtype)
    for n, p in enumerate(positions):
        for i in range((D + 1) // 2):
            a = p * 10000.0 ** (-2.0 * i / D)
            out[n, 2 * i] = math.sin(a)
            if 2 * i + 1 < D:
                out[n, 2 * i + 1] = math.cos(a)
    return out


def token_shift(h, mu):
    """h [T, D] -> h[t] + (h[t-1] - h[t]) * mu, with zeros before the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]])
    return h + (prev - h) * mu


# ------------------------------------------------------------------------------------------------ mixers
def causal_conv(x, w):
    """x [T, C], w [C, taps]; y[t, c] = sum_j w[c, taps-1-j] * x[t-j, c], zeros before the sequence."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j] * x[t - j]
    return y


def channel_delta_rule(q, k, v, beta, g):
    """Gated delta rule for ONE head with a decay per key channel.  q, k, g [T, dk]; v [T, dv]; beta [T]."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    o = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t].unsqueeze(1) * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.t() @ q[t]
    return o


def channel_delta_mixer(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """h [T, D] -> [T, D].  p = '<layer>.mix'."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[p + ".q"].t(), W[p + ".q.conv"])).view(T, G, dk)
    k = silu(causal_conv(h @ W[p + ".k"].t(), W[p + ".k.conv"])).view(T, G, dk)
    v = silu(causal_conv(h @ W[p + ".v"].t(), W[p + ".v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + ".b"].t())                                        # [T, H]
    a = (h @ W[p + ".a1"].t()) @ W[p + ".a2"].t() + W[p + ".dt_bias"]                # [T, H * dk]
    g = torch.exp(-torch.exp(W[p + ".A_log"]).view(1, H, 1) * softplus(a).view(T, H, dk))
    gate = torch.sigmoid((h @ W[p + ".g1"].t()) @ W[p + ".g2"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        kv = hh // (H // G)
        o = channel_delta_rule(q[:, kv], k[:, kv], v[:, hh], beta[:, hh], g[:, hh])
        out[:, hh] = rms_div(o, eps) * W[p + ".norm"] * gate[:, hh]
    return out.reshape(T, H * dv) @ W[p + ".o"].t()


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def causal_attention(q, k, v, scale: float):
    """ONE head.  q, k [T, dk]; v [T, dv]; position i sees every j <= i; ordinary softmax."""
    T = q.shape[0]
    o = torch.zeros(T, v.shape[1], dtype=q.dtype)
    for i in range(T):
        s = (k[:i + 1] @ q[i]) * scale
        e = torch.exp(s - s.max())
        o[i] = (e.unsqueeze(1) * v[:i + 1]).sum(0) / e.sum()
    return o


def gated_attention_mixer(h, W, p: str, m: dict):
    """Softmax attention with biased projections, a position-dependent query factor and a sigmoid output gate."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[p + ".q"].t() + W[p + ".q.b"]).view(T, H, dk)
    k = (h @ W[p + ".k"].t() + W[p + ".k.b"]).view(T, G, dk)
    v = (h @ W[p + ".v"].t() + W[p + ".v.b"]).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        f = torch.tensor([query_temperature(i, qt["coef"], qt["every"]) for i in range(T)], dtype=h.dtype)
        q = q * f.view(T, 1, 1)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        kv = hh // (H // G)
        out[:, hh] = causal_attention(q[:, hh], k[:, kv], v[:, kv], m["scale"])
    gate = torch.sigmoid(h @ W[p + ".g"].t())
    return (out.reshape(T, H * dv) * gate) @ W[p + ".o"].t() + W[p + ".o.b"]


def gated_linear_rule(q, k, v, alpha):
    """ONE head: S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k, alpha [T, dk]; v [T, dv]."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=q.dtype)
    o = torch.zeros(T, dv, dtype=q.dtype)
    for t in range(T):
        S = alpha[t].unsqueeze(1) * S + torch.outer(k[t], v[t])
        o[t] = S.t() @ q[t]
    return o


def gated_linear_mixer(h, W, p: str, m: dict, eps: float):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ W[p + ".q"].t()).view(T, H, dk) * dk ** -0.5
    k = (h @ W[p + ".k"].t()).view(T, H, dk)
    v = (h @ W[p + ".v"].t()).view(T, H, dv)
    z = (h @ W[p + ".a1"].t()) @ W[p + ".a2"].t() + W[p + ".a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        out[:, hh] = rms_div(gated_linear_rule(q[:, hh], k[:, hh], v[:, hh], alpha[:, hh]), eps) * W[p + ".norm"]
    return (out.reshape(T, H * dv) * silu(h @ W[p + ".g"].t())) @ W[p + ".o"].t()


def parallel_mixer(h, W, p: str, m: dict, eps: float):
    left = gated_attention_mixer(h, W, p + ".left", m["left"])
    right = gated_linear_mixer(h, W, p + ".right", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, W, p: str):
    return (gelu_tanh(h @ W[p + ".gate"].t()) * (h @ W[p + ".up"].t())) @ W[p + ".down"].t()


def grouped_route(z, correction, r: dict):
    """Router logits z [E] of ONE token -> (expert indices, weights).  Scores are sigmoids; the choice looks at score +
    correction, inside the `keep` groups with the largest sum of their two best choice scores; the weights are the plain
    scores of the chosen, normalised to sum 1 and scaled."""
    E, top = z.shape[0], r["top"]
    s = torch.sigmoid(z)
    c = s + correction
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        n, per = groups["count"], E // groups["count"]
        gs = [float(torch.topk(c[j * per:(j + 1) * per], min(2, per)).values.sum()) for j in range(n)]
        kept = sorted(range(n), key=lambda j: (-gs[j], j))[:groups["keep"]]
        allowed = [e for e in range(E) if e // per in kept]
    else:
        allowed = list(range(E))
    order = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    w = torch.stack([s[e] for e in order])
    return order, w / (w.sum() + 1e-20) * r["scale"]


def moe_ff(h, W, p: str, f: dict):
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, wt = grouped_route(W[p + ".router"] @ h[t], W[p + ".correction"], f["router"])
        for j, e in enumerate(idx):
            a = torch.relu(W[f"{p}.e{e}.up"] @ h[t]) ** 2
            y[t] += wt[j] * (W[f"{p}.e{e}.down"] @ a)
    return y


# ------------------------------------------------------------------------------------------------ whole model
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens, dtype=F64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the residual after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    D = cfg["width"]
    T = len(tokens)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] + sinusoid(range(T), D).to(dtype)
    x = group_rms_norm(x, W["embed.norm"], groups, eps)
    trail = []
    for li, L in enumerate(cfg["layers"]):
        p = f"l{li}"
        h = token_shift(group_rms_norm(x, W[p + ".norm1"], groups, eps), W[p + ".shift"])
        if L["type"] == "channel_delta":
            y = channel_delta_mixer(h, W, p + ".mix", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(h, W, p + ".mix", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + y * W[p + ".ls1"]
        f = L.get("mlp")
        if f:
            h = group_rms_norm(x, W[p + ".norm2"], groups, eps)
            y = dense_ff(h, W, p + ".mlp") if f["kind"] == "dense" else moe_ff(h, W, p + ".mlp", f)
            x = x + y * W[p + ".ls2"]
        trail.append(x)
    logits = group_rms_norm(x, W["final.norm"], groups, eps) @ W["head"].t()
    return (logits, torch.stack(trail)) if return_layers else logits


# ------------------------------------------------------------------------------------------------ random models
def random_model(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 weights (every name the loader expects) for a config, scaled so that activations stay O(1)."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def rnd(*shape, std):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    W = {"embed": rnd(cfg["vocab"], D, std=1.0), "embed.norm": 1 + rnd(D, std=0.1), "head": rnd(cfg["vocab"], D, std=D ** -0.5),
         "final.norm": 1 + rnd(D, std=0.1)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        W[p + ".norm1"] = 1 + rnd(D, std=0.1)
        W[p + ".ls1"] = 1 + rnd(D, std=0.2)
        W[p + ".shift"] = (torch.rand(D, generator=g) * 0.8).to(torch.bfloat16)
        if L["type"] == "channel_delta":
            H, G, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            q = p + ".mix"
            W[q + ".q"] = rnd(G * dk, D, std=D ** -0.5)
            W[q + ".k"] = rnd(G * dk, D, std=D ** -0.5)
            W[q + ".v"] = rnd(H * dv, D, std=D ** -0.5)
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                W[f"{q}.{n}.conv"] = rnd(c, taps, std=taps ** -0.5)
            ra, rg = m.get("_rank_a", 8), m.get("_rank_g", 8)
            W[q + ".b"] = rnd(H, D, std=D ** -0.5)
            W[q + ".a1"] = rnd(ra, D, std=D ** -0.5)
            W[q + ".a2"] = rnd(H * dk, ra, std=ra ** -0.5)
            W[q + ".A_log"] = rnd(H, std=0.5) - 1.0
            W[q + ".dt_bias"] = rnd(H * dk, std=0.5)
            W[q + ".norm"] = 1 + rnd(dv, std=0.1)
            W[q + ".g1"] = rnd(rg, D, std=D ** -0.5)
            W[q + ".g2"] = rnd(H * dv, rg, std=rg ** -0.5)
            W[q + ".o"] = rnd(D, H * dv, std=(H * dv) ** -0.5)
        else:
            a, b = m["left"], m["right"]
            q = p + ".mix.left"
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for n, c in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                W[f"{q}.{n}"] = rnd(c, D, std=D ** -0.5)
                W[f"{q}.{n}.b"] = rnd(c, std=0.1)
            W[q + ".g"] = rnd(H * dv, D, std=D ** -0.5)
            W[q + ".o"] = rnd(D, H * dv, std=(H * dv) ** -0.5)
            W[q + ".o.b"] = rnd(D, std=0.1)
            q = p + ".mix.right"
            H, dk, dv, ra = b["heads"], b["dim"], b["vdim"], b.get("_rank_a", 8)
            W[q + ".q"] = rnd(H * dk, D, std=D ** -0.5)
            W[q + ".k"] = rnd(H * dk, D, std=D ** -0.5)
            W[q + ".v"] = rnd(H * dv, D, std=D ** -0.5)
            W[q + ".g"] = rnd(H * dv, D, std=D ** -0.5)
            W[q + ".o"] = rnd(D, H * dv, std=(H * dv) ** -0.5)
            W[q + ".norm"] = 1 + rnd(dv, std=0.1)
            W[q + ".a1"] = rnd(ra, D, std=D ** -0.5)
            W[q + ".a2"] = rnd(H * dk, ra, std=ra ** -0.5)
            W[q + ".a2.b"] = rnd(H * dk, std=0.5) + 2.0
        f = L.get("mlp")
        if f:
            W[p + ".norm2"] = 1 + rnd(D, std=0.1)
            W[p + ".ls2"] = 1 + rnd(D, std=0.2)
            if f["kind"] == "dense":
                W[p + ".mlp.gate"] = rnd(f["ff"], D, std=D ** -0.5)
                W[p + ".mlp.up"] = rnd(f["ff"], D, std=D ** -0.5)
                W[p + ".mlp.down"] = rnd(D, f["ff"], std=f["ff"] ** -0.5)
            else:
                ff, E = f["expert"]["ff"], f["router"]["experts"]
                for e in range(E):
                    W[f"{p}.mlp.e{e}.up"] = rnd(ff, D, std=D ** -0.5)
                    W[f"{p}.mlp.e{e}.down"] = rnd(D, ff, std=ff ** -0.5)
                W[p + ".mlp.router"] = rnd(E, D, std=4.0 * D ** -0.5)
                W[p + ".mlp.correction"] = rnd(E, std=0.3)
    return W
