"""Every mechanism of the Tonilix family alone, against the plain oracle (oracle/tonilix_ref.py): the positional embedding,
the norm in groups with sublayer scale and token shift (state carried across calls, dirty slots), the recurrences with a
decay per key channel (delta correction and plain write) in portions, the attention's query temperature at its steps and a
loud key far back, the output gates, the grouped sigmoid router and the ungated experts.  fp32 compares tightly; bf16
against the same oracle fed the rounded inputs."""
import math

import pytest
import torch

import tonilix_ref as R

pytestmark = pytest.mark.gpu

F64 = torch.float64


def _ops():
    from b200attn import ops
    return ops


def _close(got, want, tol, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / (want.abs().max() + 1e-30))
    assert err <= tol, f"{what}: relative error {err:.3e} above {tol:.1e}"


def _batch(cuda, lens, ctx, slots, tables=None):
    ops = _ops()
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=cuda)      # noqa: E731
    return ops.SeqBatch(i32(cu), i32(ctx), None if tables is None else i32(tables), i32(slots), len(lens), cu[-1])


# ------------------------------------------------------------------------------------------------ embedding
@pytest.mark.parametrize("D,groups", [(48, 1), (64, 4), (30, 5), (33, 3), (2048, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_positions_near_and_far(cuda, D, groups, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(D)
    emb = torch.randn(23, D, generator=g).to(dtype)
    w = 1 + 0.2 * torch.randn(D, generator=g)
    pos = [0, 1, 2, 17, 255, 256, 4095, 65537, 1000003]
    tok = torch.randint(0, 23, (len(pos),), generator=g)
    freq = ops.sinusoid_frequencies(D, device=cuda)
    x = ops.embed_sinusoid_norm(emb.to(cuda), tok.to(cuda), torch.tensor(pos, dtype=torch.int32, device=cuda), freq, w.to(cuda),
                                groups, 1e-6)
    want = R.group_rms_norm(emb.to(F64)[tok] + R.sinusoid(pos, D), w.to(F64), groups, 1e-6)
    assert x.dtype == torch.float32
    _close(x, want, 2e-6, "embedding")          # the angle is exact in fp32 at any position
    raw = ops.embed_sinusoid_norm(emb.to(cuda), tok.to(cuda), torch.tensor(pos, dtype=torch.int32, device=cuda), freq, None, 1, 0.0)
    _close(raw, emb.to(F64)[tok] + R.sinusoid(pos, D), 2e-6, "embedding without a norm")


# ------------------------------------------------------------------------------------------------ norm, scale, shift
@pytest.mark.parametrize("D,groups", [(48, 1), (64, 4), (30, 5), (36, 12), (40, 40), (1024, 2), (4096, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_norm_step_without_shift(cuda, D, groups, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(D + groups)
    T = 5
    x = torch.randn(T, D, generator=g) * 3 + 0.5
    y = torch.randn(T, D, generator=g).to(dtype)
    ls, yb, w = 1 + 0.3 * torch.randn(D, generator=g), 0.2 * torch.randn(D, generator=g), 1 + 0.2 * torch.randn(D, generator=g)
    xd = x.to(cuda)
    h = ops.group_norm_step(xd, y.to(cuda), ls.to(cuda), yb.to(cuda), w.to(cuda), groups, 1e-5, h_dtype=dtype)
    x2 = x.to(F64) + ls.to(F64) * (y.to(F64) + yb.to(F64))
    _close(xd, x2, 1e-6, "residual")
    _close(h, R.group_rms_norm(x2, w.to(F64), groups, 1e-5), 1e-5 if dtype == torch.float32 else 1e-2, "read-out")
    # the read-out alone leaves the residual untouched; the write-back alone returns nothing; no scale means ones
    before = xd.clone()
    h2 = ops.group_norm_step(xd, norm_w=w.to(cuda), groups=groups, eps=1e-5, h_dtype=dtype)
    assert torch.equal(before, xd) and torch.equal(h2, h)
    assert ops.group_norm_step(xd, y.to(cuda)) is None
    _close(xd, x2 + y.to(F64), 1e-6, "plain residual add")


@pytest.mark.parametrize("D,groups", [(64, 4), (30, 3), (512, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_in_portions_with_dirty_slots(cuda, D, groups, dtype):
    """Two sequences fed in portions (down to one and two tokens) beside each other, their slots swapped relative to their
    order and dirty from an earlier occupant: the shifted read-out equals the oracle over the whole sequences, the first
    token blends with zeros, and a portion's first row blends with the row the state kept."""
    ops = _ops()
    g = torch.Generator().manual_seed(D)
    lens = [23, 12]
    xs = [torch.randn(n, D, generator=g) * 2 for n in lens]
    ys = [torch.randn(n, D, generator=g).to(dtype) for n in lens]
    ls, w, mu = 1 + 0.3 * torch.randn(D, generator=g), 1 + 0.2 * torch.randn(D, generator=g), torch.rand(D, generator=g)
    want_x = [x.to(F64) + ls.to(F64) * y.to(F64) for x, y in zip(xs, ys)]
    want_h = [R.token_shift(R.group_rms_norm(x, w.to(F64), groups, 1e-5), mu.to(F64)) for x in want_x]
    state = torch.full((3, D), 77.0, device=cuda)
    slots = [2, 0]
    cuts = [[1, 2, 5, 1, 14], [2, 1, 1, 8]]
    at = [0, 0]
    for step in range(5):
        rows, lens_now, ctx, sl, who = [], [], [], [], []
        for s in (0, 1):
            if step < len(cuts[s]):
                n = cuts[s][step]
                lens_now.append(n), ctx.append(at[s]), sl.append(slots[s]), who.append((s, at[s], n))
                at[s] += n
        x = torch.cat([xs[s][a:a + n] for s, a, n in who]).to(cuda)
        y = torch.cat([ys[s][a:a + n] for s, a, n in who]).to(cuda)
        out = torch.empty_like(x)
        b = _batch(cuda, lens_now, ctx, sl)
        h = ops.group_norm_step(x, y, ls.to(cuda), None, w.to(cuda), groups, 1e-5, h_dtype=dtype, shift_mu=mu.to(cuda),
                                shift_state=state, batch=b, x_out=out)
        off = 0
        for s, a, n in who:
            _close(out[off:off + n], want_x[s][a:a + n], 1e-6, f"residual of sequence {s} at {a}")
            _close(h[off:off + n], want_h[s][a:a + n], 2e-5 if dtype == torch.float32 else 1.5e-2, f"shifted rows of sequence {s} at {a}")
            off += n
    assert bool((state[1] == 77.0).all())                       # a slot no sequence holds is not touched
    with pytest.raises(ValueError, match="x_out"):
        ops.group_norm_step(x, y, ls.to(cuda), None, w.to(cuda), groups, 1e-5, h_dtype=dtype, shift_mu=mu.to(cuda),
                            shift_state=state, batch=b)


def test_token_shift_skips_padding_rows(cuda):
    ops = _ops()
    D = 32
    x = torch.randn(3, D, device=cuda)
    state = torch.full((2, D), 5.0, device=cuda)
    w, mu = torch.ones(D, device=cuda), torch.full((D,), 0.5, device=cuda)
    b = _batch(cuda, [1, 1, 1], [4, -1, 0], [1, 0, 0])           # row 1 is padding that names slot 0 like row 2
    h = ops.group_norm_step(x, norm_w=w, groups=1, eps=1e-6, h_dtype=torch.float32, shift_mu=mu, shift_state=state, batch=b)
    n = R.group_rms_norm(x.double().cpu(), torch.ones(D, dtype=F64), 1, 1e-6)
    _close(h[0], n[0] + (5.0 - n[0]) * 0.5, 1e-5, "row with context")
    _close(h[2], n[2] * 0.5, 1e-5, "row at position 0")
    _close(state[0], n[2], 1e-5, "slot 0 holds row 2, not the padding row")
    _close(state[1], n[0], 1e-5)


# ------------------------------------------------------------------------------------------------ recurrences
def _recur_oracle(kind, proj, a, conv_w, A_log, bias, beta_w, H, G, dk, dv, tau):
    """One sequence in fp64: q | k | v (prepared), decay, o."""
    T = proj.shape[0]
    C = 2 * G * dk + H * dv
    z = proj[:, :C]
    if kind == "delta":
        z = R.silu(R.causal_conv(z, conv_w))
    q, k, v = z[:, :G * dk].view(T, G, dk), z[:, G * dk:2 * G * dk].view(T, G, dk), z[:, 2 * G * dk:].view(T, H, dv)
    if kind == "delta":
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-torch.exp(A_log).view(1, H, 1) * R.softplus(a + bias).view(T, H, dk))
        beta = torch.sigmoid(proj[:, C:C + H])
    else:
        decay = (torch.sigmoid(a + bias) ** (1.0 / tau)).view(T, H, dk)
    q = q * dk ** -0.5
    o = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        kv = h // (H // G)
        o[:, h] = R.channel_delta_rule(q[:, kv], k[:, kv], v[:, h], beta[:, h], decay[:, h]) if kind == "delta" \
            else R.gated_linear_rule(q[:, kv], k[:, kv], v[:, h], decay[:, h])
    return torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1), decay.reshape(T, H * dk), o


@pytest.mark.parametrize("kind", ["delta", "plain"])
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 16, 24, 3), (2, 2, 40, 72, 1), (3, 1, 10, 6, 6), (2, 1, 128, 64, 4),
                                            (1, 1, 200, 40, 2), (1, 1, 30, 6, 3), (2, 2, 32, 32, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrences_with_a_decay_per_channel_in_portions(cuda, kind, H, G, dk, dv, taps, dtype):
    """Two sequences of unequal length fed in portions (down to one and two tokens), their slots swapped and dirty: the
    prepared inputs, the decay and the read-out equal the oracle run over the whole sequences."""
    ops = _ops()
    if kind == "plain":
        G, taps = H, 1
    g = torch.Generator().manual_seed(dk * 7 + taps)
    C = 2 * G * dk + H * dv
    P = C + H + 3                                                # beta columns behind q | k | v, and a few unused ones
    lens = [23, 12]
    proj = [(torch.randn(n, P, generator=g) * 1.5).to(dtype) for n in lens]
    a = [torch.randn(n, H * dk, generator=g) * 2 for n in lens]
    conv_w = torch.randn(C, taps, generator=g) * taps ** -0.5
    A_log = torch.randn(H, generator=g) - 1
    bias = torch.randn(H * dk, generator=g) + (2.0 if kind == "plain" else 0.0)
    tau = 5.0
    want = [_recur_oracle(kind, p.to(F64), x.to(F64), conv_w.to(F64), A_log.to(F64), bias.to(F64), None, H, G, dk, dv, tau)
            for p, x in zip(proj, a)]
    state = torch.full((3, H, dk, dv), 9.0, device=cuda)
    conv_state = torch.full((3, max(taps - 1, 1), C), 9.0, dtype=dtype, device=cuda)[:, :taps - 1].contiguous() if taps > 1 else None
    slots, cuts, at = [2, 0], [[1, 2, 5, 1, 14], [2, 1, 1, 8]], [0, 0]
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    for step in range(5):
        lens_now, ctx, sl, who = [], [], [], []
        for s in (0, 1):
            if step < len(cuts[s]):
                n = cuts[s][step]
                lens_now.append(n), ctx.append(at[s]), sl.append(slots[s]), who.append((s, at[s], n))
                at[s] += n
        pj = torch.cat([proj[s][x:x + n] for s, x, n in who]).to(cuda)
        aa = torch.cat([a[s][x:x + n] for s, x, n in who]).to(cuda)
        b = _batch(cuda, lens_now, ctx, sl)
        if kind == "delta":
            qkv, beta, decay = ops.recur_prep(pj, H, G, dk, dv, b, taps=taps, conv_w=conv_w.to(cuda), conv_state=conv_state,
                                              conv_silu=True, unit=True, q_scale=dk ** -0.5, off_beta=C,
                                              decay_mode=ops.DECAY_CHANNEL_SOFTPLUS, a=aa, A_log=A_log.to(cuda),
                                              decay_bias=bias.to(cuda))
        else:
            qkv, beta, decay = ops.recur_prep(pj, H, G, dk, dv, b, q_scale=dk ** -0.5, decay_mode=ops.DECAY_CHANNEL_SIGMOID_POW,
                                              a=aa, decay_bias=bias.to(cuda), tau=tau)
            assert beta is None
        o = ops.channel_scan(qkv, beta, decay, H, G, dk, dv, b, state, delta=kind == "delta")
        off = 0
        for s, x, n in who:
            _close(qkv[off:off + n], want[s][0][x:x + n], tol, f"inputs of sequence {s} at {x}")
            _close(decay[off:off + n], want[s][1][x:x + n], 1e-5, f"decay of sequence {s} at {x}")
            _close(o[off:off + n], want[s][2][x:x + n], tol * 4, f"read-out of sequence {s} at {x}")
            off += n
    assert bool((state[1] == 9.0).all())


@pytest.mark.parametrize("delta", [False, True])
def test_a_token_far_back_stays_in_the_state(cuda, delta):
    """One key channel does not decay and only token 3 writes to it; 900 tokens later, in single-token steps, a query on that
    channel still reads token 3's value -- and nothing when the decay of that channel is 0.9."""
    ops = _ops()
    H, dk, dv, T = 1, 8, 4, 904
    for keep in (1.0, 0.9):
        q = torch.zeros(T, dk)
        k = torch.zeros(T, dk)
        k[:, 1:] = 0.05 * torch.randn(T, dk - 1, generator=torch.Generator().manual_seed(1))
        v = torch.randn(T, dv, generator=torch.Generator().manual_seed(2))
        k[3] = 0
        k[3, 0], q[T - 1, 0] = 1.0, 1.0
        decay = torch.full((T, dk), 0.5)
        decay[:, 0] = keep
        beta = torch.ones(T, 1)
        qkv = torch.cat([q, k, v], 1).to(cuda)
        state = torch.zeros(1, H, dk, dv, device=cuda)
        o = ops.channel_scan(qkv[:600], beta[:600].to(cuda), decay[:600].to(cuda), H, H, dk, dv, _batch(cuda, [600], [0], [0]), state, delta)
        for t in range(600, T):
            o = ops.channel_scan(qkv[t:t + 1], beta[t:t + 1].to(cuda), decay[t:t + 1].to(cuda), H, H, dk, dv,
                                 _batch(cuda, [1], [t], [0]), state, delta)
        if keep == 1.0:
            _close(o[0, 0], v[3].double(), 1e-5)
        else:
            assert float(o.abs().max()) < 1e-6


@pytest.mark.parametrize("kind", ["silu", "sigmoid"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_head_norm_and_gate_mul(cuda, kind, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    T, H, dv = 7, 3, 20
    o = torch.randn(T, H, dv, generator=g) * 4
    wide = torch.randn(T, H * dv + 11, generator=g).to(dtype)        # the gate is a view into wider rows
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    k = ops.GATE_SILU if kind == "silu" else ops.GATE_SIGMOID
    act = R.silu if kind == "silu" else torch.sigmoid
    gate = wide.to(cuda)[:, 5:5 + H * dv]
    out = torch.zeros(T, H * dv + 4, dtype=dtype, device=cuda)
    ops.gated_head_norm(o.to(cuda), gate, w.to(cuda), 1e-5, k, 1.3, out=out[:, 4:])
    want = (R.rms_div(o.to(F64), 1e-5) * w.to(F64)).reshape(T, H * dv) * act(wide.to(F64)[:, 5:5 + H * dv]) * 1.3
    _close(out[:, 4:], want, 1e-5 if dtype == torch.float32 else 1e-2)
    assert bool((out[:, :4] == 0).all())
    x = torch.randn(T, H * dv, generator=g).to(dtype)
    got = ops.gate_mul(x.to(cuda), gate, k, 0.7)
    _close(got, x.to(F64) * act(wide.to(F64)[:, 5:5 + H * dv]) * 0.7, 1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_gated_unit(cuda, dtype):
    ops = _ops()
    gu = (torch.randn(5, 2 * 37, generator=torch.Generator().manual_seed(8)) * 3).to(dtype)
    got = ops.glu_and_mul(gu.to(cuda), ops.GLU_GELU_TANH)
    _close(got, R.gelu_tanh(gu.to(F64)[:, :37]) * gu.to(F64)[:, 37:], 1e-6 if dtype == torch.float32 else 1e-2)


# ------------------------------------------------------------------------------------------------ attention
def _paged(cuda, ops, dtype, G, dk, dv, bs, n_pages, seed):
    kc = torch.full((n_pages, G, bs, dk), float("nan"), dtype=dtype, device=cuda)
    vc = torch.full((n_pages, G, bs, dv), float("nan"), dtype=dtype, device=cuda)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    return kc, vc, perm


@pytest.mark.parametrize("H,G,dk,dv,every", [(4, 2, 16, 24, 7), (3, 3, 40, 8, 1), (2, 1, 32, 64, 16), (1, 1, 14, 14, 1000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_query_temperature_over_shuffled_pages(cuda, H, G, dk, dv, every, dtype):
    """A prompt of 45 tokens, then a portion of 2 and single tokens up to 70: the temperature steps at every multiple of
    `every` (positions just before and at a step are queried in the prompt and in decoding); pages are shuffled and the
    pages of no sequence hold NaN."""
    ops = _ops()
    g = torch.Generator().manual_seed(dk + every)
    T, bs, coef, scale = 70, 8, 0.9, 0.31
    qkv = torch.randn(T, (H + G) * dk + G * dv, generator=g).to(dtype)
    q64 = qkv.to(F64)[:, :H * dk].view(T, H, dk)
    k64 = qkv.to(F64)[:, H * dk:(H + G) * dk].view(T, G, dk)
    v64 = qkv.to(F64)[:, (H + G) * dk:].view(T, G, dv)
    f = torch.tensor([R.query_temperature(p, coef, every) for p in range(T)], dtype=F64)
    want = torch.stack([R.causal_attention(q64[:, h] * f.view(T, 1), k64[:, h // (H // G)], v64[:, h // (H // G)], scale)
                        for h in range(H)], 1)
    kc, vc, perm = _paged(cuda, ops, dtype, G, dk, dv, bs, 12, every)
    table = perm[:9]
    at = 0
    for n in [45, 2] + [1] * 23:
        pos = torch.arange(at, at + n, dtype=torch.int32, device=cuda)
        slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(at, at + n)], dtype=torch.int64, device=cuda)
        q = ops.qk_prep_cache(qkv[at:at + n].to(cuda), H, G, dk, dv, slots, kc, vc, pos, coef, every)
        o = ops.chunk_attention(q, kc, vc, _batch(cuda, [n], [at], [0], [table]), scale)
        _close(o, want[at:at + n], 2e-5 if dtype == torch.float32 else 2e-2, f"rows {at}..{at + n}")
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_loud_key_far_back_is_found(cuda, dtype):
    """Among 700 keys one (position 5) matches the query of the last prompt row and of a decoded row; the output is its value."""
    ops = _ops()
    H, G, dk, dv, bs, T = 2, 1, 16, 8, 16, 700
    g = torch.Generator().manual_seed(3)
    qkv = (torch.randn(T + 1, (H + G) * dk + G * dv, generator=g) * 0.3).to(dtype)
    qkv[5, H * dk:(H + G) * dk] = 0
    qkv[5, H * dk] = 30.0
    for t in (T - 1, T):
        qkv[t, :H * dk] = 0
        qkv[t, 0], qkv[t, dk] = 30.0, 30.0
    kc, vc, perm = _paged(cuda, ops, dtype, G, dk, dv, bs, 50, 1)
    table = perm[:44]
    for at, n in ((0, T), (T, 1)):
        slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(at, at + n)], dtype=torch.int64, device=cuda)
        q = ops.qk_prep_cache(qkv[at:at + n].to(cuda), H, G, dk, dv, slots, kc, vc)
        o = ops.chunk_attention(q, kc, vc, _batch(cuda, [n], [at], [0], [table]), 1.0)
        for h in range(H):
            _close(o[-1, h], qkv[5, (H + G) * dk:].double(), 1e-3 if dtype == torch.float32 else 1e-2, f"head {h} at {at + n - 1}")


# ------------------------------------------------------------------------------------------------ router and experts
def _route_oracle(z, corr, top, groups, keep, scale):
    r = {"top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups, "keep": keep}
    ids, wts = [], []
    for t in range(z.shape[0]):
        i, w = R.grouped_route(z[t], corr, r)
        ids.append(i), wts.append(w)
    return torch.tensor(ids), torch.stack(wts)


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 4, 2), (6, 2, 3, 1), (9, 3, 3, 2), (6, 2, 6, 3), (5, 5, 1, 1), (64, 6, 8, 4), (3, 1, 0, 0)])
@pytest.mark.parametrize("T", [5, 40])
def test_grouped_router_against_the_oracle(cuda, E, top, groups, keep, T):
    """T = 5 computes the logits in the routing kernel, T = 40 in a library GEMM with the choice in a kernel of its own.
    The correction is large enough to change choices and to make choice scores negative."""
    ops = _ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    D = 24
    h = torch.randn(T, D, generator=g)
    wr = torch.randn(E, D, generator=g) * 0.5
    corr = torch.randn(E, generator=g) * 0.8 - 0.5
    ids, wts = ops.moe_route(h.to(cuda), wr.to(cuda), corr.to(cuda), top, ops.ROUTE_SIGMOID_GROUPED, max(groups, 1), max(keep, 1), 1.75)
    z = h.to(F64) @ wr.to(F64).t()
    want_ids, want_w = _route_oracle(z, corr.to(F64), top, groups, keep, 1.75)
    plain_ids, _ = _route_oracle(z, torch.zeros(E, dtype=F64), top, 0, 0, 1.75)
    assert torch.equal(ids.cpu().long(), want_ids), "choice"
    _close(wts, want_w, 1e-5, "weights")
    assert E < 6 or E <= top or not torch.equal(want_ids, plain_ids)       # the correction and the groups do change the choice
    assert torch.allclose(wts.sum(1).cpu(), torch.full((T,), 1.75), atol=1e-5)


@pytest.mark.parametrize("dtype,T", [(torch.float32, 9), (torch.bfloat16, 9), (torch.bfloat16, 1500)])
def test_ungated_experts_and_their_independence_of_the_batch(cuda, dtype, T):
    ops = _ops()
    g = torch.Generator().manual_seed(T)
    D, F, E, top = 32, 24, 5, 2
    h = torch.randn(T, D, generator=g).to(dtype)
    up = (torch.randn(E, F, D, generator=g) * D ** -0.5).to(dtype)
    down = (torch.randn(E, D, F, generator=g) * F ** -0.5).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    y = ops.moe_experts(h.to(cuda), ids.to(cuda), wts.to(cuda), None, up.to(cuda), down.to(cuda), glu=ops.FF_RELU_SQ)
    want = torch.zeros(T, D, dtype=F64)
    for t in range(min(T, 40)):
        for j in range(top):
            e = int(ids[t, j])
            want[t] += wts[t, j].double() * (down[e].to(F64) @ torch.relu(up[e].to(F64) @ h[t].to(F64)) ** 2)
    _close(y[:40], want[:40], 1e-5 if dtype == torch.float32 else 3e-2)
    if T < 100:
        one = ops.moe_experts(h[3:4].to(cuda), ids[3:4].to(cuda), wts[3:4].to(cuda), None, up.to(cuda), down.to(cuda), glu=ops.FF_RELU_SQ)
        assert torch.equal(one[0], y[3])
    with pytest.raises(ValueError, match="gate"):
        ops.moe_experts(h.to(cuda), ids.to(cuda), wts.to(cuda), up.to(cuda), up.to(cuda), down.to(cuda), glu=ops.FF_RELU_SQ)
