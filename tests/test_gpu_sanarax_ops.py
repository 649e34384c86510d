"""Every mechanism of the Sanarax family alone, against the plain oracle (oracle/sanarax_ref.py): the norm of a latent, the
partial rotation in both pair layouts with the values taken from the unrotated keys, the window that keeps the first
tokens (mixed batches over shuffled pages, loud keys just inside and just outside every edge, in prompts and in decoding),
the sink per head, the gate per head, the linear attention with a fixed decay per head in portions over dirty state slots,
the norm over the concatenated heads, and the latent write from rows of two buffers.  fp32 compares tightly; bf16 against
the same oracle fed the rounded inputs."""
import math

import pytest
import torch

import sanarax_ref as R

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


def _pools(cuda, dtype, G, dk, bs, n_pages, seed):
    """K and V pools full of NaN and a shuffled page order: a read of a page no sequence owns shows."""
    kc = torch.full((n_pages, G, bs, dk), float("nan"), dtype=dtype, device=cuda)
    vc = torch.full((n_pages, G, bs, dk), float("nan"), dtype=dtype, device=cuda)
    return kc, vc, torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()


def _slots(cuda, table, bs, lo, hi):
    return torch.tensor([table[p // bs] * bs + p % bs for p in range(lo, hi)], dtype=torch.int64, device=cuda)


# ------------------------------------------------------------------------------------------------ norm of a latent
@pytest.mark.parametrize("n,stride", [(40, 40), (13, 29), (128, 200), (1500, 1500), (9000, 9004), (4098, 4100)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_norm_on_a_column_slice(cuda, n, stride, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(n)
    wide = (torch.randn(7, stride, generator=g) * 3).to(dtype)
    w = 1 + 0.3 * torch.randn(n, generator=g)
    x = wide.to(cuda)[:, stride - n:]
    got = ops.row_norm(x, w.to(cuda), 1e-5)
    assert got.dtype == dtype and got.is_contiguous()
    _close(got, R.rms_norm(wide.to(F64)[:, stride - n:], w.to(F64), 1e-5), 2e-6 if dtype == torch.float32 else 1e-2)
    _close(ops.row_norm(x, None, 1e-5), R.rms_norm(wide.to(F64)[:, stride - n:], None, 1e-5), 2e-6 if dtype == torch.float32 else 1e-2)


# ------------------------------------------------------------------------------------------------ rotation and pool write
@pytest.mark.parametrize("H,G,dk,dims", [(4, 2, 16, 8), (3, 1, 10, 10), (2, 2, 24, 0), (5, 5, 6, 2), (2, 1, 128, 64), (2, 2, 24, 12),
                                         (3, 1, 32, 32), (1, 1, 16, 4)])
@pytest.mark.parametrize("layout", ["half", "interleaved"])
@pytest.mark.parametrize("pad", [5, 8])              # a row stride that forbids / allows the four-entry accesses
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_and_values_from_the_unrotated_keys(cuda, H, G, dk, dims, layout, pad, dtype):
    """Positions 0, next to a page's end, and a million away; a token with a negative slot is rotated but not cached; the V
    pool holds the keys as projected, the K pool the rotated ones."""
    ops = _ops()
    g = torch.Generator().manual_seed(dk + dims)
    pos = [0, 1, 7, 8, 9, 63, 64, 4097, 99991]
    T, bs, base = len(pos), 8, 730.0
    rows = torch.randn(T, (H + G) * dk + pad, generator=g).to(dtype)      # further columns behind q | k, as a fused projection has
    table = ops.rotary_table(100000, dims, base, None, cuda) if dims else None
    kc, vc, _ = _pools(cuda, dtype, G, dk, bs, 6, 1)
    slots = torch.tensor([3, 47, 12, -1, 0, 20, 21, 8, 30], dtype=torch.int64, device=cuda)
    q = ops.qk_rope_cache(rows.to(cuda), H, G, dk, dk, torch.tensor(pos, dtype=torch.int32, device=cuda), table, dims, slots, kc, vc,
                          interleaved=layout == "interleaved", v_from_k=True)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    r64 = rows.to(F64)
    for t, p in enumerate(pos):
        qw = R.rotate(r64[t, :H * dk].view(H, dk), p, dims, base, layout)
        _close(q[t], qw, tol, f"query at {p}")
        s = int(slots[t])
        if s < 0:
            continue
        kw = R.rotate(r64[t, H * dk:(H + G) * dk].view(G, dk), p, dims, base, layout)
        _close(kc[s // bs, :, s % bs], kw, tol, f"key at {p}")
        assert torch.equal(vc[s // bs, :, s % bs].cpu(), rows[t, H * dk:(H + G) * dk].view(G, dk)), "values = keys as projected"
    used = {int(s) for s in slots if s >= 0}
    free = [s for s in range(6 * bs) if s not in used]
    assert bool(torch.isnan(kc.view(6, G, bs, dk).permute(0, 2, 1, 3).reshape(6 * bs, -1)[free]).all()), "no other slot is written"


def test_values_of_their_own_go_to_the_value_pool(cuda):
    ops = _ops()
    H, G, dk, dv, bs = 2, 1, 8, 12, 4
    g = torch.Generator().manual_seed(0)
    rows = torch.randn(3, (H + G) * dk + G * dv, generator=g)
    kc = torch.zeros(2, G, bs, dk, device=cuda)
    vc = torch.zeros(2, G, bs, dv, device=cuda)
    pos = torch.tensor([4, 5, 6], dtype=torch.int32, device=cuda)
    table = ops.rotary_table(16, 4, 50.0, None, cuda)
    ops.qk_rope_cache(rows.to(cuda), H, G, dk, dv, pos, table, 4, torch.tensor([0, 1, 6], dtype=torch.int64, device=cuda), kc, vc)
    assert torch.equal(vc[1, 0, 2].cpu(), rows[2, (H + G) * dk:])
    _close(kc[0, 0, 1], R.rotate(rows[1, H * dk:(H + G) * dk].to(F64), 5, 4, 50.0, "half"), 3e-6)


# ------------------------------------------------------------------------------------------------ windowed attention
def _attention_case(cuda, dtype, H, G, dk, bs, T, seed, scale_rows=0.6):
    g = torch.Generator().manual_seed(seed)
    rows = (torch.randn(T, (H + G) * dk + H, generator=g) * scale_rows).to(dtype)      # q | k | gate
    sinks = torch.randn(H, generator=g) * 1.5
    return rows, sinks


def _attention_oracle(rows, sinks, H, G, dk, scale, window, keep, dims, base, with_sink=True, with_gate=True):
    T = rows.shape[0]
    r = rows.to(F64)
    q, k = r[:, :H * dk].view(T, H, dk), r[:, H * dk:(H + G) * dk].view(T, G, dk)
    qr = torch.stack([R.rotate(q[t], t, dims, base, "half") for t in range(T)])
    kr = torch.stack([R.rotate(k[t], t, dims, base, "half") for t in range(T)])
    gates = R.sigmoid(r[:, (H + G) * dk:]) if with_gate else None
    return R.masked_attention(qr, kr, k, scale, window, keep, sinks.to(F64) if with_sink else None, gates)


def _run_attention(cuda, ops, rows, sinks, H, G, dk, bs, table, kc, vc, steps, scale, window, keep, dims, base, other=None):
    """Feed one sequence in the given portions; `other` = (rows, table, portions) of a second sequence that shares every step
    it has a portion for.  Returns the first sequence's outputs [T, H, dk]."""
    rot = ops.rotary_table(4096, dims, base, None, cuda) if dims else None
    outs, at, at2 = [], 0, 0
    for i, n in enumerate(steps):
        parts, lens, ctx, tabs = [rows[at:at + n]], [n], [at], [table]
        pos, slots = list(range(at, at + n)), [_slots(cuda, table, bs, at, at + n)]
        if other is not None and i < len(other[2]):
            m = other[2][i]
            parts.insert(0, other[0][at2:at2 + m]), lens.insert(0, m), ctx.insert(0, at2), tabs.insert(0, other[1])
            pos = list(range(at2, at2 + m)) + pos
            slots.insert(0, _slots(cuda, other[1], bs, at2, at2 + m))
            at2 += m
        x = torch.cat(parts).to(cuda)
        width = max(len(t) for t in tabs)
        tabs = [t + [0] * (width - len(t)) for t in tabs]
        q = ops.qk_rope_cache(x, H, G, dk, dk, torch.tensor(pos, dtype=torch.int32, device=cuda), rot, dims, torch.cat(slots), kc, vc,
                              v_from_k=True)
        o = ops.chunk_attention(q, kc, vc, _batch(cuda, lens, ctx, [0] * len(lens), tabs), scale, window=window, keep_first=keep,
                                sink=1.0, sink_logits=sinks.to(cuda), gate=x[:, (H + G) * dk:])
        outs.append(o[-n:])
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,dk,bs", [(4, 1, 24, 16), (2, 2, 16, 8), (3, 3, 40, 16), (4, 2, 64, 16), (8, 1, 128, 32), (12, 1, 32, 16),
                                       (1, 1, 6, 8)])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (1, 1), (9, 2), (16, 0), (17, 5), (8, 20), (64, 3), (500, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_windowed_attention_in_mixed_batches_over_shuffled_pages(cuda, H, G, dk, bs, window, keep, dtype):
    """A sequence of 150 tokens in portions of 70, 2, 1, 1, 33, 1, ..., beside a second sequence of other portions in the
    same steps: every row equals the oracle over the whole sequence (rows just after a cut, single rows, rows whose window
    starts inside an earlier portion and whose kept tokens lie pages back)."""
    ops = _ops()
    T, T2 = 150, 61
    rows, sinks = _attention_case(cuda, dtype, H, G, dk, bs, T, H + dk + window)
    rows2, _ = _attention_case(cuda, dtype, H, G, dk, bs, T2, 99)
    kc, vc, perm = _pools(cuda, dtype, G, dk, bs, 40, window + keep)
    n1 = (T + bs - 1) // bs
    table, table2 = perm[:n1], perm[n1:n1 + (T2 + bs - 1) // bs]
    steps = [70, 2, 1, 1, 33, 1, 1, 1, 40]
    got = _run_attention(cuda, ops, rows, sinks, H, G, dk, bs, table, kc, vc, steps, 0.21, window, keep, dk // 2 // 2 * 2, 300.0,
                         other=(rows2, table2, [1, 20, 1, 37, 2]))
    want = _attention_oracle(rows, sinks, H, G, dk, 0.21, window, keep, dk // 2 // 2 * 2, 300.0)
    _close(got, want, 3e-5 if dtype == torch.float32 else 2.5e-2, f"window {window} keep {keep}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk", [(2, 1, 16), (4, 2, 64)])
@pytest.mark.parametrize("loud,seen", [("window_in", True), ("window_out", False), ("kept_in", True), ("kept_out", False), ("far", True)])
@pytest.mark.parametrize("how", ["prompt", "portion", "decoded"])
def test_a_loud_key_at_every_edge(cuda, dtype, H, G, dk, loud, seen, how):
    """One key matches the query of the last row far better than any other.  It sits on the last position the window still
    holds, on the first it has dropped, on the last kept first token, on the first token that is not kept, or (without a
    window) 600 positions back, at page borders; the row is the last of a whole prompt, of a two-token portion, or a single
    decoded token.  Seen: the output is that key's value; not seen: it is not."""
    ops = _ops()
    bs, T, window, keep = 16, 704, 64, 16                      # both edges fall on page borders for the last row
    if loud == "far":
        window, keep = 0, 0
    i = T - 1
    j = {"window_in": i - window + 1, "window_out": i - window, "kept_in": keep - 1, "kept_out": keep, "far": 99}[loud]
    g = torch.Generator().manual_seed(7)
    rows = (torch.randn(T, (H + G) * dk + H, generator=g) * 0.3).to(dtype)
    rows[:, (H + G) * dk:] = 20.0                                # gates open
    rows[j, H * dk:(H + G) * dk] = 0
    rows[i, :H * dk] = 0
    for g_ in range(G):
        rows[j, H * dk + g_ * dk + dk - 1] = 30.0               # an entry that does not turn
    for h in range(H):
        rows[i, h * dk + dk - 1] = 30.0
    sinks = torch.full((H,), -20.0)
    kc, vc, perm = _pools(cuda, dtype, G, dk, bs, 50, 3)
    table = perm[:44]
    steps = {"prompt": [T], "portion": [T - 2, 2], "decoded": [T - 1, 1]}[how]
    got = _run_attention(cuda, ops, rows, sinks, H, G, dk, bs, table, kc, vc, steps, 1.0, window, keep, dk // 2, 1e4)
    value = rows[j, H * dk:(H + G) * dk].double().view(G, dk)
    for h in range(H):
        d = float((got[-1, h].double().cpu() - value[h // (H // G)]).abs().max())
        assert (d < 0.05) == seen, f"head {h}: distance {d:.3f} from the loud key's value, key {j} for row {i} ({loud}, {how})"
    qr, kr, k = _qkv(rows, H, G, dk, dk // 2, 1e4)
    want = R.masked_attention(qr[-1:], kr, k, 1.0, window, keep, sinks.to(F64), first_pos=i)
    _close(got[-1], want[0], 1e-4 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_gate_and_padding_rows(cuda, dtype):
    """A sink far above the scores takes all the weight (output ~ 0), one far below none; heads have sinks of their own; a
    closed gate silences its head only; a padding sequence (negative context) gives zero rows."""
    ops = _ops()
    H, G, dk, bs, T = 4, 2, 16, 8, 21
    rows, _ = _attention_case(cuda, dtype, H, G, dk, bs, T, 5)
    rows[:, (H + G) * dk:] = torch.tensor([9.0, -30.0, 0.0, 9.0]).to(dtype)
    sinks = torch.tensor([-30.0, -30.0, 1.0, 40.0])
    kc, vc, perm = _pools(cuda, dtype, G, dk, bs, 8, 0)
    got = _run_attention(cuda, ops, rows, sinks, H, G, dk, bs, perm[:3], kc, vc, [T], 0.3, 0, 0, 8, 100.0)
    want = _attention_oracle(rows, sinks, H, G, dk, 0.3, 0, 0, 8, 100.0)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    _close(got, want, tol)
    plain = _attention_oracle(rows, sinks, H, G, dk, 0.3, 0, 0, 8, 100.0, with_sink=False, with_gate=False)
    _close(got[:, 0], plain[:, 0], 1e-3 if dtype == torch.float32 else 2e-2, "sink far below, gate open")
    assert float(got[:, 1].abs().max()) < 1e-6 and float(got[:, 3].abs().max()) < 1e-6
    _close(got[:, 2] * 2, R.masked_attention(*_qkv(rows, H, G, dk, 8, 100.0), 0.3, sinks=sinks.to(F64))[:, 2], tol, "gate of one half")
    # a decode batch with a padding row
    q = torch.randn(2, H, dk, generator=torch.Generator().manual_seed(1)).to(dtype).to(cuda)
    b = _batch(cuda, [1, 1], [T - 1, -1], [0, 0], [perm[:3], [0, 0, 0]])
    o = ops.chunk_attention(q, kc, vc, b, 0.3, sink=1.0, sink_logits=sinks.to(cuda))
    assert bool(torch.isfinite(o[0]).all()) and float(o[1].abs().max()) == 0.0


def _qkv(rows, H, G, dk, dims, base):
    T = rows.shape[0]
    r = rows.to(F64)
    q, k = r[:, :H * dk].view(T, H, dk), r[:, H * dk:(H + G) * dk].view(T, G, dk)
    return (torch.stack([R.rotate(q[t], t, dims, base, "half") for t in range(T)]),
            torch.stack([R.rotate(k[t], t, dims, base, "half") for t in range(T)]), k)


# ------------------------------------------------------------------------------------------------ linear attention
def _lightning_oracle(rows, H, dk, dv, decay):
    T = rows.shape[0]
    a = R.silu(rows.to(F64))
    return R.decay_scan(a[:, :H * dk].view(T, H, dk), a[:, H * dk:2 * H * dk].view(T, H, dk), a[:, 2 * H * dk:].view(T, H, dv), decay)


@pytest.mark.parametrize("H,dk,dv", [(3, 16, 24), (1, 40, 12), (5, 12, 20), (2, 6, 10), (2, 128, 64), (2, 32, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fixed_decay_scan_in_portions_with_dirty_slots(cuda, H, dk, dv, dtype):
    """Two sequences in portions down to one and two tokens beside each other, their slots swapped and dirty from an earlier
    occupant; decays from 0 (no memory) to 1 (nothing forgotten)."""
    ops = _ops()
    g = torch.Generator().manual_seed(dk)
    decay = [0.0, 1.0, 0.9, 0.5, 0.999][:H] if H > 1 else [0.8]
    lens = [37, 14]
    rows = [(torch.randn(n, H * (2 * dk + dv), generator=g)).to(dtype) for n in lens]
    want = [_lightning_oracle(r, H, dk, dv, decay)[0] for r in rows]
    state = torch.full((3, H, dk, dv), 55.0, device=cuda)
    slots, cuts, at = [2, 0], [[1, 2, 17, 1, 16], [2, 1, 1, 10]], [0, 0]
    dec = torch.tensor(decay, dtype=torch.float32, device=cuda)
    for step in range(5):
        lens_now, ctx, sl, who = [], [], [], []
        for s in (0, 1):
            if step < len(cuts[s]):
                n = cuts[s][step]
                lens_now.append(n), ctx.append(at[s]), sl.append(slots[s]), who.append((s, at[s], n))
                at[s] += n
        x = torch.cat([rows[s][a:a + n] for s, a, n in who]).to(cuda)
        b = _batch(cuda, lens_now, ctx, sl)
        qkv, beta, d = ops.recur_prep(x, H, H, dk, dv, b, conv_silu=True, decay_mode=ops.DECAY_HEAD_CONST, decay_bias=dec)
        assert beta is None and tuple(d.shape) == (x.shape[0], H) and qkv.dtype == torch.float32
        o = ops.channel_scan(qkv, None, d, H, H, dk, dv, b, state, delta=False)
        off = 0
        for s, a, n in who:
            _close(o[off:off + n], want[s][a:a + n], 3e-5, f"sequence {s} at {a}")
            off += n
    assert bool((state[1] == 55.0).all())                       # a slot no sequence holds is not touched
    _close(state[2], _lightning_oracle(rows[0], H, dk, dv, decay)[1], 2e-5, "the state after the last token")


def test_a_token_far_back_stays_in_a_state_that_does_not_decay(cuda):
    """Head 0 forgets nothing: 900 single-token steps later the first token's value still answers a query that matches its
    key; head 1 (decay 0.9) has lost it."""
    ops = _ops()
    H, dk, dv, n = 2, 8, 8, 900
    state = torch.zeros(1, H, dk, dv, device=cuda)
    dec = torch.tensor([1.0, 0.9], device=cuda)
    first = torch.full((1, H * (2 * dk + dv)), -30.0)            # silu(-30) ~ 0
    for h in range(H):
        first[0, H * dk + h * dk] = 4.0                         # key entry 0
        first[0, 2 * H * dk + h * dv:2 * H * dk + (h + 1) * dv] = torch.arange(1, dv + 1, dtype=torch.float32)
    quiet = torch.full((1, H * (2 * dk + dv)), -30.0)
    ask = quiet.clone()
    for h in range(H):
        ask[0, h * dk] = 4.0
    o = None
    for t in range(n + 1):
        x = (first if t == 0 else (ask if t == n else quiet)).to(cuda)
        b = _batch(cuda, [1], [t], [0])
        qkv, _, d = ops.recur_prep(x, H, H, dk, dv, b, conv_silu=True, decay_mode=ops.DECAY_HEAD_CONST, decay_bias=dec)
        o = ops.channel_scan(qkv, None, d, H, H, dk, dv, b, state, delta=False)
    s4 = float(R.silu(torch.tensor(4.0, dtype=F64)))
    want = s4 * s4 * R.silu(torch.arange(1, dv + 1, dtype=F64))
    _close(o[0, 0], want, 1e-5, "the head that does not decay")
    assert float(o[0, 1].abs().max()) < 1e-6 * float(want.max())


@pytest.mark.parametrize("n", [36, 384, 2050])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_the_concatenated_heads_with_a_sigmoid_gate(cuda, n, dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(n)
    T = 6
    o = torch.randn(T, n, generator=g) * 4
    wide = torch.randn(T, n + 24, generator=g).to(dtype)         # the gate is a column range of a wider projection
    w = 1 + 0.3 * torch.randn(n, generator=g)
    got = ops.gated_head_norm(o.to(cuda).view(T, 1, n), wide.to(cuda)[:, 24:], w.to(cuda), 1e-5, ops.GATE_SIGMOID)
    want = R.rms_norm(o.to(F64), w.to(F64), 1e-5) * R.sigmoid(wide.to(F64)[:, 24:])
    _close(got, want, 3e-6 if dtype == torch.float32 else 1e-2)


# ------------------------------------------------------------------------------------------------ latent attention
@pytest.mark.parametrize("H,dn,dr,dims,R_", [(3, 16, 8, 8, 24), (2, 8, 16, 6, 20), (3, 6, 6, 2, 14), (4, 32, 16, 16, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_write_from_rows_of_two_buffers(cuda, H, dn, dr, dims, R_, dtype):
    """The query heads come from one product and the down-projection from another: the rotated query parts, the normed
    latent and the rotated shared key part equal the oracle's; a causal attention over them equals attention over keys and
    values rebuilt per head."""
    ops = _ops()
    g = torch.Generator().manual_seed(dn + R_)
    T, bs, base, dv, scale = 45, 8, 90.0, 12, 0.2
    qh = torch.randn(T, H * (dn + dr), generator=g).to(dtype)
    off = 16
    kv = torch.randn(T, off + R_ + dr, generator=g).to(dtype)
    nw = 1 + 0.2 * torch.randn(R_, generator=g)
    w_uk = (torch.randn(H * dn, R_, generator=g) * R_ ** -0.5).to(dtype)
    w_uv = (torch.randn(H * dv, R_, generator=g) * R_ ** -0.5).to(dtype)
    perm = torch.randperm(9, generator=g).tolist()
    table = perm[:6]
    cache = torch.full((9, bs, R_ + dr), float("nan"), dtype=dtype, device=cuda)
    rot = ops.rotary_table(64, dims, base, None, cuda)
    pos = torch.arange(T, dtype=torch.int32, device=cuda)
    qa = ops.latent_prep(qh.to(cuda), H, dn, dr, dims, R_, 0, off, nw.to(cuda), 1e-5, pos, rot, _slots(cuda, table, bs, 0, T), cache,
                         kv=kv.to(cuda))
    q64 = qh.to(F64).view(T, H, dn + dr).clone()
    c = R.rms_norm(kv.to(F64)[:, off:off + R_], nw.to(F64), 1e-5)
    kt = torch.stack([R.rotate(kv.to(F64)[t, off + R_:], t, dims, base, "interleaved") for t in range(T)])
    for t in range(T):
        q64[t, :, dn:] = R.rotate(q64[t, :, dn:], t, dims, base, "interleaved")
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    _close(qa[:, :, R_:], q64[:, :, dn:], tol, "rotated query parts")
    s = _slots(cuda, table, bs, 0, T)
    rows = cache.view(-1, R_ + dr)[s]
    _close(rows[:, :R_], c, tol, "latent")
    _close(rows[:, R_:], kt, tol, "shared key part")
    # attention in the latent space against per-head keys and values
    uk = w_uk.to(cuda).view(H, dn, R_)
    torch.bmm(qh.to(cuda).view(T, H, dn + dr)[:, :, :dn].transpose(0, 1), uk, out=qa[:, :, :R_].transpose(0, 1))
    o = ops.latent_attention(qa, cache, _batch(cuda, [T], [0], [0], [table]), R_, scale, 0)
    ov = torch.bmm(o.transpose(0, 1), w_uv.to(cuda).view(H, dv, R_).transpose(1, 2)).transpose(0, 1)
    keys, values = R.latent_keys_values(c, kt, w_uk.to(F64), w_uv.to(F64), H)
    _close(ov, R.masked_attention(q64, keys, values, scale), 3e-5 if dtype == torch.float32 else 3e-2, "attention")
