"""`bench.py --family kofadra|gatolix|tonilix|sanarax`: prefill and decode throughput of a model family at layer sizes of real models
(random weights), beside the Llama model of equal width, heads, head size and ACTIVE feed-forward width, plus the device
time of every kernel of the family with the roofline that bounds it beside the like kernel of the Llama path (Tonilix:
beside the Kofadra family, whose recurrent mixer, attention without rotation and routed experts are the closest; Sanarax:
beside the Gatolix family, whose norms on both sides, latent attention and squared-ReLU feed-forward are the closest, with
the like kernel of Kofadra and Tonilix for the sink attention and the linear attention).

Both models run through the same engine (LLMEngine.replay_step: scheduler, pools, state slots, CUDA-graph decode).
  prefill   one prompt chunk of T tokens in one step; wall clock around the step (it ends with a stream synchronize)
  decode    B sequences with `ctx` cached tokens each, one token per sequence per step; CUDA events around the graph replay
Kernel lines: CUDA events, 3 warm-ups, median of 10, L2 flushed between iterations (a 256 MiB write).
One JSON line per measurement; fractions are of the measured copy bandwidth / cuBLAS bf16 burst in MEASURED_PEAKS.json.
"""
import json
import statistics
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path[:0] = [str(ROOT / "vllm-backend-public_b200")]

SIZES = {
    # name: hidden, layers, heads, kv heads, head size, expert width, experts, chosen, vocabulary
    "2k": dict(hidden=2048, layers=4, heads=16, kv_heads=4, head_dim=128, ff=1024, experts=32, top=4, vocab=32000),
    "4k": dict(hidden=4096, layers=4, heads=32, kv_heads=8, head_dim=128, ff=1792, experts=64, top=8, vocab=32000),
}

# Gatolix: the latent geometry of the public DeepSeek-V2 family (512 + 64 numbers cached per token, heads of 128 + 64 / 128)
GATOLIX_SIZES = {
    "2k": dict(hidden=2048, layers=4, heads=16, kv_heads=4, dim=128, rot_dim=64, vdim=128, kv_rank=512, ff=1024, experts=32,
               top=4, vocab=32000, window=1024),
    "4k": dict(hidden=4096, layers=4, heads=32, kv_heads=8, dim=128, rot_dim=64, vdim=128, kv_rank=512, ff=1792, experts=64,
               top=8, vocab=32000, window=1024),
}


# Sanarax: the head geometry of SIZES, the latent geometry of GATOLIX_SIZES, a dense feed-forward of the active width; six
# layers = two of each mixer, the second three on the tensors of the first three
SANARAX_SIZES = {
    "2k": dict(hidden=2048, layers=6, heads=16, kv_heads=4, head_dim=128, ff=4096, vocab=32000, kv_rank=512, q_rank=1536,
               rot_dim=64, window=1024, keep_first=4),
    "4k": dict(hidden=4096, layers=6, heads=32, kv_heads=8, head_dim=128, ff=14336, vocab=32000, kv_rank=512, q_rank=1536,
               rot_dim=64, window=1024, keep_first=4),
}


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    d = json.loads(p.read_text()) if p.exists() else {}
    return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), ("measured" if d else "fallback")


def _emit(**kw):
    print(json.dumps(kw), flush=True)


def _engine(cfg, B, ctx, T):
    import torch
    from b200attn.engine import LLMEngine
    bs = 16
    per_seq = (ctx + 64 + bs - 1) // bs
    blocks = max(B * per_seq, (T + bs - 1) // bs + 1) + 8
    return LLMEngine(cfg, torch.device("cuda", 0), max_num_seqs=B, max_model_len=max(ctx + 64, T + 16), block_size=bs,
                     num_blocks=blocks, max_num_batched_tokens=max(T, 8192), seed=0)


def _throughput(name, cfg, B, ctx, T, steps):
    import torch
    eng = _engine(cfg, B, ctx, T)
    g = torch.Generator().manual_seed(0)
    rnd = lambda n: torch.randint(0, cfg.vocab, (n,), generator=g).tolist()          # noqa: E731
    # prefill: a fresh request of T tokens per step
    ts = []
    for i in range(5):
        toks = rnd(T)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.replay_step([(("p", i), toks, [T - 1])], [("p", i)])
        ts.append(time.perf_counter() - t0)
    pre = statistics.median(ts[2:])
    _emit(bench="prefill", model=name, tokens=T, ms=round(pre * 1e3, 3), tok_per_s=round(T / pre), timing="wall clock around one engine step")
    # decode: fill B sequences to ctx tokens (prompt chunks of up to 8192 tokens per step), then single tokens
    per_step = max(1, 8192 // ctx)
    for lo in range(0, B, per_step):
        eng.replay_step([(("d", i), rnd(ctx), []) for i in range(lo, min(B, lo + per_step))], [])
    eng.time_device = True
    for k in range(steps + 5):
        if k == 5:
            eng.stats.device_ms, eng.stats.device_steps = 0.0, 0
        eng.replay_step([(("d", i), rnd(1), []) for i in range(B)], [])
    ms = eng.stats.device_ms / max(eng.stats.device_steps, 1)
    _emit(bench="decode", model=name, batch=B, ctx=ctx, ms_per_step=round(ms, 4), tok_per_s=round(B / ms * 1e3),
          weight_gib=round(eng.model.weight_bytes() / 2 ** 30, 2), timing="CUDA events around the decode graph replay")
    eng.close()
    del eng
    torch.cuda.empty_cache()


def _time(fn, flush, iters=10):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def _kernels_kofadra(size, s, B, ctx, T):
    """Device time of the new kernels and of the like Llama kernels on the same shapes."""
    import torch
    from b200attn import ops
    dev = torch.device("cuda", 0)
    HBM, TF, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, H, G, d, F, E, top = s["hidden"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["experts"], s["top"]
    bf = torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731

    def line(kernel, phase, ms, bytes_=0, flops=0, like=None):
        gbs, tfs = bytes_ / ms / 1e6, flops / ms / 1e9
        _emit(bench="kernel", size=size, kernel=kernel, phase=phase, ms=round(ms, 4), gb_per_s=round(gbs, 1),
              tflop_per_s=round(tfs, 2), frac_hbm=round(gbs / HBM, 3), frac_bf16=round(tfs / TF, 4), peaks=src, like=like)

    S, chunk = 2, 1024
    for phase, n_seq, q_len, c in (("prefill", 1, T, 0), ("decode", B, 1, ctx)):
        rows = n_seq * q_len
        nb_seq = (c + q_len + 15) // 16
        tables = torch.arange(n_seq * nb_seq, dtype=torch.int32, device=dev).view(n_seq, nb_seq)
        batch = ops.SeqBatch(i32([i * q_len for i in range(n_seq + 1)]), i32([c] * n_seq), tables, i32(list(range(n_seq))),
                             n_seq, rows)
        # ---- residual streams + norm  |  like: fused residual add + RMS norm
        x = torch.randn(rows, S, D, device=dev)
        y = torch.randn(rows, D, device=dev).to(bf)
        mix, ow, iw, nw = torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev), torch.ones(D, device=dev)
        ms = _time(lambda: ops.hc_step(x, y, mix, ow, iw, nw, 1e-6, h_dtype=bf), flush)
        line("hc_step (2 fp32 streams)", phase, ms, bytes_=rows * D * (2 * S * 4 + 2 + 2), like="rms_norm")
        res, wn = torch.randn(rows, D, device=dev).to(bf), torch.ones(D, device=dev).to(bf)
        ms = _time(lambda: ops.rms_norm(y, wn, 1e-6, residual=res), flush)
        line("rms_norm (Llama, bf16 residual)", phase, ms, bytes_=rows * D * 2 * 4)
        # ---- attention  |  like: tcgen05 prompt attention / paged decode
        kc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        vc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        q = torch.randn(rows, H, d, device=dev).to(bf)
        ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, chunk, sink=1.0), flush)
        if phase == "prefill":
            pairs = sum(min(p % chunk, p) + 1 for p in range(T))               # visible (query, key) pairs per head
            line("chunk_attention", phase, ms, flops=4 * pairs * H * d, like="prefill_attention")
            cu, cs = i32([0, T]), i32([0])
            ms = _time(lambda: ops.prefill_attention(q, kc, vc, tables, cu, cs, total_tokens=T), flush)
            line("prefill_attention (Llama, tcgen05, causal)", phase, ms, flops=4 * (T * (T + 1) // 2) * H * d)
        else:
            seen = min((c % chunk) + 1, c + 1)
            line("chunk_attention", phase, ms, bytes_=n_seq * seen * G * 2 * d * 2, like="paged_decode")
            sl = i32([c + 1] * n_seq)
            ms = _time(lambda: ops.paged_decode(q, kc, vc, tables, sl), flush)
            line("paged_decode (Llama)", phase, ms, bytes_=n_seq * (c + 1) * G * 2 * d * 2)
        # ---- delta rule: scan (+ prep + out); no like kernel in the Llama path
        C = 2 * G * d + H * d
        proj = torch.randn(rows, C + H * d + 2 * H, device=dev).to(bf)
        conv_w, A, dtb = torch.randn(C, 4, device=dev) * 0.5, -torch.ones(H, device=dev), torch.zeros(H, device=dev)
        cstate = torch.zeros(n_seq, 3, C, dtype=bf, device=dev)
        state = torch.zeros(n_seq, H, d, d, device=dev)
        ms = _time(lambda: ops.delta_prep(proj, C + H * d, C + H * d + H, H, G, d, d, 4, conv_w, A, dtb, batch, cstate), flush)
        line("delta_prep (+ conv state)", phase, ms, bytes_=rows * (C * 2 + C * 4 + 8 * H))
        qkv, beta, decay = ops.delta_prep(proj, C + H * d, C + H * d + H, H, G, d, d, 4, conv_w, A, dtb, batch, cstate)
        ms = _time(lambda: ops.delta_scan(qkv, beta, decay, H, G, d, d, batch, state), flush)
        line("delta_scan", phase, ms, bytes_=n_seq * H * d * d * 4 * 2 + rows * (C + H * d) * 4, flops=6 * rows * H * d * d)
        o = ops.delta_scan(qkv, beta, decay, H, G, d, d, batch, state)
        ms = _time(lambda: ops.delta_out(o, proj, C, nw[:d].contiguous(), 1e-6), flush)
        line("delta_out", phase, ms, bytes_=rows * H * d * (4 + 2 + 2))
        # ---- experts  |  like: the dense gated feed-forward of equal active width (two cuBLAS GEMMs + silu_and_mul)
        h = torch.randn(rows, D, device=dev).to(bf)
        wr, rb = (torch.randn(E, D, device=dev) * D ** -0.5).to(bf), torch.zeros(E, device=dev)
        wgu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
        wg, wu = wgu[:, :F], wgu[:, F:]
        wd = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
        ms = _time(lambda: ops.moe_route(h, wr, rb, top), flush)
        line("moe_route", phase, ms, bytes_=rows * D * 2 + E * D * 2, flops=2 * rows * E * D)
        ids, wts = ops.moe_route(h, wr, rb, top)
        ms = _time(lambda: ops.moe_experts(h, ids, wts, wg, wu, wd, w_gate_up=wgu), flush)
        used = min(E, rows * top)
        path = "vendor grouped GEMM" if rows * top >= ops.MOE_GROUPED_GEMM_MIN_PAIRS else "own tiled kernels"
        line(f"moe_experts (sort + 2 grouped products + combine; {path})", phase, ms, bytes_=used * 3 * F * D * 2,
             flops=6 * rows * top * F * D, like="dense gated MLP")
        w1, w2 = (torch.randn(2 * top * F, D, device=dev) * D ** -0.5).to(bf), (torch.randn(D, top * F, device=dev) * 0.02).to(bf)
        ms = _time(lambda: torch.nn.functional.linear(ops.silu_and_mul(torch.nn.functional.linear(h, w1)), w2), flush)
        line("dense gated MLP (Llama: cuBLAS + silu_and_mul)", phase, ms, bytes_=3 * top * F * D * 2, flops=6 * rows * top * F * D)
        del wg, wu, wgu, wd, w1, w2, kc, vc, state
        torch.cuda.empty_cache()


def _kernels_gatolix(size, s, B, ctx, T):
    """Device time of the Gatolix kernels and of the like Llama kernels on the same shapes."""
    import torch
    from b200attn import ops
    dev = torch.device("cuda", 0)
    HBM, TF, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, H, G, F, E, top = s["hidden"], s["heads"], s["kv_heads"], s["ff"], s["experts"], s["top"]
    dn, dr, dv, R, W = s["dim"], s["rot_dim"], s["vdim"], s["kv_rank"], s["window"]
    Dc, d = R + dr, 128
    bf = torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731

    def line(kernel, phase, ms, bytes_=0, flops=0, like=None):
        gbs, tfs = bytes_ / ms / 1e6, flops / ms / 1e9
        _emit(bench="kernel", size=size, kernel=kernel, phase=phase, ms=round(ms, 4), gb_per_s=round(gbs, 1),
              tflop_per_s=round(tfs, 2), frac_hbm=round(gbs / HBM, 3), frac_bf16=round(tfs / TF, 4), peaks=src, like=like)

    tab = ops.rotary_table(ctx + T + 64, dr, 10000.0, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}, dev)
    for phase, n_seq, q_len, c in (("prefill", 1, T, 0), ("decode", B, 1, ctx)):
        rows = n_seq * q_len
        nb_seq = (c + q_len + 15) // 16
        tables = torch.arange(n_seq * nb_seq, dtype=torch.int32, device=dev).view(n_seq, nb_seq)
        batch = ops.SeqBatch(i32([i * q_len for i in range(n_seq + 1)]), i32([c] * n_seq), tables, None, n_seq, rows)
        # ---- norm after the sublayer + residual + norm before the next  |  like: fused residual add + RMS norm
        x = torch.randn(rows, D, device=dev)
        y = torch.randn(rows, D, device=dev).to(bf)
        ws = [torch.ones(D, device=dev) for _ in range(4)]
        ms = _time(lambda: ops.sandwich_norm(x, y, *ws, eps=1e-6, h_dtype=bf), flush)
        line("sandwich_norm (2 layer norms, fp32 residual)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2), like="rms_norm")
        res, wn = torch.randn(rows, D, device=dev).to(bf), torch.ones(D, device=dev).to(bf)
        ms = _time(lambda: ops.rms_norm(y, wn, 1e-6, residual=res), flush)
        line("rms_norm (Llama, bf16 residual)", phase, ms, bytes_=rows * D * 2 * 4)
        # ---- rotation + pool write  |  like: rotary + KV write
        P = H * (dn + dr) + H + (-H) % 8 + Dc
        proj = torch.randn(rows, P, device=dev).to(bf)
        pos = (torch.arange(rows, device=dev) % q_len + c).to(torch.int32)
        slots = (torch.arange(rows, device=dev) // q_len * (nb_seq * 16) + pos).to(torch.int64)
        cache = torch.randn(n_seq * nb_seq, 16, Dc, device=dev).to(bf)
        nw = torch.ones(R, device=dev)
        g_off = H * (dn + dr)
        ms = _time(lambda: ops.latent_prep(proj, H, dn, dr, dr, R, 0, g_off + H + (-H) % 8, nw, 1e-6, pos, tab, slots, cache), flush)
        line("latent_prep (rotation + norm + pool write)", phase, ms, bytes_=rows * (H * dr * 4 + Dc * 4), like="rope_and_cache")
        qkv = torch.randn(rows, (H + 2 * G) * d, device=dev).to(bf)
        kc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        vc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        cos_sin = torch.randn(ctx + T + 64, d, device=dev)
        ms = _time(lambda: ops.rope_and_cache(qkv, pos, cos_sin, kc, vc, slots, H), flush)
        line("rope_and_cache (Llama)", phase, ms, bytes_=rows * ((H + G) * d * 4 + 2 * G * d * 4))
        # ---- the per-head up-projections, carried to the query and to the output (library batched GEMMs)
        qa = torch.randn(rows, H, Dc, device=dev).to(bf)
        wuk = (torch.randn(H, dn, R, device=dev) * dn ** -0.5).to(bf)
        wuv = (torch.randn(H, R, dv, device=dev) * R ** -0.5).to(bf)
        qn = proj[:, :g_off].view(rows, H, dn + dr)[:, :, :dn].transpose(0, 1)
        ol = torch.randn(rows, H, R, device=dev).to(bf)
        ov = torch.empty(rows, H, dv, dtype=bf, device=dev)

        def updown():
            torch.bmm(qn, wuk, out=qa[:, :, :R].transpose(0, 1))
            torch.bmm(ol.transpose(0, 1), wuv, out=ov.transpose(0, 1))
        ms = _time(updown, flush)
        line("query absorption + value up-projection (2 cuBLAS batched GEMMs)", phase, ms, flops=2 * rows * H * R * (dn + dv),
             bytes_=H * R * (dn + dv) * 2 + rows * H * (dn + 2 * R + dv) * 2)
        # ---- attention  |  like: tcgen05 prompt attention / paged decode
        gate = proj[:, g_off:g_off + H]
        ms = _time(lambda: ops.latent_attention(qa, cache, batch, R, 0.07, W, gate=gate), flush)
        if phase == "prefill":
            pairs = sum(min(p + 1, W) for p in range(T))                       # visible (query, key) pairs per head
            line("latent_attention (window %d; portions below 256 rows)" % W, phase, ms, flops=2 * pairs * H * (Dc + R),
                 like="prefill_attention")
            # what the engine runs for a long portion instead: pool rows gathered, keys and values rebuilt per head
            cu, cs = i32([0, T]), i32([0])
            ms = _time(lambda: ops.latent_gather(cache, tables, cu, cs, 1, T), flush)
            line("latent_gather", phase, ms, bytes_=T * Dc * 4)
            lat = ops.latent_gather(cache, tables, cu, cs, 1, T)
            wukf = wuk.view(H * dn, R)
            vbuf = torch.empty(T, H, dv, dtype=bf, device=dev)

            def rebuild():
                torch.nn.functional.linear(lat[:, :R], wukf)
                torch.bmm(lat[:, :R].unsqueeze(0).expand(H, T, R), wuv, out=vbuf.transpose(0, 1))
            ms = _time(rebuild, flush)
            line("keys and values per head (2 cuBLAS GEMMs)", phase, ms, flops=2 * T * R * H * (dn + dv))
            kn = torch.nn.functional.linear(lat[:, :R], wukf).view(T, H, dn)
            qh = proj[:, :g_off].view(rows, H, dn + dr)
            ms = _time(lambda: ops.window_attention(qh[:, :, :dn], qa[:, :, R:], kn, lat[:, R:], vbuf, cu, cs, cu, cs, 1, 0.07, W,
                                                    gate=gate), flush)
            line("window_attention (per-head keys, window %d)" % W, phase, ms, flops=2 * pairs * H * (dn + dr + dv),
                 like="prefill_attention")
            q = torch.randn(rows, H, d, device=dev).to(bf)
            ms = _time(lambda: ops.prefill_attention(q, kc, vc, tables, cu, cs, total_tokens=T), flush)
            line("prefill_attention (Llama, tcgen05, causal)", phase, ms, flops=4 * (T * (T + 1) // 2) * H * d)
        else:
            seen = min(W, c + 1)
            line("latent_attention (window %d)" % W, phase, ms, bytes_=n_seq * seen * Dc * 2 + rows * H * (Dc + R) * 2,
                 flops=2 * n_seq * seen * H * (Dc + R), like="paged_decode")
            q = torch.randn(rows, H, d, device=dev).to(bf)
            sl = i32([c + 1] * n_seq)
            ms = _time(lambda: ops.paged_decode(q, kc, vc, tables, sl), flush)
            line("paged_decode (Llama)", phase, ms, bytes_=n_seq * (c + 1) * G * 2 * d * 2)
        # ---- dense feed-forward activation  |  like: silu_and_mul
        a = torch.randn(rows, top * F, device=dev).to(bf)
        ms = _time(lambda: ops.relu_sq(a), flush)
        line("relu_sq", phase, ms, bytes_=rows * top * F * 4, like="silu_and_mul")
        gu = torch.randn(rows, 2 * top * F, device=dev).to(bf)
        ms = _time(lambda: ops.silu_and_mul(gu), flush)
        line("silu_and_mul (Llama)", phase, ms, bytes_=rows * top * F * 6)
        # ---- experts  |  like: the dense gated feed-forward of equal active width (two cuBLAS GEMMs + silu_and_mul)
        h = torch.randn(rows, D, device=dev).to(bf)
        wr, rb = (torch.randn(E, D, device=dev) * D ** -0.5).to(bf), torch.zeros(E, device=dev)
        wgu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
        wg, wu = wgu[:, :F], wgu[:, F:]
        wd = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
        ms = _time(lambda: ops.moe_route(h, wr, rb, top, scoring=ops.ROUTE_SOFTMAX_ALL), flush)
        line("moe_route (softmax over all + correction)", phase, ms, bytes_=rows * D * 2 + E * D * 2, flops=2 * rows * E * D)
        ids, wts = ops.moe_route(h, wr, rb, top, scoring=ops.ROUTE_SOFTMAX_ALL)
        ms = _time(lambda: ops.moe_experts(h, ids, wts, wg, wu, wd, w_gate_up=wgu, glu=ops.GLU_CLAMPED, glu_alpha=1.702,
                                           glu_limit=7.0), flush)
        used = min(E, rows * top)
        path = "vendor grouped GEMM" if rows * top >= ops.MOE_GROUPED_GEMM_MIN_PAIRS else "own tiled kernels"
        line(f"moe_experts, bounded units (sort + 2 grouped products + combine; {path})", phase, ms,
             bytes_=used * 3 * F * D * 2, flops=6 * rows * top * F * D, like="dense gated MLP")
        w1, w2 = (torch.randn(2 * top * F, D, device=dev) * D ** -0.5).to(bf), (torch.randn(D, top * F, device=dev) * 0.02).to(bf)
        ms = _time(lambda: torch.nn.functional.linear(ops.silu_and_mul(torch.nn.functional.linear(h, w1)), w2), flush)
        line("dense gated MLP (Llama: cuBLAS + silu_and_mul)", phase, ms, bytes_=3 * top * F * D * 2, flops=6 * rows * top * F * D)
        # ---- soft cap on the sampled rows' logits
        z = torch.randn(n_seq, s["vocab"], device=dev).to(bf)
        ms = _time(lambda: ops.softcap_(z, 30.0), flush)
        line("softcap", phase, ms, bytes_=n_seq * s["vocab"] * 4)
        del wg, wu, wgu, wd, w1, w2, kc, vc, cache, qa, proj
        torch.cuda.empty_cache()


def _kernels_tonilix(size, s, B, ctx, T):
    """Device time of the Tonilix kernels and of the like Kofadra kernels on the same shapes."""
    import torch
    from b200attn import ops
    dev = torch.device("cuda", 0)
    HBM, TF, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, H, G, d, F, E, top, R = s["hidden"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["experts"], s["top"], 64
    bf = torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731

    def line(kernel, phase, ms, bytes_=0, flops=0, like=None):
        gbs, tfs = bytes_ / ms / 1e6, flops / ms / 1e9
        _emit(bench="kernel", size=size, kernel=kernel, phase=phase, ms=round(ms, 4), gb_per_s=round(gbs, 1),
              tflop_per_s=round(tfs, 2), frac_hbm=round(gbs / HBM, 3), frac_bf16=round(tfs / TF, 4), peaks=src, like=like)

    for phase, n_seq, q_len, c in (("prefill", 1, T, 0), ("decode", B, 1, ctx)):
        rows = n_seq * q_len
        nb_seq = (c + q_len + 15) // 16
        tables = torch.arange(n_seq * nb_seq, dtype=torch.int32, device=dev).view(n_seq, nb_seq)
        batch = ops.SeqBatch(i32([i * q_len for i in range(n_seq + 1)]), i32([c] * n_seq), tables, i32(list(range(n_seq))),
                             n_seq, rows)
        pos = (torch.arange(rows, device=dev) % q_len + c).to(torch.int32)
        slots = (torch.arange(rows, device=dev) // q_len * (nb_seq * 16) + pos).to(torch.int64)
        # ---- embedding with positions + norm  |  like: Kofadra's embedding into the streams
        emb = torch.randn(s["vocab"], D, device=dev).to(bf)
        tok = torch.randint(0, s["vocab"], (rows,), device=dev)
        freq, nw = ops.sinusoid_frequencies(D, device=dev), torch.ones(D, device=dev)
        ms = _time(lambda: ops.embed_sinusoid_norm(emb, tok, pos, freq, nw, 8, 1e-6), flush)
        line("embed_sinusoid_norm", phase, ms, bytes_=rows * D * (2 + 4), like="embed_streams")
        ms = _time(lambda: ops.embed_streams(emb, tok, 1, 1.0), flush)
        line("embed_streams (Kofadra, 1 stream)", phase, ms, bytes_=rows * D * (2 + 4))
        # ---- residual + scale + norm in groups (+ token shift)  |  like: Kofadra's stream step with one stream
        x, x2 = torch.randn(rows, D, device=dev), torch.empty(rows, D, device=dev)
        y = torch.randn(rows, D, device=dev).to(bf)
        ls, mu = torch.ones(D, device=dev), torch.full((D,), 0.3, device=dev)
        sst = torch.zeros(n_seq, D, device=dev)
        ms = _time(lambda: ops.group_norm_step(x, y, ls, None, nw, 8, 1e-6, h_dtype=bf), flush)
        line("group_norm_step (scale + norm in 8 groups)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2), like="hc_step")
        ms = _time(lambda: ops.group_norm_step(x, y, ls, None, nw, 8, 1e-6, h_dtype=bf, shift_mu=mu, shift_state=sst, batch=batch,
                                               x_out=x2), flush)
        line("group_norm_step (+ token shift and its state)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2), like="hc_step")
        xs = torch.randn(rows, 1, D, device=dev)
        one = torch.ones(1, device=dev)
        ms = _time(lambda: ops.hc_step(xs, y, None, one, one, nw, 1e-6, ops.NORM_RMS, h_dtype=bf), flush)
        line("hc_step (Kofadra, 1 fp32 stream, RMS)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2))
        # ---- attention: query temperature + pool write  |  like: Kofadra's per-head norm + pool write; the attention kernel is shared
        kc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        vc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        qkv = torch.randn(rows, (H + 2 * G) * d, device=dev).to(bf)
        ms = _time(lambda: ops.qk_prep_cache(qkv, H, G, d, d, slots, kc, vc, pos, 0.25, 512), flush)
        line("qk_prep_cache (query temperature + pool write)", phase, ms, bytes_=rows * (2 * H + 4 * G) * d * 2, like="qknorm_cache")
        ms = _time(lambda: ops.qknorm_cache(qkv, H, G, d, d, nw[:d].contiguous(), nw[:d].contiguous(), 1e-6, slots, kc, vc), flush)
        line("qknorm_cache (Kofadra)", phase, ms, bytes_=rows * (2 * H + 4 * G) * d * 2)
        q = torch.randn(rows, H, d, device=dev).to(bf)
        ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5), flush)
        if phase == "prefill":
            line("chunk_attention (plain causal; heads of other sizes than 128)", phase, ms, flops=4 * (T * (T + 1) // 2) * H * d,
                 like="chunk_attention (Kofadra)")
            if d == 128:
                cu, cs = i32([0, T]), i32([0])
                ms = _time(lambda: ops.prefill_attention(q, kc, vc, tables, cu, cs, total_tokens=T), flush)
                line("prefill_attention (heads of 128: the tcgen05 kernel of the Llama path)", phase, ms,
                     flops=4 * (T * (T + 1) // 2) * H * d, like="chunk_attention (Kofadra)")
            ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, 1024, sink=1.0), flush)
            pairs = sum(min(p % 1024, p) + 1 for p in range(T))
            line("chunk_attention (Kofadra: blocks of 1024, sink)", phase, ms, flops=4 * pairs * H * d)
        else:
            line("chunk_attention (plain causal; heads of other sizes than 128)", phase, ms, bytes_=n_seq * (c + 1) * G * 2 * d * 2,
                 like="chunk_attention (Kofadra)")
            if d == 128:
                sl = i32([c + 1] * n_seq)
                ms = _time(lambda: ops.paged_decode(q, kc, vc, tables, sl), flush)
                line("paged_decode (heads of 128: the kernel of the Llama path)", phase, ms, bytes_=n_seq * (c + 1) * G * 2 * d * 2,
                     like="chunk_attention (Kofadra)")
            ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, 1024, sink=1.0), flush)
            line("chunk_attention (Kofadra: blocks of 1024, sink)", phase, ms, bytes_=n_seq * ((c % 1024) + 1) * G * 2 * d * 2)
        o = torch.randn(rows, H * d, device=dev).to(bf)
        gate = torch.randn(rows, H * d, device=dev).to(bf)
        ms = _time(lambda: ops.gate_mul(o, gate, ops.GATE_SIGMOID, 1.2), flush)
        line("gate_mul (sigmoid output gate)", phase, ms, bytes_=rows * H * d * 6, like="silu_and_mul")
        gu = torch.randn(rows, 2 * H * d, device=dev).to(bf)
        ms = _time(lambda: ops.silu_and_mul(gu), flush)
        line("silu_and_mul (Llama)", phase, ms, bytes_=rows * H * d * 6)
        # ---- recurrences with a decay per channel  |  like: Kofadra's delta rule with a decay per head
        C = 2 * G * d + H * d
        proj = torch.randn(rows, C + H * d + 2 * H, device=dev).to(bf)
        a = torch.randn(rows, H * d, device=dev)
        conv_w, A, dtb = torch.randn(C, 4, device=dev) * 0.5, -torch.ones(H, device=dev), torch.zeros(H * d, device=dev)
        cstate = torch.zeros(n_seq, 3, C, dtype=bf, device=dev)
        state = torch.zeros(n_seq, H, d, d, device=dev)
        prep = lambda: ops.recur_prep(proj, H, G, d, d, batch, taps=4, conv_w=conv_w, conv_state=cstate, conv_silu=True, unit=True,  # noqa: E731
                                      q_scale=d ** -0.5, off_beta=C, decay_mode=ops.DECAY_CHANNEL_SOFTPLUS, a=a, A_log=A, decay_bias=dtb)
        ms = _time(prep, flush)
        line("recur_prep (conv + unit vectors + decay per channel)", phase, ms, bytes_=rows * (C * 2 + C * 4 + H * d * 8 + 4 * H),
             like="delta_prep")
        dth = torch.zeros(H, device=dev)
        ms = _time(lambda: ops.delta_prep(proj, C + H * d, C + H * d + H, H, G, d, d, 4, conv_w, A, dth, batch, cstate), flush)
        line("delta_prep (Kofadra, decay per head)", phase, ms, bytes_=rows * (C * 2 + C * 4 + 8 * H))
        qkv32, beta, decay = prep()
        ms = _time(lambda: ops.channel_scan(qkv32, beta, decay, H, G, d, d, batch, state, delta=True), flush)
        line("channel_scan (delta rule, decay per channel)", phase, ms, flops=8 * rows * H * d * d,
             bytes_=n_seq * H * d * d * 4 * 2 + rows * (C + 2 * H * d) * 4, like="delta_scan")
        Hr = max(H // 2, 1)
        Cr = 3 * Hr * d
        qr, dr_ = torch.randn(rows, Cr, device=dev), torch.rand(rows, Hr * d, device=dev)
        st_r = torch.zeros(n_seq, Hr, d, d, device=dev)
        ms = _time(lambda: ops.channel_scan(qr, None, dr_, Hr, Hr, d, d, batch, st_r, delta=False), flush)
        line("channel_scan (gated linear attention, half the heads)", phase, ms, flops=6 * rows * Hr * d * d,
             bytes_=n_seq * Hr * d * d * 4 * 2 + rows * (Cr + 2 * Hr * d) * 4, like="delta_scan")
        _, beta_h, decay_h = ops.delta_prep(proj, C + H * d, C + H * d + H, H, G, d, d, 4, conv_w, A, dth, batch, cstate)
        ms = _time(lambda: ops.delta_scan(qkv32, beta_h, decay_h, H, G, d, d, batch, state), flush)
        line("delta_scan (Kofadra, decay per head)", phase, ms, flops=6 * rows * H * d * d,
             bytes_=n_seq * H * d * d * 4 * 2 + rows * (C + H * d) * 4)
        o32 = torch.randn(rows, H, d, device=dev)
        ms = _time(lambda: ops.gated_head_norm(o32, gate, nw[:d].contiguous(), 1e-6, ops.GATE_SIGMOID), flush)
        line("gated_head_norm (sigmoid gate)", phase, ms, bytes_=rows * H * d * (4 + 2 + 2), like="delta_out")
        ms = _time(lambda: ops.delta_out(o32, proj, C, nw[:d].contiguous(), 1e-6), flush)
        line("delta_out (Kofadra)", phase, ms, bytes_=rows * H * d * (4 + 2 + 2))
        # ---- feed-forwards  |  like: Kofadra's router and gated experts; the Llama gated unit
        act_in = torch.randn(rows, 2 * top * F, device=dev).to(bf)
        ms = _time(lambda: ops.glu_and_mul(act_in, ops.GLU_GELU_TANH), flush)
        line("glu_and_mul (gelu_tanh)", phase, ms, bytes_=rows * top * F * 6, like="silu_and_mul")
        ms = _time(lambda: ops.silu_and_mul(act_in), flush)
        line("silu_and_mul (Llama, feed-forward width)", phase, ms, bytes_=rows * top * F * 6)
        h = torch.randn(rows, D, device=dev).to(bf)
        wr, rb = (torch.randn(E, D, device=dev) * D ** -0.5).to(bf), torch.zeros(E, device=dev)
        route = lambda: ops.moe_route(h, wr, rb, top, ops.ROUTE_SIGMOID_GROUPED, 8, 4, 2.0)          # noqa: E731
        ms = _time(route, flush)
        line("moe_route (sigmoid scores, 4 of 8 groups)", phase, ms, bytes_=rows * D * 2 + E * D * 2, flops=2 * rows * E * D, like="moe_route")
        ms = _time(lambda: ops.moe_route(h, wr, rb, top), flush)
        line("moe_route (Kofadra, softmax over the chosen)", phase, ms, bytes_=rows * D * 2 + E * D * 2, flops=2 * rows * E * D)
        ids, wts = route()
        wgu = (torch.randn(E, 2 * F, D, device=dev) * D ** -0.5).to(bf)
        wup = wgu[:, :F].contiguous()
        wd = (torch.randn(E, D, F, device=dev) * F ** -0.5).to(bf)
        used = min(E, rows * top)
        path = "vendor grouped GEMM" if rows * top >= ops.MOE_GROUPED_GEMM_MIN_PAIRS else "own tiled kernels"
        ms = _time(lambda: ops.moe_experts(h, ids, wts, None, wup, wd, glu=ops.FF_RELU_SQ), flush)
        line(f"moe_experts, ungated squared ReLU (sort + 2 grouped products + combine; {path})", phase, ms,
             bytes_=used * 2 * F * D * 2, flops=4 * rows * top * F * D, like="moe_experts (Kofadra)")
        ms = _time(lambda: ops.moe_experts(h, ids, wts, wgu[:, :F], wgu[:, F:], wd, w_gate_up=wgu), flush)
        line(f"moe_experts (Kofadra, gated; {path})", phase, ms, bytes_=used * 3 * F * D * 2, flops=6 * rows * top * F * D)
        del wgu, wup, wd, kc, vc, state, st_r, emb
        torch.cuda.empty_cache()


def _kernels_sanarax(size, s, B, ctx, T):
    """Device time of the Sanarax kernels and of the like kernels of Gatolix, Kofadra and Tonilix on the same shapes."""
    import torch
    from b200attn import ops
    dev = torch.device("cuda", 0)
    HBM, TF, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    D, H, G, d, F = s["hidden"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"]
    R, Rq, dr, W, keep = s["kv_rank"], s["q_rank"], s["rot_dim"], s["window"], s["keep_first"]
    Dc = R + dr
    bf = torch.bfloat16
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)          # noqa: E731

    def line(kernel, phase, ms, bytes_=0, flops=0, like=None):
        gbs, tfs = bytes_ / ms / 1e6, flops / ms / 1e9
        _emit(bench="kernel", size=size, kernel=kernel, phase=phase, ms=round(ms, 4), gb_per_s=round(gbs, 1),
              tflop_per_s=round(tfs, 2), frac_hbm=round(gbs / HBM, 3), frac_bf16=round(tfs / TF, 4), peaks=src, like=like)

    tab_w = ops.rotary_table(ctx + T + 64, d // 2, 1e6, None, dev)
    tab_l = ops.rotary_table(ctx + T + 64, dr, 1e4, None, dev)
    for phase, n_seq, q_len, c in (("prefill", 1, T, 0), ("decode", B, 1, ctx)):
        rows = n_seq * q_len
        nb_seq = (c + q_len + 15) // 16
        tables = torch.arange(n_seq * nb_seq, dtype=torch.int32, device=dev).view(n_seq, nb_seq)
        batch = ops.SeqBatch(i32([i * q_len for i in range(n_seq + 1)]), i32([c] * n_seq), tables, i32(list(range(n_seq))),
                             n_seq, rows)
        pos = (torch.arange(rows, device=dev) % q_len + c).to(torch.int32)
        slots = (torch.arange(rows, device=dev) // q_len * (nb_seq * 16) + pos).to(torch.int64)
        # ---- RMS norm after the sublayer + residual + RMS norm before the next  |  like: Gatolix's two layer norms
        x = torch.randn(rows, D, device=dev)
        y = torch.randn(rows, D, device=dev).to(bf)
        ws = [torch.ones(D, device=dev) for _ in range(4)]
        ms = _time(lambda: ops.sandwich_norm(x, y, ws[0], None, ws[1], None, eps=1e-6, norm_kind=ops.NORM_RMS, h_dtype=bf), flush)
        line("sandwich_norm (2 RMS norms, fp32 residual)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2), like="sandwich_norm (Gatolix)")
        ms = _time(lambda: ops.sandwich_norm(x, y, *ws, eps=1e-6, h_dtype=bf), flush)
        line("sandwich_norm (Gatolix, 2 layer norms)", phase, ms, bytes_=rows * D * (4 + 4 + 2 + 2))
        # ---- window attention: rotation + pool write  |  like: Tonilix's query temperature + pool write
        kc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        vc = torch.randn(n_seq * nb_seq, G, 16, d, device=dev).to(bf)
        qk = torch.randn(rows, (H + G) * d + H, device=dev).to(bf)
        ms = _time(lambda: ops.qk_rope_cache(qk, H, G, d, d, pos, tab_w, d // 2, slots, kc, vc, v_from_k=True), flush)
        line("qk_rope_cache (half of every head turns; values = unrotated keys)", phase, ms, bytes_=rows * (2 * H + 3 * G) * d * 2,
             like="qk_prep_cache (Tonilix)")
        qkv = torch.randn(rows, (H + 2 * G) * d, device=dev).to(bf)
        ms = _time(lambda: ops.qk_prep_cache(qkv, H, G, d, d, slots, kc, vc, pos, 0.25, 512), flush)
        line("qk_prep_cache (Tonilix)", phase, ms, bytes_=rows * (2 * H + 4 * G) * d * 2)
        # ---- the attention itself  |  like: Kofadra's mask blocks of the same size with one sink
        q = torch.randn(rows, H, d, device=dev).to(bf)
        sinks = torch.randn(H, device=dev)
        gate = qk[:, (H + G) * d:]
        ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, window=W, keep_first=keep, sink=1.0, sink_logits=sinks,
                                               gate=gate), flush)
        name = "chunk_attention (window %d + %d kept, sink per head, gate)" % (W, keep)
        if phase == "prefill":
            pairs = sum(min(p + 1, W) + max(0, min(keep, p - W + 1)) for p in range(T))
            line(name, phase, ms, flops=4 * pairs * H * d, like="chunk_attention (Kofadra)")
            ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, W, sink=1.0), flush)
            line("chunk_attention (Kofadra: blocks of %d, sink)" % W, phase, ms, flops=4 * sum(p % W + 1 for p in range(T)) * H * d)
        else:
            seen = min(c + 1, W) + max(0, min(keep, c - W + 1))
            line(name, phase, ms, bytes_=n_seq * seen * G * 2 * d * 2, like="chunk_attention (Kofadra)")
            ms = _time(lambda: ops.chunk_attention(q, kc, vc, batch, d ** -0.5, W, sink=1.0), flush)
            line("chunk_attention (Kofadra: blocks of %d, sink)" % W, phase, ms, bytes_=n_seq * (c % W + 1) * G * 2 * d * 2)
        # ---- latent attention: norm of the query latent, rotation + pool write from two buffers  |  like: Gatolix's
        P = Rq + 8 * ((H + 7) // 8) + Dc
        proj = torch.randn(rows, P, device=dev).to(bf)
        nq, nw = torch.ones(Rq, device=dev), torch.ones(R, device=dev)
        ms = _time(lambda: ops.row_norm(proj[:, :Rq], nq, 1e-6), flush)
        line("row_norm (query latent of %d)" % Rq, phase, ms, bytes_=rows * Rq * 4, like="rms_norm (Llama)")
        xq, wq = torch.randn(rows, Rq, device=dev).to(bf), torch.ones(Rq, device=dev).to(bf)
        ms = _time(lambda: ops.rms_norm(xq, wq, 1e-6), flush)
        line("rms_norm (Llama, same rows)", phase, ms, bytes_=rows * Rq * 4)
        qh = torch.randn(rows, H * (d + dr), device=dev).to(bf)
        cache = torch.randn(n_seq * nb_seq, 16, Dc, device=dev).to(bf)
        ms = _time(lambda: ops.latent_prep(qh, H, d, dr, dr, R, 0, P - Dc, nw, 1e-6, pos, tab_l, slots, cache, kv=proj), flush)
        line("latent_prep (queries and down-projection in two buffers)", phase, ms, bytes_=rows * (H * dr * 4 + Dc * 4),
             like="latent_prep (Gatolix)")
        Pg = H * (d + dr) + 8 * ((H + 7) // 8) + Dc
        pg = torch.randn(rows, Pg, device=dev).to(bf)
        ms = _time(lambda: ops.latent_prep(pg, H, d, dr, dr, R, 0, Pg - Dc, nw, 1e-6, pos, tab_l, slots, cache), flush)
        line("latent_prep (Gatolix, one buffer)", phase, ms, bytes_=rows * (H * dr * 4 + Dc * 4))
        qa = torch.randn(rows, H, Dc, device=dev).to(bf)
        lgate = proj[:, Rq:Rq + H]
        if phase == "prefill":
            # a long portion: pool rows gathered, keys and values rebuilt per head, causal attention over them
            cu, cs = i32([0, T]), i32([0])
            lat = ops.latent_gather(cache, tables, cu, cs, 1, T)
            kn = torch.randn(T, H, d, device=dev).to(bf)
            vb = torch.randn(T, H, d, device=dev).to(bf)
            q3 = qh.view(rows, H, d + dr)
            ms = _time(lambda: ops.window_attention(q3[:, :, :d], qa[:, :, R:], kn, lat[:, R:], vb, cu, cs, cu, cs, 1, 0.07, 0,
                                                    gate=lgate), flush)
            line("window_attention (per-head keys, causal)", phase, ms, flops=2 * (T * (T + 1) // 2) * H * (2 * d + dr),
                 like="window_attention (Gatolix)")
            ms = _time(lambda: ops.window_attention(q3[:, :, :d], qa[:, :, R:], kn, lat[:, R:], vb, cu, cs, cu, cs, 1, 0.07, W,
                                                    gate=lgate), flush)
            line("window_attention (Gatolix, window %d)" % W, phase, ms, flops=2 * sum(min(p + 1, W) for p in range(T)) * H * (2 * d + dr))
        else:
            ms = _time(lambda: ops.latent_attention(qa, cache, batch, R, 0.07, 0, gate=lgate), flush)
            line("latent_attention (causal)", phase, ms, bytes_=n_seq * (c + 1) * Dc * 2 + rows * H * (Dc + R) * 2,
                 flops=2 * n_seq * (c + 1) * H * (Dc + R), like="latent_attention (Gatolix)")
            ms = _time(lambda: ops.latent_attention(qa, cache, batch, R, 0.07, W, gate=lgate), flush)
            seen = min(W, c + 1)
            line("latent_attention (Gatolix, window %d)" % W, phase, ms, bytes_=n_seq * seen * Dc * 2 + rows * H * (Dc + R) * 2,
                 flops=2 * n_seq * seen * H * (Dc + R))
        # ---- linear attention with a fixed decay per head  |  like: Tonilix's gated linear attention (decay per key channel)
        C = 3 * H * d
        lp = torch.randn(rows, C + H * d, device=dev).to(bf)
        dec = torch.full((H,), 0.99, device=dev)
        prep = lambda: ops.recur_prep(lp, H, H, d, d, batch, conv_silu=True, decay_mode=ops.DECAY_HEAD_CONST, decay_bias=dec)  # noqa: E731
        ms = _time(prep, flush)
        line("recur_prep (SiLU, fixed decay)", phase, ms, bytes_=rows * (C * 2 + C * 4 + 4 * H), like="recur_prep (Tonilix)")
        a = torch.randn(rows, H * d, device=dev)
        ab = torch.zeros(H * d, device=dev)
        prep_t = lambda: ops.recur_prep(lp, H, H, d, d, batch, q_scale=d ** -0.5, decay_mode=ops.DECAY_CHANNEL_SIGMOID_POW, a=a,  # noqa: E731
                                        decay_bias=ab, tau=8.0)
        ms = _time(prep_t, flush)
        line("recur_prep (Tonilix: decay per key channel)", phase, ms, bytes_=rows * (C * 2 + C * 4 + H * d * 8))
        state = torch.zeros(n_seq, H, d, d, device=dev)
        qkv32, _, decay = prep()
        ms = _time(lambda: ops.channel_scan(qkv32, None, decay, H, H, d, d, batch, state, delta=False), flush)
        line("channel_scan (fixed decay per head)", phase, ms, flops=6 * rows * H * d * d,
             bytes_=n_seq * H * d * d * 4 * 2 + rows * (C + H * d) * 4, like="channel_scan (Tonilix)")
        _, _, decay_c = prep_t()
        ms = _time(lambda: ops.channel_scan(qkv32, None, decay_c, H, H, d, d, batch, state, delta=False), flush)
        line("channel_scan (Tonilix: decay per key channel)", phase, ms, flops=6 * rows * H * d * d,
             bytes_=n_seq * H * d * d * 4 * 2 + rows * (C + 2 * H * d) * 4)
        o32 = torch.randn(rows, H, d, device=dev)
        nrow = torch.ones(H * d, device=dev)
        ms = _time(lambda: ops.gated_head_norm(o32.view(rows, 1, H * d), lp[:, C:], nrow, 1e-6, ops.GATE_SIGMOID), flush)
        line("gated_head_norm (one norm over all heads)", phase, ms, bytes_=rows * H * d * (4 + 2 + 2), like="gated_head_norm (Tonilix)")
        ms = _time(lambda: ops.gated_head_norm(o32, lp[:, C:], nrow[:d].contiguous(), 1e-6, ops.GATE_SIGMOID), flush)
        line("gated_head_norm (Tonilix: a norm per head)", phase, ms, bytes_=rows * H * d * (4 + 2 + 2))
        # ---- feed-forward activation: the kernel Gatolix uses
        act = torch.randn(rows, F, device=dev).to(bf)
        ms = _time(lambda: ops.relu_sq(act), flush)
        line("relu_sq (shared with Gatolix)", phase, ms, bytes_=rows * F * 4, like="relu_sq")
        del kc, vc, cache, state, qkv32, lp, proj
        torch.cuda.empty_cache()


def run(family: str, sizes, steps: int, kernels: bool = True) -> None:
    import torch
    from b200attn.model import ModelConfig
    if family not in ("kofadra", "gatolix", "tonilix", "sanarax"):
        raise SystemExit(f"unknown family {family!r}")
    B, ctx, T = 64, 2560, 4096          # ctx: 2.5 mask blocks / windows of the bench geometries
    for name in sizes:
        if family == "kofadra":
            from b200attn.kofadra import bench_config
            s = SIZES[name]
            fcfg = bench_config(s["hidden"], s["layers"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["experts"],
                                s["top"], s["vocab"], name=f"kofadra-{name}")
        elif family == "tonilix":
            from b200attn.tonilix import bench_config
            s = SIZES[name]
            fcfg = bench_config(s["hidden"], s["layers"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["experts"],
                                s["top"], s["vocab"], name=f"tonilix-{name}")
        elif family == "sanarax":
            from b200attn.sanarax import bench_config
            s = SANARAX_SIZES[name]
            fcfg = bench_config(s["hidden"], s["layers"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["vocab"],
                                kv_rank=s["kv_rank"], q_rank=s["q_rank"], rot_dim=s["rot_dim"], window=s["window"],
                                keep_first=s["keep_first"], name=f"sanarax-{name}")
        else:
            from b200attn.gatolix import bench_config
            s = GATOLIX_SIZES[name]
            fcfg = bench_config(s["hidden"], s["layers"], s["heads"], s["dim"], s["rot_dim"], s["vdim"], s["kv_rank"], s["ff"],
                                s["experts"], s["top"], s["vocab"], window=s["window"], name=f"gatolix-{name}")
        lcfg = ModelConfig(f"llama-{name}", s["hidden"], s["layers"], s["heads"], s["kv_heads"], s.get("top", 1) * s["ff"],
                           s["vocab"], max_position=8192)
        _emit(bench="config", size=name, **s, **{f"{family}_params": fcfg.params}, llama_params=lcfg.params, prefill_tokens=T,
              decode_batch=B, decode_ctx=ctx, data="synthetic", dtype="bf16")
        _throughput(fcfg.name, fcfg, B, ctx, T, steps)
        if family == "tonilix":                 # the closest family at equal size: plain residual, delta and attention layers
            from b200attn.kofadra import bench_config as kofadra_config
            kcfg = kofadra_config(s["hidden"], s["layers"], s["heads"], s["kv_heads"], s["head_dim"], s["ff"], s["experts"],
                                  s["top"], s["vocab"], streams=0, name=f"kofadra-{name}")
            _throughput(kcfg.name, kcfg, B, ctx, T, steps)
        if family == "sanarax":                 # the closest family at equal size: norms on both sides, latent attention
            from b200attn.gatolix import bench_config as gatolix_config
            g = GATOLIX_SIZES[name]
            gcfg = gatolix_config(s["hidden"], s["layers"], s["heads"], s["head_dim"], s["rot_dim"], s["head_dim"], s["kv_rank"],
                                  g["ff"], g["experts"], g["top"], s["vocab"], window=s["window"], name=f"gatolix-{name}")
            _throughput(gcfg.name, gcfg, B, ctx, T, steps)
        _throughput(lcfg.name, lcfg, B, ctx, T, steps)
        if kernels:
            {"kofadra": _kernels_kofadra, "gatolix": _kernels_gatolix, "tonilix": _kernels_tonilix,
             "sanarax": _kernels_sanarax}[family](name, s, B, ctx, T)
        torch.cuda.empty_cache()
