// delta_rule.cu -- a gated delta-rule recurrent mixer over a varlen token batch with per-sequence state slots.
//
// One fused projection gives, per token, the row  [ q (G*dk) | k (G*dk) | v (H*dv) | ... ]  and three more column
// ranges for the gate inputs (b: H, a: H) and the output gate (H*dv).  The mixer then runs
//
//   b2_delta_prep          short causal depthwise convolution (taps) + SiLU over the q|k|v channels, reading the
//                          taps-1 inputs before the chunk from the sequence's state slot; q and k made unit vectors per
//                          head (q also times dk^-1/2); beta = sigmoid(b); decay = exp(-exp(A_log) * softplus(a + dt_bias)).
//                          All of it in fp32, written as fp32 rows for the scan.
//   b2_delta_conv_state    the slot's convolution tail becomes the last taps-1 inputs of the sequence.
//   b2_delta_scan          per (sequence, head): S <- decay*S;  u = beta*(v - S^T k);  S <- S + k u^T;  o = S^T q,
//                          token after token, S [dk, dv] fp32 held in registers for the whole chunk and loaded from /
//                          stored to the slot once.  A one-token chunk is the decode step: one read and one write of
//                          the state, which is its HBM roofline.
//   b2_delta_out           o / rms(o over dv) * w  * SiLU(output gate)  -> activation type, ready for the out projection.
//
// The same three stages serve other linear recurrences over a matrix state (b2_recur_prep, b2_channel_scan,
// b2_gated_head_norm): the decay may act per key channel instead of per head (decay [T, H, dk], computed in fp32 from a
// separate fp32 input a [T, H*dk]: exp(-exp(A_log[h]) softplus(a + bias)) or sigmoid(a + bias)^(1/tau)) or be one fixed
// number per head (linear attention with a constant decay: S <- lambda_h S + k v^T), the write may be
// the plain outer product k v^T instead of the delta correction (gated linear attention: S <- diag(decay) S + k v^T),
// the convolution, its activation and the unit-vector step are optional, and the output gate is SiLU or a sigmoid of
// a gate row given on its own.  With a decay per channel the decay is applied first: S <- diag(g) S; u = beta (v - S^T k).
//
// A batch is n sequences; sequence i owns rows cu_q[i] .. cu_q[i+1]-1, has ctx_start[i] tokens before them (< 0: the row
// group is padding and is skipped) and keeps its state in slot state_slot[i] (< 0: no state is read or written).  A
// sequence with ctx_start = 0 starts from a zero state whatever the slot holds, so slots need no clearing on reuse.
#include "b2_act.cuh"

namespace {

constexpr int kMaxTaps = 16;

// ------------------------------------------------------------------------------------------------- prep
// What b2_recur_prep computes beyond the convolution (see the file comment); passed by value.
struct PrepSpec {
    int H, G, dk, dv, taps;
    int act;                 // 1: SiLU after the convolution, 0: none
    int unit;                // 1: q and k heads become x / sqrt(sum x^2 + unit_eps)
    float unit_eps, q_scale;
    int off_beta;            // column of the H beta inputs in proj, < 0: no beta
    int decay_mode;          // B2_DECAY_*
    int off_a;               // B2_DECAY_HEAD_SOFTPLUS: column of the H decay inputs in proj
    const float* a;          // channel modes: fp32 [T, H*dk]
    int64_t a_stride;
    const float* A_log;      // [H] (softplus modes)
    const float* bias;       // [H] or [H*dk]
    float inv_tau;           // B2_DECAY_CHANNEL_SIGMOID_POW
};

template <typename T>
__global__ void recur_prep_kernel(const T* __restrict__ proj, int64_t proj_stride, PrepSpec sp, const float* __restrict__ conv_w,
                                  const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start,
                                  const int32_t* __restrict__ state_slot, int n_seq, const T* __restrict__ conv_state,
                                  float* __restrict__ qkv, float* __restrict__ beta, float* __restrict__ decay) {
    extern __shared__ float ch[];                    // [C] conv (+ activation) outputs of this token
    const int row = blockIdx.x;
    const int H = sp.H, G = sp.G, dk = sp.dk, dv = sp.dv, taps = sp.taps;
    const int C = 2 * G * dk + H * dv;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int li = row - cu_q[seq];
    const int ctx = ctx_start[seq];
    if (ctx < 0) return;
    const int slot = state_slot[seq];
    const T* st = (taps > 1 && slot >= 0 && ctx > 0) ? conv_state + (size_t)slot * (taps - 1) * C : nullptr;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc;
        if (taps == 1 && !conv_w) {
            acc = b2::ld(proj + (size_t)row * proj_stride + c);
        } else {
            acc = 0.f;
            for (int j = 0; j < taps; ++j) {         // input at position ctx + li - j times the tap taps-1-j
                const int l = li - j;
                float xin = 0.f;
                if (l >= 0) xin = b2::ld(proj + (size_t)(row - j) * proj_stride + c);
                else if (ctx + l >= 0 && st) xin = b2::ld(st + (size_t)(l + taps - 1) * C + c);
                acc = fmaf(conv_w[(size_t)c * taps + (taps - 1 - j)], xin, acc);
            }
        }
        ch[c] = sp.act ? b2::silu_f(acc) : acc;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float* out = qkv + (size_t)row * C;
    for (int g = wid; g < 2 * G; g += nw) {          // q heads then k heads
        const float* v = ch + (size_t)g * dk;
        float sc = g < G ? sp.q_scale : 1.f;
        if (sp.unit) {
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(v[i], v[i], ss);
            ss = b2::warp_sum(ss);
            sc *= rsqrtf(ss + sp.unit_eps);
        }
        for (int i = lane; i < dk; i += 32) out[(size_t)g * dk + i] = v[i] * sc;
    }
    for (int c = 2 * G * dk + threadIdx.x; c < C; c += blockDim.x) out[c] = ch[c];
    const T* pr = proj + (size_t)row * proj_stride;
    if (sp.off_beta >= 0)
        for (int hh = threadIdx.x; hh < H; hh += blockDim.x) beta[(size_t)row * H + hh] = b2::sigmoid_f(b2::ld(pr + sp.off_beta + hh));
    if (sp.decay_mode == B2_DECAY_HEAD_SOFTPLUS) {
        for (int hh = threadIdx.x; hh < H; hh += blockDim.x)
            decay[(size_t)row * H + hh] = expf(-expf(sp.A_log[hh]) * b2::softplus_f(b2::ld(pr + sp.off_a + hh) + sp.bias[hh]));
    } else if (sp.decay_mode == B2_DECAY_HEAD_CONST) {
        for (int hh = threadIdx.x; hh < H; hh += blockDim.x) decay[(size_t)row * H + hh] = sp.bias[hh];
    } else {
        const float* ar = sp.a + (size_t)row * sp.a_stride;
        float* dr = decay + (size_t)row * H * dk;
        for (int c = threadIdx.x; c < H * dk; c += blockDim.x) {
            const float z = ar[c] + (sp.bias ? sp.bias[c] : 0.f);
            dr[c] = sp.decay_mode == B2_DECAY_CHANNEL_SOFTPLUS ? expf(-expf(sp.A_log[c / dk]) * b2::softplus_f(z))
                                                               : expf(-b2::softplus_f(-z) * sp.inv_tau);
        }
    }
}

template <typename T>
__global__ void delta_conv_state_kernel(const T* __restrict__ proj, int64_t proj_stride, int C, int taps,
                                        const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start,
                                        const int32_t* __restrict__ state_slot, T* __restrict__ conv_state) {
    const int seq = blockIdx.x;
    const int ctx = ctx_start[seq], slot = state_slot[seq];
    if (ctx < 0 || slot < 0) return;
    const int r0 = cu_q[seq], n = cu_q[seq + 1] - r0;
    T* st = conv_state + (size_t)slot * (taps - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float win[kMaxTaps];
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i) {
            if (i < taps - 1) {
                const int l = n - (taps - 1) + i;    // chunk-local index of the input that lands in tail place i
                float v = 0.f;
                if (l >= 0) v = b2::ld(proj + (size_t)(r0 + l) * proj_stride + c);
                else if (ctx + l >= 0 && ctx > 0) v = b2::ld(st + (size_t)(l + taps - 1) * C + c);
                win[i] = v;
            }
        }
#pragma unroll
        for (int i = 0; i < kMaxTaps; ++i)
            if (i < taps - 1) b2::st(st + (size_t)i * C + c, win[i]);
    }
}

// ------------------------------------------------------------------------------------------------- scan
// One warp owns 8 columns of S; a column's dk rows are spread over 4 lanes (rows r, r+4, r+8, ...), NR rows a lane.
// lane = r * 8 + jj.  The two dot products of a token reduce over the 4 lanes of a column with two shuffles.
// CH: the decay is per key channel (decay [T, H, dk]) and is applied before the prediction; DELTA: the write is the delta
// correction beta (v - S^T k), else the plain value v.
template <int NR, bool CH, bool DELTA>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                  int H, int G, int dk, int dv, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start,
                  const int32_t* __restrict__ state_slot, float* __restrict__ state, float* __restrict__ o) {
    const int seq = blockIdx.x, hh = blockIdx.y;
    const int ctx = ctx_start[seq];
    if (ctx < 0) return;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int r = lane >> 3, jj = lane & 7;
    const int j = (blockIdx.z * 4 + wid) * 8 + jj;   // column of S
    const bool col_ok = j < dv;
    const int slot = state_slot[seq];
    const int C = 2 * G * dk + H * dv;
    const int kvh = hh / (H / G);
    const int r0 = cu_q[seq], n = cu_q[seq + 1] - r0;
    constexpr int NG = CH ? NR : 1;                  // decay values a lane holds per token
    const int gw = CH ? dk : 1;                      // decay values per (token, head)
    float S[NR];
    float* sp = slot >= 0 ? state + ((size_t)slot * H + hh) * dk * dv : nullptr;
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r + 4 * m;
        S[m] = (sp && ctx > 0 && col_ok && i < dk) ? sp[(size_t)i * dv + j] : 0.f;
    }
    const float* qrow = qkv + (size_t)r0 * C + (size_t)kvh * dk;
    const float* krow = qrow + (size_t)G * dk;
    const float* vrow = qkv + (size_t)r0 * C + (size_t)2 * G * dk + (size_t)hh * dv;
    const float* vcol = vrow + (col_ok ? j : 0);
    const float* grow = decay + ((size_t)r0 * H + hh) * gw;
    const float* brow = DELTA ? beta + (size_t)r0 * H + hh : nullptr;
    float* ocol = o + ((size_t)r0 * H + hh) * dv + (col_ok ? j : 0);
    // inputs of token t (they do not depend on S: the next token's are fetched while this one's chain runs)
    auto load = [&](int t, float (&k)[NR], float (&q)[NR], float (&g)[NG], float& be, float& v) {
#pragma unroll
        for (int m = 0; m < NR; ++m) {
            const int i = r + 4 * m;
            k[m] = i < dk ? krow[(size_t)t * C + i] : 0.f;
            q[m] = i < dk ? qrow[(size_t)t * C + i] : 0.f;
            if (CH) g[m] = i < dk ? grow[(size_t)t * H * gw + i] : 0.f;
        }
        if (!CH) g[0] = grow[(size_t)t * H];
        be = DELTA ? brow[(size_t)t * H] : 1.f;
        v = col_ok ? vcol[(size_t)t * C] : 0.f;
    };
    auto step = [&](int t, const float (&k)[NR], const float (&q)[NR], const float (&g)[NG], float be, float v) {
        if (CH) {
#pragma unroll
            for (int m = 0; m < NR; ++m) S[m] *= g[m];
        }
        float u = v;
        if (DELTA) {
            float pr[4] = {0.f, 0.f, 0.f, 0.f};        // independent partial sums: the chain is NR / 4 deep
#pragma unroll
            for (int m = 0; m < NR; ++m) pr[m & 3] = fmaf(S[m], k[m], pr[m & 3]);
            float pred = (pr[0] + pr[1]) + (pr[2] + pr[3]);
            pred += __shfl_xor_sync(0xffffffffu, pred, 8);
            pred += __shfl_xor_sync(0xffffffffu, pred, 16);
            u = be * (v - (CH ? pred : g[0] * pred));
        }
        float ac[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int m = 0; m < NR; ++m) {
            S[m] = fmaf(k[m], u, CH ? S[m] : g[0] * S[m]);
            ac[m & 3] = fmaf(S[m], q[m], ac[m & 3]);
        }
        float acc = (ac[0] + ac[1]) + (ac[2] + ac[3]);
        acc += __shfl_xor_sync(0xffffffffu, acc, 8);
        acc += __shfl_xor_sync(0xffffffffu, acc, 16);
        if (r == 0 && col_ok) ocol[(size_t)t * H * dv] = acc;
    };
    float ka[NR], qa[NR], ga[NG], ba, va;
    if (NR <= 32 && !CH) {
        float kb[NR], qb[NR], gb[NG], bb, vb;
        if (n > 0) load(0, ka, qa, ga, ba, va);
        for (int t = 0; t < n; t += 2) {
            if (t + 1 < n) load(t + 1, kb, qb, gb, bb, vb);
            step(t, ka, qa, ga, ba, va);
            if (t + 1 < n) {
                if (t + 2 < n) load(t + 2, ka, qa, ga, ba, va);
                step(t + 1, kb, qb, gb, bb, vb);
            }
        }
    } else {
        for (int t = 0; t < n; ++t) {
            load(t, ka, qa, ga, ba, va);
            step(t, ka, qa, ga, ba, va);
        }
    }
    if (sp && col_ok) {
#pragma unroll
        for (int m = 0; m < NR; ++m) {
            const int i = r + 4 * m;
            if (i < dk) sp[(size_t)i * dv + j] = S[m];
        }
    }
}

// The same scan with the inputs of TT tokens at a time staged in shared memory by cp.async, two stages deep: the chain
// of a token then only touches registers and broadcast shared-memory reads, and the next tile's global loads are in
// flight while it runs (with per-token global loads the chain waited an L2 round trip per token).  Needs 16-byte
// aligned rows: dk, dv and the row length multiples of 4 floats.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(b2::smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(b2::smem_u32(dst)), "l"(src) : "memory");
}

// R lanes share a column of S (R = 4: eight columns a warp, full 32-byte sectors when the state streams through in a
// decode step; R = 8: four columns a warp, half the work per lane on the per-token chain of a long chunk).  A lane owns
// the NR consecutive rows r*NR .. r*NR+NR-1, so its k and q values are 16-byte shared-memory reads; rows of the staged
// k / q are padded by four floats per lane group to spread the banks.  FULL: dk == R*NR, no row predicates.
template <int NR, int R, int TT, bool FULL, bool CH, bool DELTA>
__global__ void __launch_bounds__(128)
delta_scan_staged_kernel(const float* __restrict__ qkv, const float* __restrict__ beta, const float* __restrict__ decay,
                         int H, int G, int dk, int dv, const int32_t* __restrict__ cu_q,
                         const int32_t* __restrict__ ctx_start, const int32_t* __restrict__ state_slot,
                         float* __restrict__ state, float* __restrict__ o) {
    constexpr int CW = 32 / R;                       // columns per warp
    constexpr int CB = 4 * CW;                       // columns per CTA
    constexpr int LDR = NR + 4;                      // padded row group
    constexpr int KQ = R * LDR;                      // floats of one token's staged k (or q)
    extern __shared__ __align__(16) float scan_sm[];
    const int seq = blockIdx.x, hh = blockIdx.y;
    const int ctx = ctx_start[seq];
    if (ctx < 0) return;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int r = lane / CW, jj = lane % CW;
    const int j0 = blockIdx.z * CB;
    const int jl = wid * CW + jj, j = j0 + jl;       // column of S (local, global)
    const bool col_ok = j < dv;
    const int slot = state_slot[seq];
    const int C = 2 * G * dk + H * dv;
    const int kvh = hh / (H / G);
    const int r0 = cu_q[seq], n = cu_q[seq + 1] - r0;
    // stage layout: k [TT][KQ] | q [TT][KQ] | decay per channel [TT][KQ] (CH) | v [TT][CB] | decay [TT] | beta [TT]
    constexpr int NKQ = CH ? 3 : 2;
    constexpr int stage_floats = TT * (NKQ * KQ + CB + 2);
    const int gw = CH ? dk : 1;                      // decay values per (token, head)
    float S[NR];
    float* sp = slot >= 0 ? state + ((size_t)slot * H + hh) * dk * dv : nullptr;
#pragma unroll
    for (int m = 0; m < NR; ++m) {
        const int i = r * NR + m;
        S[m] = (sp && ctx > 0 && col_ok && (FULL || i < dk)) ? sp[(size_t)i * dv + j] : 0.f;
    }
    const float* qrow = qkv + (size_t)r0 * C + (size_t)kvh * dk;
    const float* krow = qrow + (size_t)G * dk;
    const float* vrow = qkv + (size_t)r0 * C + (size_t)2 * G * dk + (size_t)hh * dv + j0;
    const float* grow = decay + ((size_t)r0 * H + hh) * gw;
    const float* brow = DELTA ? beta + (size_t)r0 * H + hh : nullptr;
    float* ocol = o + ((size_t)r0 * H + hh) * dv + (col_ok ? j : 0);
    const int vcols = min(CB, dv - j0);              // a multiple of 4
    auto issue = [&](int tile, int buf) {
        float* ks = scan_sm + (size_t)buf * stage_floats;
        float* qs = ks + TT * KQ;
        float* gc = qs + TT * KQ;
        float* vs = ks + NKQ * TT * KQ;
        float* gs = vs + TT * CB;
        float* bs_ = gs + TT;
        const int t0 = tile * TT, nt = min(TT, n - t0);
        const int per = dk / 4;
        for (int idx = tid; idx < nt * per; idx += 128) {
            const int tt = idx / per, c = (idx % per) * 4;
            const int dst = tt * KQ + (c / NR) * LDR + c % NR;
            cp_async16(ks + dst, krow + (size_t)(t0 + tt) * C + c);
            cp_async16(qs + dst, qrow + (size_t)(t0 + tt) * C + c);
            if (CH) cp_async16(gc + dst, grow + (size_t)(t0 + tt) * H * gw + c);
        }
        for (int idx = tid; idx < nt * (CB / 4); idx += 128) {
            const int tt = idx / (CB / 4), c = (idx % (CB / 4)) * 4;
            if (c < vcols) cp_async16(vs + tt * CB + c, vrow + (size_t)(t0 + tt) * C + c);
        }
        if (tid < nt) {
            if (!CH) cp_async4(gs + tid, grow + (size_t)(t0 + tid) * H);
            if (DELTA) cp_async4(bs_ + tid, brow + (size_t)(t0 + tid) * H);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int ntiles = (n + TT - 1) / TT;
    if (ntiles > 0) issue(0, 0);
    for (int tile = 0; tile < ntiles; ++tile) {
        const int buf = tile & 1;
        if (tile + 1 < ntiles) {
            issue(tile + 1, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* ks = scan_sm + (size_t)buf * stage_floats;
        const float* qs = ks + TT * KQ;
        const float* gc = qs + TT * KQ;
        const float* vs = ks + NKQ * TT * KQ;
        const float* gs = vs + TT * CB;
        const float* bs_ = gs + TT;
        const int t0 = tile * TT, nt = min(TT, n - t0);
        for (int tt = 0; tt < nt; ++tt) {
            const float g = CH ? 1.f : gs[tt], be = DELTA ? bs_[tt] : 1.f;
            const float v = col_ok ? vs[tt * CB + jl] : 0.f;
            float kv[NR], qv[NR];
#pragma unroll
            for (int m = 0; m < NR; m += 4) {
                const float4 a = *reinterpret_cast<const float4*>(ks + tt * KQ + r * LDR + m);
                const float4 c = *reinterpret_cast<const float4*>(qs + tt * KQ + r * LDR + m);
                kv[m] = a.x; kv[m + 1] = a.y; kv[m + 2] = a.z; kv[m + 3] = a.w;
                qv[m] = c.x; qv[m + 1] = c.y; qv[m + 2] = c.z; qv[m + 3] = c.w;
            }
            if (!FULL) {
#pragma unroll
                for (int m = 0; m < NR; ++m)
                    if (r * NR + m >= dk) kv[m] = qv[m] = 0.f;      // rows past dk: stale shared memory
            }
            if (CH) {                                // the decay per channel comes first (stale rows hold S = 0, k = 0)
#pragma unroll
                for (int m = 0; m < NR; m += 4) {
                    const float4 d = *reinterpret_cast<const float4*>(gc + tt * KQ + r * LDR + m);
                    S[m] *= d.x; S[m + 1] *= d.y; S[m + 2] *= d.z; S[m + 3] *= d.w;
                }
                if (!FULL) {
#pragma unroll
                    for (int m = 0; m < NR; ++m)
                        if (r * NR + m >= dk) S[m] = 0.f;
                }
            }
            float u = v;
            if (DELTA) {
                float pr[4] = {0.f, 0.f, 0.f, 0.f};  // independent partial sums: the chain is NR / 4 deep
#pragma unroll
                for (int m = 0; m < NR; ++m) pr[m & 3] = fmaf(S[m], kv[m], pr[m & 3]);
                float pred = (pr[0] + pr[1]) + (pr[2] + pr[3]);
#pragma unroll
                for (int x = CW; x < 32; x <<= 1) pred += __shfl_xor_sync(0xffffffffu, pred, x);
                u = be * (v - g * pred);
            }
            float ac[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int m = 0; m < NR; ++m) {
                S[m] = fmaf(kv[m], u, g * S[m]);
                ac[m & 3] = fmaf(S[m], qv[m], ac[m & 3]);
            }
            float acc = (ac[0] + ac[1]) + (ac[2] + ac[3]);
#pragma unroll
            for (int x = CW; x < 32; x <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
            if (r == 0 && col_ok) ocol[(size_t)(t0 + tt) * H * dv] = acc;
        }
        __syncthreads();                             // the stage is free for the tile after next
    }
    if (sp && col_ok) {
#pragma unroll
        for (int m = 0; m < NR; ++m) {
            const int i = r * NR + m;
            if (FULL || i < dk) sp[(size_t)i * dv + j] = S[m];
        }
    }
}

template <typename T>
__global__ void gated_head_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t gate_stride, int gate_kind,
                                       int H, int dv, const float* __restrict__ norm_w, float eps, float out_scale,
                                       T* __restrict__ out, int64_t out_stride, int rows) {
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);    // (row, head)
    if (item >= rows * H) return;
    const int row = item / H, hh = item % H;
    const float* ov = o + (size_t)item * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(ov[i], ov[i], ss);
    const float inv = rsqrtf(b2::warp_sum(ss) / (float)dv + eps);
    const T* g = gate + (size_t)row * gate_stride + (size_t)hh * dv;
    T* dst = out + (size_t)row * out_stride + (size_t)hh * dv;
    for (int i = lane; i < dv; i += 32) {
        const float z = b2::ld(g + i);
        const float gv = gate_kind == B2_GATE_SIGMOID ? b2::sigmoid_f(z) : b2::silu_f(z);
        b2::st(dst + i, ov[i] * inv * norm_w[i] * gv * out_scale);
    }
}

// The same for wide rows (a norm over all the heads of a token at once is one "head" of H * dv entries): a CTA per
// (row, head), four entries a thread per access when the sizes and addresses allow.
template <typename T, int W>
__global__ void __launch_bounds__(256)
gated_row_norm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t gate_stride, int gate_kind, int H, int dv,
                      const float* __restrict__ norm_w, float eps, float out_scale, T* __restrict__ out, int64_t out_stride) {
    __shared__ float red[33];
    const int row = blockIdx.x / H, hh = blockIdx.x % H;
    const float* ov = o + (size_t)blockIdx.x * dv;
    const int step = blockDim.x * W;
    float ss = 0.f;
    for (int i = threadIdx.x * W; i < dv; i += step) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (W == 4) b2::ld4(ov + i, v); else v[0] = ov[i];
#pragma unroll
        for (int c = 0; c < W; ++c) ss = fmaf(v[c], v[c], ss);
    }
    const float inv = rsqrtf(b2::block_sum(ss, red) / (float)dv + eps) * out_scale;
    const T* g = gate + (size_t)row * gate_stride + (size_t)hh * dv;
    T* dst = out + (size_t)row * out_stride + (size_t)hh * dv;
    for (int i = threadIdx.x * W; i < dv; i += step) {
        float v[4] = {0.f, 0.f, 0.f, 0.f}, z[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        if (W == 4) { b2::ld4(ov + i, v); b2::ld4(g + i, z); b2::ld4(norm_w + i, w); }
        else { v[0] = ov[i]; z[0] = b2::ld(g + i); w[0] = norm_w[i]; }
#pragma unroll
        for (int c = 0; c < W; ++c) v[c] *= inv * w[c] * (gate_kind == B2_GATE_SIGMOID ? b2::sigmoid_f(z[c]) : b2::silu_f(z[c]));
        if (W == 4) b2::st4(dst + i, v); else b2::st(dst + i, v[0]);
    }
}

template <bool CH, bool DELTA>
int launch_scan(const float* qkv, const float* beta, const float* decay, int total_rows, int H, int G, int dk, int dv,
                const int32_t* cu_q, const int32_t* ctx_start, const int32_t* state_slot, int n_seq, float* state, float* o,
                cudaStream_t st) {
    const bool staged = dk % 4 == 0 && dv % 4 == 0 && dk <= 256 && b2_aligned16(qkv) &&      // rows of 2*G*dk + H*dv floats stay aligned
                        (!CH || b2_aligned16(decay));
    if (!staged) {
        const dim3 grid(n_seq, H, (dv + 31) / 32);
#define B2_SCAN_PLAIN(NR) delta_scan_kernel<NR, CH, DELTA><<<grid, 128, 0, st>>>(qkv, beta, decay, H, G, dk, dv, cu_q, ctx_start, state_slot, state, o)
        if (dk <= 32) B2_SCAN_PLAIN(8);
        else if (dk <= 64) B2_SCAN_PLAIN(16);
        else if (dk <= 128) B2_SCAN_PLAIN(32);
        else if (dk <= 256) B2_SCAN_PLAIN(64);
        else B2_SCAN_PLAIN(128);
#undef B2_SCAN_PLAIN
        B2_CUDA_OK(cudaGetLastError());
        return B2_OK;
    }
#define B2_SCAN(NR, R, TT)                                                                                                 \
    do {                                                                                                                   \
        const dim3 grid(n_seq, H, (dv + 128 / R - 1) / (128 / R));                                                         \
        const size_t smem = (size_t)2 * TT * ((CH ? 3 : 2) * R * (NR + 4) + 128 / R + 2) * sizeof(float);                  \
        if (dk == R * NR) {                                                                                                \
            auto kern = delta_scan_staged_kernel<NR, R, TT, true, CH, DELTA>;                                              \
            if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            kern<<<grid, 128, smem, st>>>(qkv, beta, decay, H, G, dk, dv, cu_q, ctx_start, state_slot, state, o);           \
        } else {                                                                                                           \
            auto kern = delta_scan_staged_kernel<NR, R, TT, false, CH, DELTA>;                                             \
            if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            kern<<<grid, 128, smem, st>>>(qkv, beta, decay, H, G, dk, dv, cu_q, ctx_start, state_slot, state, o);           \
        }                                                                                                                  \
    } while (0)
    // chunks of several tokens: the per-token chain dominates, eight lanes a column; single tokens: the state streams
    // through once, four lanes a column keep whole sectors
    if (total_rows > 2 * n_seq) {
        if (dk <= 32) B2_SCAN(4, 8, 16);
        else if (dk <= 64) B2_SCAN(8, 8, 16);
        else if (dk <= 128) B2_SCAN(16, 8, 16);
        else B2_SCAN(32, 8, 8);
    } else {
        if (dk <= 32) B2_SCAN(8, 4, 16);
        else if (dk <= 64) B2_SCAN(16, 4, 16);
        else if (dk <= 128) B2_SCAN(32, 4, 16);
        else B2_SCAN(64, 4, 8);
    }
#undef B2_SCAN
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

template <typename A>
int launch_prep(const void* proj, int64_t proj_stride, const PrepSpec& sp, int T, const float* conv_w, const int32_t* cu_q,
                const int32_t* ctx_start, const int32_t* state_slot, int n_seq, void* conv_state, float* qkv, float* beta,
                float* decay, cudaStream_t st) {
    const int C = 2 * sp.G * sp.dk + sp.H * sp.dv;
    const size_t smem = (size_t)C * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "recurrence prep: %d channels do not fit shared memory", C);
    auto kern = recur_prep_kernel<A>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<T, 256, smem, st>>>(static_cast<const A*>(proj), proj_stride, sp, conv_w, cu_q, ctx_start, state_slot, n_seq,
                               static_cast<const A*>(conv_state), qkv, beta, decay);
    B2_CUDA_OK(cudaGetLastError());
    if (sp.taps > 1) {
        const int by = (C + 255) / 256;
        delta_conv_state_kernel<A><<<dim3(n_seq, by), 256, 0, st>>>(static_cast<const A*>(proj), proj_stride, C, sp.taps, cu_q,
                                                                   ctx_start, state_slot, static_cast<A*>(conv_state));
        B2_CUDA_OK(cudaGetLastError());
    }
    return B2_OK;
}

}  // namespace

extern "C" int b2_delta_prep(const void* proj, int64_t proj_stride, int off_b, int off_a, int act_dtype, int T, int H,
                             int G, int dk, int dv, int taps, const float* conv_w, const float* A_log,
                             const float* dt_bias, const int32_t* cu_q, const int32_t* ctx_start,
                             const int32_t* state_slot, int n_seq, void* conv_state, float* qkv, float* beta, float* decay,
                             void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && taps >= 1 && taps <= kMaxTaps, B2_EINVAL,
               "delta_prep: bad sizes H=%d G=%d dk=%d dv=%d taps=%d", H, G, dk, dv, taps);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(proj && conv_w && A_log && dt_bias && cu_q && ctx_start && state_slot && qkv && beta && decay, B2_EINVAL,
               "delta_prep: null pointer");
    B2_REQUIRE(conv_state || taps == 1, B2_EINVAL, "delta_prep: a convolution of %d taps needs its state", taps);
    PrepSpec sp{H, G, dk, dv, taps, 1, 1, 1e-6f, 1.f / sqrtf((float)dk), off_b, B2_DECAY_HEAD_SOFTPLUS, off_a, nullptr, 0, A_log,
                dt_bias, 0.f};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = B2_OK;
    B2_DISPATCH_ACT(act_dtype, A, rc = launch_prep<A>(proj, proj_stride, sp, T, conv_w, cu_q, ctx_start, state_slot, n_seq,
                                                      conv_state, qkv, beta, decay, st));
    return rc;
}

extern "C" int b2_recur_prep(const void* proj, int64_t proj_stride, int act_dtype, int T, int H, int G, int dk, int dv,
                             int taps, const float* conv_w, int conv_silu, int unit, float unit_eps, float q_scale,
                             int off_beta, int decay_mode, int off_a, const float* a, int64_t a_stride, const float* A_log,
                             const float* decay_bias, float tau, const int32_t* cu_q, const int32_t* ctx_start,
                             const int32_t* state_slot, int n_seq, void* conv_state, float* qkv, float* beta, float* decay,
                             void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && taps >= 1 && taps <= kMaxTaps, B2_EINVAL,
               "recur_prep: bad sizes H=%d G=%d dk=%d dv=%d taps=%d", H, G, dk, dv, taps);
    B2_REQUIRE(decay_mode == B2_DECAY_HEAD_SOFTPLUS || decay_mode == B2_DECAY_CHANNEL_SOFTPLUS ||
               decay_mode == B2_DECAY_CHANNEL_SIGMOID_POW || decay_mode == B2_DECAY_HEAD_CONST, B2_EINVAL,
               "recur_prep: unknown decay mode %d", decay_mode);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(proj && cu_q && ctx_start && state_slot && qkv && decay, B2_EINVAL, "recur_prep: null pointer");
    B2_REQUIRE(conv_w || taps == 1, B2_EINVAL, "recur_prep: a convolution of %d taps needs its weights", taps);
    B2_REQUIRE(conv_state || taps == 1, B2_EINVAL, "recur_prep: a convolution of %d taps needs its state", taps);
    B2_REQUIRE(off_beta < 0 || beta, B2_EINVAL, "recur_prep: beta columns without an output");
    if (decay_mode == B2_DECAY_HEAD_SOFTPLUS) B2_REQUIRE(A_log && decay_bias && off_a >= 0, B2_EINVAL, "recur_prep: decay inputs missing");
    else if (decay_mode == B2_DECAY_HEAD_CONST) B2_REQUIRE(decay_bias, B2_EINVAL, "recur_prep: the decay constants are missing");
    else B2_REQUIRE(a && a_stride >= (int64_t)H * dk, B2_EINVAL, "recur_prep: the decay input per channel is missing");
    if (decay_mode == B2_DECAY_CHANNEL_SOFTPLUS) B2_REQUIRE(A_log, B2_EINVAL, "recur_prep: A_log missing");
    if (decay_mode == B2_DECAY_CHANNEL_SIGMOID_POW) B2_REQUIRE(tau > 0.f, B2_EINVAL, "recur_prep: tau must be positive");
    PrepSpec sp{H, G, dk, dv, taps, conv_silu ? 1 : 0, unit ? 1 : 0, unit_eps, q_scale, off_beta, decay_mode, off_a, a, a_stride,
                A_log, decay_bias, decay_mode == B2_DECAY_CHANNEL_SIGMOID_POW ? 1.f / tau : 0.f};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = B2_OK;
    B2_DISPATCH_ACT(act_dtype, A, rc = launch_prep<A>(proj, proj_stride, sp, T, conv_w, cu_q, ctx_start, state_slot, n_seq,
                                                      conv_state, qkv, beta, decay, st));
    return rc;
}

extern "C" int b2_delta_scan(const float* qkv, const float* beta, const float* decay, int total_rows, int H, int G, int dk,
                             int dv, const int32_t* cu_q, const int32_t* ctx_start, const int32_t* state_slot, int n_seq,
                             float* state, float* o, void* stream) {
    return b2_channel_scan(qkv, beta, decay, total_rows, H, G, dk, dv, 0, 1, cu_q, ctx_start, state_slot, n_seq, state, o, stream);
}

extern "C" int b2_channel_scan(const float* qkv, const float* beta, const float* decay, int total_rows, int H, int G, int dk,
                               int dv, int decay_per_channel, int delta, const int32_t* cu_q, const int32_t* ctx_start,
                               const int32_t* state_slot, int n_seq, float* state, float* o, void* stream) {
    B2_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0, B2_EINVAL, "recurrence scan: bad sizes");
    B2_REQUIRE(dk <= 512, B2_EUNSUPPORTED, "recurrence scan: key size %d above 512", dk);
    if (n_seq == 0) return B2_OK;
    B2_REQUIRE(qkv && decay && cu_q && ctx_start && state_slot && state && o && (beta || !delta), B2_EINVAL,
               "recurrence scan: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B2_SCAN_ARGS qkv, beta, decay, total_rows, H, G, dk, dv, cu_q, ctx_start, state_slot, n_seq, state, o, st
    if (decay_per_channel) return delta ? launch_scan<true, true>(B2_SCAN_ARGS) : launch_scan<true, false>(B2_SCAN_ARGS);
    return delta ? launch_scan<false, true>(B2_SCAN_ARGS) : launch_scan<false, false>(B2_SCAN_ARGS);
#undef B2_SCAN_ARGS
}

extern "C" int b2_delta_out(const float* o, const void* proj, int64_t proj_stride, int off_g, int act_dtype, int T, int H,
                            int dv, const float* norm_w, float eps, void* out, int64_t out_stride, void* stream) {
    B2_REQUIRE(off_g >= 0, B2_EINVAL, "delta_out: bad gate column");
    const size_t esz = act_dtype == B2_ACT_BF16 ? 2 : 4;
    return b2_gated_head_norm(o, proj ? static_cast<const char*>(proj) + (size_t)off_g * esz : nullptr, proj_stride, B2_GATE_SILU,
                              act_dtype, T, H, dv, norm_w, eps, 1.f, out, out_stride, stream);
}

extern "C" int b2_gated_head_norm(const float* o, const void* gate, int64_t gate_stride, int gate_kind, int act_dtype, int T,
                                  int H, int dv, const float* norm_w, float eps, float out_scale, void* out,
                                  int64_t out_stride, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && dv > 0, B2_EINVAL, "gated_head_norm: bad sizes");
    B2_REQUIRE(gate_kind == B2_GATE_SILU || gate_kind == B2_GATE_SIGMOID, B2_EINVAL, "gated_head_norm: unknown gate %d", gate_kind);
    if (T == 0) return B2_OK;
    B2_REQUIRE(o && gate && norm_w && out, B2_EINVAL, "gated_head_norm: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dv > 512) {                                  // wide rows: a CTA per (row, head) instead of a warp
        const size_t esz = act_dtype == B2_ACT_BF16 ? 2 : 4;
        const bool vec = dv % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 && b2_aligned16(o) && b2_aligned16(norm_w) &&
                         reinterpret_cast<uintptr_t>(gate) % (4 * esz) == 0 && reinterpret_cast<uintptr_t>(out) % (4 * esz) == 0;
        B2_DISPATCH_ACT(act_dtype, A, {
            if (vec)
                gated_row_norm_kernel<A, 4><<<T * H, 256, 0, st>>>(o, static_cast<const A*>(gate), gate_stride, gate_kind, H, dv,
                                                                  norm_w, eps, out_scale, static_cast<A*>(out), out_stride);
            else
                gated_row_norm_kernel<A, 1><<<T * H, 256, 0, st>>>(o, static_cast<const A*>(gate), gate_stride, gate_kind, H, dv,
                                                                  norm_w, eps, out_scale, static_cast<A*>(out), out_stride);
        });
        B2_CUDA_OK(cudaGetLastError());
        return B2_OK;
    }
    const int items = T * H, blocks = (items + 7) / 8;
    B2_DISPATCH_ACT(act_dtype, A, (gated_head_norm_kernel<A><<<blocks, 256, 0, st>>>(o, static_cast<const A*>(gate), gate_stride,
                                                                                    gate_kind, H, dv, norm_w, eps, out_scale,
                                                                                    static_cast<A*>(out), out_stride, T)));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
