// moe.cu -- a routed mixture of gated feed-forward experts over a token batch.
//
//   b2_moe_route     z = W_r h in fp32 (one warp per token).  B2_ROUTE_TOPK_SOFTMAX: the `top` largest of z + b (lowest index
//                    wins a tie), weights = softmax over the chosen logits only.  B2_ROUTE_SOFTMAX_ALL: s = softmax(z) over
//                    all experts, the `top` largest of s + b are chosen, weights = their s (not renormalised).
//                    B2_ROUTE_SIGMOID_GROUPED: s = sigmoid(z); the choice looks at c = s + b; the experts form `n_groups` equal
//                    groups of neighbours, a group's score is the sum of its two largest c, and only experts of the
//                    `keep_groups` best groups can be chosen (the others count as -inf); weights = the chosen s divided by
//                    their sum (+ 1e-20), times `weight_scale`.  (b2_moe_route_ex / b2_moe_select_ex carry the three
//                    parameters; n_groups = 1 is the ungrouped case.)
//   b2_moe_select    the same choice from fp32 logits computed elsewhere (a library GEMM over a prompt batch).
//   b2_moe_align     counting sort of the T*top (token, choice) pairs by expert into row tiles of kMoeBM rows: every tile
//                    belongs to one expert, experts are padded to a tile boundary with -1.  Entirely on the device (no host
//                    read of the counts), so the step stays capturable in a CUDA graph and never waits for the GPU.
//   b2_moe_gate_up   per tile: act = glu(h W_gate[e]^T, h W_up[e]^T), rows gathered through the sorted list.  glu(g, u) is
//                    SiLU(g) * u (B2_GLU_SILU) or, with g' = min(g, limit) and u' = clamp(u, -limit, limit),
//                    g' * sigmoid(alpha * g') * (u' + 1) (B2_GLU_CLAMPED).  B2_FF_RELU_SQ: experts without a gate,
//                    act = max(h W_up[e]^T, 0)^2 (w_gate is not read).
//   b2_moe_down      per tile: rows = act W_down[e]^T, fp32.
//   b2_moe_combine   y[t] = sum_j weight[t, j] * rows[place of (t, j)], summed in choice order in fp32: a token's result
//                    does not depend on what else is in the batch.
// The two grouped products are tiled through shared memory; bf16 runs on the tensor cores (16x16x16 fragments, fp32
// accumulation), the all-32-bit mode on fp32 FMAs.  Expert weights are stacked: w_gate, w_up [E, F, D]; w_down [E, D, F].
#include "b2_act.cuh"

#include <mma.h>
#include <type_traits>

namespace {

constexpr int kMoeBM = 32, kMoeBN = 64, kMoeBK = 32;

// ------------------------------------------------------------------------------------------------- router
// One warp picks the `top` experts of token t from its fp32 logits z [E] in shared memory (overwritten).
struct RouteSpec {
    int scoring, n_groups, keep_groups;
    float weight_scale;
};

// floats of scratch per token beside its E logits
__host__ __device__ __forceinline__ int route_scratch(int scoring, int E) { return scoring == B2_ROUTE_SIGMOID_GROUPED ? 2 * E : 0; }

// lowest index wins a tie; every lane returns the winner
__device__ __forceinline__ int warp_argmax(const float* c, int E, int lane, float& best_out) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
        if (c[e] > best) { best = c[e]; arg = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    best_out = best;
    return arg;
}

__device__ __forceinline__ void route_select(float* z, int t, int E, int top, RouteSpec rs, const float* __restrict__ bias,
                                             int lane, int32_t* __restrict__ ids, float* __restrict__ wts) {
    const int scoring = rs.scoring;
    if (scoring == B2_ROUTE_SIGMOID_GROUPED) {
        float* c = z + E;                            // choice scores; then the group scores
        float* gs = z + 2 * E;
        for (int e = lane; e < E; e += 32) {
            z[e] = b2::sigmoid_f(z[e]);
            c[e] = z[e] + (bias ? bias[e] : 0.f);
        }
        __syncwarp();
        const int ng = rs.n_groups;
        if (ng > 1) {
            const int per = E / ng;
            for (int g = lane; g < ng; g += 32) {    // sum of the two largest choice scores of the group
                float a = -INFINITY, b = -INFINITY;
                for (int i = 0; i < per; ++i) {
                    const float v = c[g * per + i];
                    if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
                }
                gs[g] = per > 1 ? a + b : a;
            }
            __syncwarp();
            for (int g = lane; g < ng; g += 32) {    // a group is kept when fewer than keep_groups groups come before it
                int before = 0;
                for (int o = 0; o < ng; ++o) before += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
                if (before >= rs.keep_groups)
                    for (int i = 0; i < per; ++i) c[g * per + i] = -INFINITY;
            }
            __syncwarp();
        }
        float sum = 0.f;
        for (int j = 0; j < top; ++j) {
            float best;
            int arg = warp_argmax(c, E, lane, best);
            if (arg == 0x7fffffff) arg = 0;
            const float w = best == -INFINITY ? 0.f : z[arg];
            sum += w;
            if (lane == 0) {
                ids[(size_t)t * top + j] = arg;
                wts[(size_t)t * top + j] = w;
                c[arg] = -INFINITY;
            }
            __syncwarp();
        }
        const float inv = rs.weight_scale / (sum + 1e-20f);
        for (int j = lane; j < top; j += 32) wts[(size_t)t * top + j] *= inv;
        return;
    }
    if (scoring == B2_ROUTE_SOFTMAX_ALL) {
        // scores over all experts; the choice adds the correction, the weight is the plain score
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        mx = b2::warp_max(mx);
        float den = 0.f;
        for (int e = lane; e < E; e += 32) den += expf(z[e] - mx);
        den = b2::warp_sum(den);
        for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - mx) / den;
        __syncwarp();
        for (int j = 0; j < top; ++j) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float c = z[e] + (bias ? bias[e] : 0.f);          // a chosen expert holds -inf
                if (c > best) { best = c; arg = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
            if (arg == 0x7fffffff) arg = 0;
            if (lane == 0) {
                ids[(size_t)t * top + j] = arg;
                wts[(size_t)t * top + j] = z[arg] == -INFINITY ? 0.f : z[arg];
                z[arg] = -INFINITY;
            }
            __syncwarp();
        }
        return;
    }
    float v0 = 0.f, sum = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (z[e] > best) { best = z[e]; arg = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg == 0x7fffffff) arg = 0;          // every logit is NaN or -inf: still a valid expert id
        if (j == 0) v0 = best;
        const float p = expf(best - v0);
        sum += p;
        if (lane == 0) {
            ids[(size_t)t * top + j] = arg;
            wts[(size_t)t * top + j] = p;
            z[arg] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.f / sum;
    for (int j = lane; j < top; j += 32) wts[(size_t)t * top + j] *= inv;
}

// One CTA per TOK tokens: their rows are staged once as fp32, the warps share the experts (each logit is one warp's dot
// product with independent partial sums per lane; a weight vector is loaded once and applied to all TOK rows, which
// divides the L2 traffic of a prompt batch by TOK), then warp t picks the `top` largest of token t.
template <typename T, int TOK>
__global__ void moe_route_kernel(const T* __restrict__ h, int64_t h_stride, const T* __restrict__ w_r,
                                 const float* __restrict__ bias, int rows, int D, int E, int top, RouteSpec rs, bool vec,
                                 bool vec16, int32_t* __restrict__ ids, float* __restrict__ wts) {
    extern __shared__ float route_sm[];              // h [TOK][D] | z [TOK][E + scratch]
    const int scoring = rs.scoring;
    const int ZE = E + route_scratch(scoring, E);
    float* hs = route_sm;
    float* zs = route_sm + (size_t)TOK * D;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int t0 = blockIdx.x * TOK;
    const int nt = min(TOK, rows - t0);
    for (int i = threadIdx.x; i < TOK * D; i += blockDim.x) {
        const int tt = i / D;
        hs[i] = tt < nt ? b2::ld(h + (size_t)(t0 + tt) * h_stride + (i - tt * D)) : 0.f;
    }
    __syncthreads();
    for (int e = wid; e < E; e += nw) {
        const T* w = w_r + (size_t)e * D;
        float a[TOK][2];
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) a[tt][0] = a[tt][1] = 0.f;
        if (TOK == 1 && vec16) {                     // one token: 16 bytes of the weight row per lane and step
            constexpr int VE = 16 / sizeof(T);
            for (int i = lane * VE; i < D; i += 32 * VE) {
                const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
                const T* wv = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int c = 0; c < VE; c += 2) {
                    a[0][0] = fmaf(hs[i + c], b2::ld(wv + c), a[0][0]);
                    a[0][1] = fmaf(hs[i + c + 1], b2::ld(wv + c + 1), a[0][1]);
                }
            }
        } else if (vec) {                            // two weights per lane and step: the warp reads consecutive pairs,
            for (int i = lane * 2; i < D; i += 64) { // and the TOK rows in shared memory without bank conflicts
                float w0, w1;
                if constexpr (std::is_same<T, float>::value) {
                    const float2 wv = *reinterpret_cast<const float2*>(w + i);
                    w0 = wv.x;
                    w1 = wv.y;
                } else {
                    const uint32_t wv = *reinterpret_cast<const uint32_t*>(w + i);
                    w0 = __uint_as_float(wv << 16);
                    w1 = __uint_as_float(wv & 0xffff0000u);
                }
#pragma unroll
                for (int tt = 0; tt < TOK; ++tt) {
                    const float2 hv = *reinterpret_cast<const float2*>(hs + tt * D + i);
                    a[tt][0] = fmaf(hv.x, w0, a[tt][0]);
                    a[tt][1] = fmaf(hv.y, w1, a[tt][1]);
                }
            }
        } else {
            for (int i = lane; i < D; i += 32) {
                const float w0 = b2::ld(w + i);
#pragma unroll
                for (int tt = 0; tt < TOK; ++tt) a[tt][0] = fmaf(hs[tt * D + i], w0, a[tt][0]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < TOK; ++tt) {
            const float v = b2::warp_sum(a[tt][0] + a[tt][1]);
            if (lane == 0) zs[tt * ZE + e] = v + ((bias && scoring == B2_ROUTE_TOPK_SOFTMAX) ? bias[e] : 0.f);
        }
    }
    __syncthreads();
    for (int tt = wid; tt < nt; tt += nw) route_select(zs + (size_t)tt * ZE, t0 + tt, E, top, rs, bias, lane, ids, wts);
}

// The same choice from logits that a library GEMM has produced (prompt batches): a warp per token.
__global__ void moe_select_kernel(const float* __restrict__ logits, int64_t stride, const float* __restrict__ bias, int rows, int E,
                                  int top, RouteSpec rs, int32_t* __restrict__ ids, float* __restrict__ wts) {
    extern __shared__ float route_sm[];              // z [warps][E + scratch]
    const int scoring = rs.scoring;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + wid;
    if (t >= rows) return;
    float* z = route_sm + (size_t)wid * (E + route_scratch(scoring, E));
    for (int e = lane; e < E; e += 32)
        z[e] = logits[(size_t)t * stride + e] + ((bias && scoring == B2_ROUTE_TOPK_SOFTMAX) ? bias[e] : 0.f);
    __syncwarp();
    route_select(z, t, E, top, rs, bias, lane, ids, wts);
}

// ------------------------------------------------------------------------------------------------- align
__global__ void moe_align_kernel(const int32_t* __restrict__ ids, int n, int E, int cap, int32_t* __restrict__ sorted,
                                 int32_t* __restrict__ tile_expert, int32_t* __restrict__ place,
                                 int32_t* __restrict__ group_ends) {
    extern __shared__ int sm[];                      // counts [E] | offs [E] | fill [E]
    int* counts = sm;
    int* offs = sm + E;
    int* fill = sm + 2 * E;
    __shared__ int total;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = fill[e] = 0;
    for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            offs[e] = run;
            run += (counts[e] + kMoeBM - 1) / kMoeBM * kMoeBM;
        }
        total = run;
    }
    __syncthreads();
    const int tiles = cap / kMoeBM;
    if (group_ends)                                  // row where expert e's (padded) group ends: offsets of a grouped GEMM
        for (int e = threadIdx.x; e < E; e += blockDim.x) group_ends[e] = e + 1 < E ? offs[e + 1] : total;
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int t = offs[e] / kMoeBM; t < (offs[e] + counts[e] + kMoeBM - 1) / kMoeBM; ++t) tile_expert[t] = e;
    for (int t = total / kMoeBM + threadIdx.x; t < tiles; t += blockDim.x) tile_expert[t] = -1;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < E) {
            const int p = offs[e] + atomicAdd(&fill[e], 1);
            sorted[p] = i;
            place[i] = p;
        } else {
            place[i] = -1;
        }
    }
}

// ------------------------------------------------------------------------------------------------- grouped products
template <typename T> struct Pad { static constexpr int v = 8; };
template <> struct Pad<float> { static constexpr int v = 1; };

// dst[r][0..BK) = row r of a [nrows, K] operand at columns k0.., zero outside; rowptr(r) = nullptr for a padding row
template <typename T, int NROWS, typename F>
__device__ __forceinline__ void load_tile(T* dst, F rowptr, int k0, int K, bool vec) {
    constexpr int LD = kMoeBK + Pad<T>::v;
    constexpr int VE = 16 / sizeof(T);
    if (vec) {
        for (int idx = threadIdx.x; idx < NROWS * (kMoeBK / VE); idx += blockDim.x) {
            const int r = idx / (kMoeBK / VE), kv = (idx % (kMoeBK / VE)) * VE;
            const T* p = rowptr(r);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (p && k0 + kv < K) v = *reinterpret_cast<const uint4*>(p + k0 + kv);
            if constexpr (std::is_same<T, float>::value) {
                float* d = reinterpret_cast<float*>(dst) + r * LD + kv;
                d[0] = __uint_as_float(v.x); d[1] = __uint_as_float(v.y); d[2] = __uint_as_float(v.z); d[3] = __uint_as_float(v.w);
            } else {
                *reinterpret_cast<uint4*>(dst + r * LD + kv) = v;
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < NROWS * kMoeBK; idx += blockDim.x) {
            const int r = idx / kMoeBK, kk = idx % kMoeBK;
            const T* p = rowptr(r);
            T v = T(0.f);
            if (p && k0 + kk < K) v = p[k0 + kk];
            dst[r * LD + kk] = v;
        }
    }
}

__device__ __forceinline__ void cp_async16_zfill(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;                // 0: the 16 destination bytes are zero-filled, src is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(b2::smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

constexpr int kMoeStages = 3;

// shared memory of one CTA: the operand stages, re-used for the fp32 result tile [NB][BM][BN] after the last k-step
template <typename T, int NB>
struct TileSmem {
    static constexpr int LD = kMoeBK + Pad<T>::v;
    static constexpr int A_EL = kMoeBM * LD, B_EL = NB * kMoeBN * LD, STAGE_EL = A_EL + B_EL;
    static constexpr int STAGES = std::is_same<T, float>::value ? 1 : kMoeStages;
    static constexpr int OPERAND_BYTES = STAGES * STAGE_EL * (int)sizeof(T);
    static constexpr int C_BYTES = NB * kMoeBM * kMoeBN * (int)sizeof(float);
    static constexpr int BYTES = OPERAND_BYTES > C_BYTES ? OPERAND_BYTES : C_BYTES;
};

// C[BM, BN] = A[BM, K] B[BN, K]^T for NB B operands that share A (NB = 2: gate and up).  Result as fp32 [NB][BM][BN] at
// the start of `sm`.  bf16 with 16-byte aligned rows: a three-stage cp.async pipeline feeds 16x16x16 tensor-core
// fragments, so the expert weights keep streaming while a k-step is multiplied (a decode batch is bound by that stream).
template <typename T, int NB, typename FA, typename FB0, typename FB1>
__device__ __forceinline__ void tile_product(FA a_row, FB0 b0_row, FB1 b1_row, int K, bool vec, unsigned char* sm) {
    using L = TileSmem<T, NB>;
    constexpr int LD = L::LD;
    const int tid = threadIdx.x;
    T* a_sm = reinterpret_cast<T*>(sm);
    T* b_sm = a_sm + L::A_EL;
    float* c_sm = reinterpret_cast<float*>(sm);
    if constexpr (std::is_same<T, float>::value) {
        const int ty = tid >> 4, tx = tid & 15;      // rows ty*4 .. +3, columns tx + 16 c
        float acc[NB][4][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[b][i][c] = 0.f;
        for (int k0 = 0; k0 < K; k0 += kMoeBK) {
            __syncthreads();
            load_tile<T, kMoeBM>(a_sm, a_row, k0, K, vec);
            load_tile<T, kMoeBN>(b_sm, b0_row, k0, K, vec);
            if (NB == 2) load_tile<T, kMoeBN>(b_sm + kMoeBN * LD, b1_row, k0, K, vec);
            __syncthreads();
#pragma unroll 8
            for (int kk = 0; kk < kMoeBK; ++kk) {
                float a[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = a_sm[(ty * 4 + i) * LD + kk];
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float bv = b_sm[(b * kMoeBN + tx + 16 * c) * LD + kk];
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[b][i][c] = fmaf(a[i], bv, acc[b][i][c]);
                    }
            }
        }
        __syncthreads();                             // every thread is done with the operands: the result takes their place
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) c_sm[(b * kMoeBM + ty * 4 + i) * kMoeBN + tx + 16 * c] = acc[b][i][c];
    } else {
        using namespace nvcuda;
        const int wid = tid >> 5;
        const int wm = wid >> 1, wn = wid & 1;       // warp tile: rows wm*16 .. +15, columns wn*32 .. +31
        wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[NB][2];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = 0; c < 2; ++c) wmma::fill_fragment(acc[b][c], 0.f);
        auto multiply = [&](const T* as, const T* bs) {
#pragma unroll
            for (int kk = 0; kk < kMoeBK; kk += 16) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
                wmma::load_matrix_sync(fa, as + (wm * 16) * LD + kk, LD);
#pragma unroll
                for (int b = 0; b < NB; ++b)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
                        wmma::load_matrix_sync(fb, bs + (b * kMoeBN + wn * 32 + c * 16) * LD + kk, LD);
                        wmma::mma_sync(acc[b][c], fa, fb, acc[b][c]);
                    }
            }
        };
        if (vec) {
            const T* safe = b0_row(0);               // a valid address for the copies that only zero-fill
            auto issue = [&](int ks, int buf) {
                T* as = a_sm + buf * L::STAGE_EL;
                T* bs = as + L::A_EL;
                const int k0 = ks * kMoeBK;
                for (int idx = tid; idx < kMoeBM * (kMoeBK / 8); idx += 128) {
                    const int r = idx / (kMoeBK / 8), kv = (idx % (kMoeBK / 8)) * 8;
                    const T* p = a_row(r);
                    const bool ok = p && k0 + kv < K;
                    cp_async16_zfill(as + r * LD + kv, ok ? p + k0 + kv : safe, ok);
                }
                for (int idx = tid; idx < NB * kMoeBN * (kMoeBK / 8); idx += 128) {
                    const int r = idx / (kMoeBK / 8), kv = (idx % (kMoeBK / 8)) * 8;
                    const T* p = r < kMoeBN ? b0_row(r) : b1_row(r - kMoeBN);
                    const bool ok = p && k0 + kv < K;
                    cp_async16_zfill(bs + r * LD + kv, ok ? p + k0 + kv : safe, ok);
                }
            };
            const int nk = (K + kMoeBK - 1) / kMoeBK;
            for (int st = 0; st < kMoeStages - 1; ++st) {
                if (st < nk) issue(st, st);
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            for (int ks = 0; ks < nk; ++ks) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kMoeStages - 2) : "memory");
                __syncthreads();                     // k-step ks has landed; the stage of k-step ks-1 is free again
                const int nx = ks + kMoeStages - 1;
                if (nx < nk) issue(nx, nx % kMoeStages);
                asm volatile("cp.async.commit_group;" ::: "memory");
                const T* as = a_sm + (ks % kMoeStages) * L::STAGE_EL;
                multiply(as, as + L::A_EL);
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
            for (int k0 = 0; k0 < K; k0 += kMoeBK) {
                __syncthreads();
                load_tile<T, kMoeBM>(a_sm, a_row, k0, K, false);
                load_tile<T, kMoeBN>(b_sm, b0_row, k0, K, false);
                if (NB == 2) load_tile<T, kMoeBN>(b_sm + kMoeBN * LD, b1_row, k0, K, false);
                __syncthreads();
                multiply(a_sm, b_sm);
            }
        }
        __syncthreads();                             // every warp is done with the operands: the result takes their place
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int c = 0; c < 2; ++c)
                wmma::store_matrix_sync(c_sm + (b * kMoeBM + wm * 16) * kMoeBN + wn * 32 + c * 16, acc[b][c], kMoeBN,
                                        wmma::mem_row_major);
    }
    __syncthreads();
}

template <typename T, int NB>
__global__ void __launch_bounds__(128)
moe_gate_up_kernel(const T* __restrict__ h, int64_t h_stride, const T* __restrict__ w_gate, const T* __restrict__ w_up,
                   int64_t w13_expert_stride, const int32_t* __restrict__ sorted, const int32_t* __restrict__ tile_expert,
                   int top, int D, int F, bool vec, int glu, float alpha, float limit, T* __restrict__ act) {
    __shared__ __align__(128) unsigned char sm[TileSmem<T, NB>::BYTES];
    const float* c_sm = reinterpret_cast<const float*>(sm);
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int m0 = blockIdx.x * kMoeBM, n0 = blockIdx.y * kMoeBN;
    const T* wg = (NB == 2 ? w_gate : w_up) + (size_t)e * w13_expert_stride;
    const T* wu = w_up + (size_t)e * w13_expert_stride;
    auto a_row = [&](int r) -> const T* {
        const int s = sorted[m0 + r];
        return s >= 0 ? h + (size_t)(s / top) * h_stride : nullptr;
    };
    auto g_row = [&](int r) -> const T* { return n0 + r < F ? wg + (size_t)(n0 + r) * D : nullptr; };
    auto u_row = [&](int r) -> const T* { return n0 + r < F ? wu + (size_t)(n0 + r) * D : nullptr; };
    if (NB == 2) tile_product<T, NB>(a_row, g_row, u_row, D, vec, sm);
    else tile_product<T, NB>(a_row, u_row, u_row, D, vec, sm);
    for (int idx = threadIdx.x; idx < kMoeBM * kMoeBN; idx += blockDim.x) {
        const int r = idx / kMoeBN, c = idx % kMoeBN;
        if (n0 + c < F && sorted[m0 + r] >= 0) {
            float v;
            if (NB == 1) {
                v = b2::relu_sq_f(c_sm[idx]);
            } else {
                const float g = c_sm[idx], u = c_sm[(NB - 1) * kMoeBM * kMoeBN + idx];
                v = glu == B2_GLU_CLAMPED ? b2::glu_clamped_f(g, u, alpha, limit) : b2::silu_f(g) * u;
            }
            b2::st(act + (size_t)(m0 + r) * F + n0 + c, v);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int32_t* __restrict__ sorted,
                const int32_t* __restrict__ tile_expert, int D, int F, bool vec, float* __restrict__ rows) {
    __shared__ __align__(128) unsigned char sm[TileSmem<T, 1>::BYTES];
    const float* c_sm = reinterpret_cast<const float*>(sm);
    const int e = tile_expert[blockIdx.x];
    if (e < 0) return;
    const int m0 = blockIdx.x * kMoeBM, n0 = blockIdx.y * kMoeBN;
    const T* wd = w_down + (size_t)e * D * F;
    auto a_row = [&](int r) -> const T* { return sorted[m0 + r] >= 0 ? act + (size_t)(m0 + r) * F : nullptr; };
    auto d_row = [&](int r) -> const T* { return n0 + r < D ? wd + (size_t)(n0 + r) * F : nullptr; };
    tile_product<T, 1>(a_row, d_row, d_row, F, vec, sm);
    for (int idx = threadIdx.x; idx < kMoeBM * kMoeBN; idx += blockDim.x) {
        const int r = idx / kMoeBN, c = idx % kMoeBN;
        if (n0 + c < D && sorted[m0 + r] >= 0) rows[(size_t)(m0 + r) * D + n0 + c] = c_sm[idx];
    }
}

// out[p] = h[token of sorted[p]] for the rows of the sorted list, zeros for padding rows: the A operand of a grouped GEMM
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, int64_t h_stride, const int32_t* __restrict__ sorted, int top,
                                  int D, bool vec, T* __restrict__ out) {
    const int p = blockIdx.x, s = sorted[p];
    const T* src = s >= 0 ? h + (size_t)(s / top) * h_stride : nullptr;
    T* dst = out + (size_t)p * D;
    if (vec) {
        constexpr int VE = 16 / sizeof(T);
        for (int i = threadIdx.x * VE; i < D; i += blockDim.x * VE)
            *reinterpret_cast<uint4*>(dst + i) = src ? *reinterpret_cast<const uint4*>(src + i) : make_uint4(0, 0, 0, 0);
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src ? src[i] : T(0.f);
    }
}

template <typename T, typename R>
__global__ void moe_combine_kernel(const R* __restrict__ rows, const int32_t* __restrict__ place,
                                   const float* __restrict__ wts, int top, int D, T* __restrict__ y, int64_t y_stride) {
    const int t = blockIdx.x;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float a = 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = place[(size_t)t * top + j];
            if (p >= 0) a = fmaf(wts[(size_t)t * top + j], b2::ld(rows + (size_t)p * D + d), a);
        }
        b2::st(y + (size_t)t * y_stride + d, a);
    }
}

}  // namespace

extern "C" int b2_moe_tile_rows(void) { return kMoeBM; }

// rows of the sorted list for n (token, choice) pairs over E experts: every expert that is used pads to a tile boundary
extern "C" int b2_moe_capacity(int n, int E) {
    const int used = n < E ? n : E;
    return (n + used * (kMoeBM - 1) + kMoeBM - 1) / kMoeBM * kMoeBM;
}

static bool route_spec_ok(int scoring, int E, int top, int n_groups, int keep_groups) {
    if (scoring == B2_ROUTE_TOPK_SOFTMAX || scoring == B2_ROUTE_SOFTMAX_ALL) return true;
    if (scoring != B2_ROUTE_SIGMOID_GROUPED) return false;
    return n_groups >= 1 && E % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups &&
           (int64_t)keep_groups * (E / n_groups) >= top;
}

extern "C" int b2_moe_route(const void* h, int64_t h_stride, const void* w_router, const float* bias, int act_dtype, int T,
                            int D, int E, int top, int scoring, int32_t* ids, float* weights, void* stream) {
    return b2_moe_route_ex(h, h_stride, w_router, bias, act_dtype, T, D, E, top, scoring, 1, 1, 1.f, ids, weights, stream);
}

extern "C" int b2_moe_route_ex(const void* h, int64_t h_stride, const void* w_router, const float* bias, int act_dtype, int T,
                               int D, int E, int top, int scoring, int n_groups, int keep_groups, float weight_scale,
                               int32_t* ids, float* weights, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && E > 0 && top >= 1 && top <= E, B2_EINVAL, "moe_route: bad sizes D=%d E=%d top=%d", D, E, top);
    B2_REQUIRE(route_spec_ok(scoring, E, top, n_groups, keep_groups), B2_EINVAL,
               "moe_route: scoring %d with %d groups of which %d are kept cannot choose %d of %d experts", scoring, n_groups,
               keep_groups, top, E);
    if (T == 0) return B2_OK;
    B2_REQUIRE(h && w_router && ids && weights, B2_EINVAL, "moe_route: null pointer");
    const RouteSpec rs{scoring, n_groups, keep_groups, weight_scale};
    const int ZE = E + route_scratch(scoring, E);
    // prompt batches: four tokens share a CTA (and every weight load); small batches keep a CTA per token
    const int tok = (T >= 1024 && (size_t)4 * (D + ZE) * sizeof(float) <= 96 * 1024) ? 4 : 1;
    const size_t smem = (size_t)tok * (D + ZE) * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "moe_route: width %d and %d experts do not fit shared memory", D, E);
    const int warps = E < 8 ? (E < 4 ? 4 : E) : 8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, {
        const bool vec = D % 2 == 0 && b2_aligned16(w_router);
        const bool vec16 = D % (16 / (int)sizeof(A)) == 0 && b2_aligned16(w_router);
        if (tok == 4) {
            auto kern = moe_route_kernel<A, 4>;
            if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<(T + 3) / 4, warps * 32, smem, st>>>(static_cast<const A*>(h), h_stride, static_cast<const A*>(w_router), bias,
                                                        T, D, E, top, rs, vec, vec16, ids, weights);
        } else {
            auto kern = moe_route_kernel<A, 1>;
            if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<T, warps * 32, smem, st>>>(static_cast<const A*>(h), h_stride, static_cast<const A*>(w_router), bias, T, D, E, top,
                                              rs, vec, vec16, ids, weights);
        }
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_moe_select(const float* logits, int64_t stride, const float* bias, int T, int E, int top, int scoring,
                             int32_t* ids, float* weights, void* stream) {
    return b2_moe_select_ex(logits, stride, bias, T, E, top, scoring, 1, 1, 1.f, ids, weights, stream);
}

extern "C" int b2_moe_select_ex(const float* logits, int64_t stride, const float* bias, int T, int E, int top, int scoring,
                                int n_groups, int keep_groups, float weight_scale, int32_t* ids, float* weights, void* stream) {
    B2_REQUIRE(T >= 0 && E > 0 && top >= 1 && top <= E && stride >= E, B2_EINVAL, "moe_select: bad sizes E=%d top=%d", E, top);
    B2_REQUIRE(route_spec_ok(scoring, E, top, n_groups, keep_groups), B2_EINVAL,
               "moe_select: scoring %d with %d groups of which %d are kept cannot choose %d of %d experts", scoring, n_groups,
               keep_groups, top, E);
    if (T == 0) return B2_OK;
    B2_REQUIRE(logits && ids && weights, B2_EINVAL, "moe_select: null pointer");
    const int warps = 4;
    const size_t smem = (size_t)warps * (E + route_scratch(scoring, E)) * sizeof(float);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "moe_select: %d experts do not fit shared memory", E);
    const RouteSpec rs{scoring, n_groups, keep_groups, weight_scale};
    moe_select_kernel<<<(T + warps - 1) / warps, warps * 32, smem, static_cast<cudaStream_t>(stream)>>>(logits, stride, bias, T, E, top,
                                                                                                     rs, ids, weights);
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_moe_align(const int32_t* ids, int n, int E, int cap, int32_t* sorted, int32_t* tile_expert, int32_t* place,
                            int32_t* group_ends, void* stream) {
    B2_REQUIRE(n >= 0 && E > 0 && cap % kMoeBM == 0 && cap >= b2_moe_capacity(n, E), B2_EINVAL,
               "moe_align: capacity %d below %d for %d rows over %d experts", cap, b2_moe_capacity(n, E), n, E);
    if (n == 0) return B2_OK;
    B2_REQUIRE(ids && sorted && tile_expert && place, B2_EINVAL, "moe_align: null pointer");
    const size_t smem = (size_t)3 * E * sizeof(int);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "moe_align: %d experts do not fit shared memory", E);
    moe_align_kernel<<<1, 1024, smem, static_cast<cudaStream_t>(stream)>>>(ids, n, E, cap, sorted, tile_expert, place, group_ends);
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_moe_experts(const void* h, int64_t h_stride, const void* w_gate, const void* w_up, const void* w_down,
                              int64_t w13_expert_stride, int act_dtype, int T, int D, int F, int top, int cap,
                              const int32_t* sorted,
                              const int32_t* tile_expert, const int32_t* place, const float* weights, void* act, float* rows,
                              void* y, int64_t y_stride, int glu, float glu_alpha, float glu_limit, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && F > 0 && top >= 1 && cap % kMoeBM == 0, B2_EINVAL, "moe_experts: bad sizes");
    B2_REQUIRE(glu == B2_GLU_SILU || glu == B2_GLU_CLAMPED || glu == B2_FF_RELU_SQ, B2_EINVAL,
               "moe_experts: unknown expert activation %d", glu);
    if (T == 0) return B2_OK;
    const bool gated = glu != B2_FF_RELU_SQ;
    B2_REQUIRE(h && (w_gate || !gated) && w_up && w_down && sorted && tile_expert && place && weights && act && rows && y, B2_EINVAL,
               "moe_experts: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int tiles = cap / kMoeBM;
    const int ve = act_dtype == B2_ACT_BF16 ? 8 : 4;
    B2_REQUIRE(w13_expert_stride >= (int64_t)F * D, B2_EINVAL, "moe_experts: expert stride below F*D");
    const bool vec1 = D % ve == 0 && h_stride % ve == 0 && w13_expert_stride % ve == 0 && b2_aligned16(h) &&
                      (!gated || b2_aligned16(w_gate)) && b2_aligned16(w_up);
    const bool vec2 = F % ve == 0 && b2_aligned16(act) && b2_aligned16(w_down);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (gated)
            moe_gate_up_kernel<A, 2><<<dim3(tiles, (F + kMoeBN - 1) / kMoeBN), 128, 0, st>>>(
                static_cast<const A*>(h), h_stride, static_cast<const A*>(w_gate), static_cast<const A*>(w_up), w13_expert_stride,
                sorted, tile_expert, top, D, F, vec1, glu, glu_alpha, glu_limit, static_cast<A*>(act));
        else
            moe_gate_up_kernel<A, 1><<<dim3(tiles, (F + kMoeBN - 1) / kMoeBN), 128, 0, st>>>(
                static_cast<const A*>(h), h_stride, nullptr, static_cast<const A*>(w_up), w13_expert_stride, sorted, tile_expert,
                top, D, F, vec1, glu, glu_alpha, glu_limit, static_cast<A*>(act));
        moe_down_kernel<A><<<dim3(tiles, (D + kMoeBN - 1) / kMoeBN), 128, 0, st>>>(
            static_cast<const A*>(act), static_cast<const A*>(w_down), sorted, tile_expert, D, F, vec2, rows);
        moe_combine_kernel<A, float><<<T, 256, 0, st>>>(rows, place, weights, top, D, static_cast<A*>(y), y_stride);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_moe_gather(const void* h, int64_t h_stride, int act_dtype, const int32_t* sorted, int cap, int top, int D,
                             void* out, void* stream) {
    B2_REQUIRE(cap >= 0 && top >= 1 && D > 0, B2_EINVAL, "moe_gather: bad sizes");
    if (cap == 0) return B2_OK;
    B2_REQUIRE(h && sorted && out, B2_EINVAL, "moe_gather: null pointer");
    const int ve = act_dtype == B2_ACT_BF16 ? 8 : 4;
    const bool vec = D % ve == 0 && h_stride % ve == 0 && b2_aligned16(h) && b2_aligned16(out);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, (moe_gather_kernel<A><<<cap, 128, 0, st>>>(static_cast<const A*>(h), h_stride, sorted, top, D, vec,
                                                                           static_cast<A*>(out))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

// y[t] = sum_j weights[t, j] * rows[place[t, j]] in fp32, choice order; rows in the activation type (rows_f32 = 0) or fp32
extern "C" int b2_moe_combine(const void* rows, int rows_f32, const int32_t* place, const float* weights, int T, int top, int D,
                              void* y, int64_t y_stride, int act_dtype, void* stream) {
    B2_REQUIRE(T >= 0 && top >= 1 && D > 0, B2_EINVAL, "moe_combine: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(rows && place && weights && y, B2_EINVAL, "moe_combine: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (rows_f32) moe_combine_kernel<A, float><<<T, 256, 0, st>>>(static_cast<const float*>(rows), place, weights, top, D,
                                                                      static_cast<A*>(y), y_stride);
        else moe_combine_kernel<A, A><<<T, 256, 0, st>>>(static_cast<const A*>(rows), place, weights, top, D, static_cast<A*>(y),
                                                         y_stride);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
