// group_norm.cu -- the residual path of a pre-norm decoder whose norm works in groups, whose sublayer outputs pass a
// learned per-channel scale before the residual sum, and whose sequence mixers read a blend of the current and the
// previous token's normalised row ("token shift"); plus an embedding that adds sinusoidal positions.
//
//   b2_embed_sinusoid_norm   x[t] = gnorm(embed[token[t]] + pe(position[t]); w): the fp32 residual.  pe(p)[2i] = sin(p f_i),
//                            pe(p)[2i+1] = cos(p f_i) with the frequencies f_i given as a double table; the angle p f_i is
//                            formed and reduced to [-pi, pi] in double, so it is exact to fp32 at any position.
//                            norm_w NULL: no norm.
//   b2_group_norm_step       one pass over residual rows (fp32):
//                            (1) x_out[t] = x_in[t] + y_scale * (y[t] + y_bias)       (y NULL: x_out = x_in; y_scale NULL: ones)
//                            (2) when h is given: hn = gnorm(x_out[t]; w), and without a shift h[t] = hn; with shift_mu
//                                h[t] = hn + (prev - hn) * shift_mu, prev = the same normalised row of the token before:
//                                computed from row t-1 of the batch when that row belongs to the same sequence, read from
//                                the sequence's state slot for the first row of a portion with context, zeros at position 0.
//                            x_out may be x_in unless y and shift_mu are both given (a row's CTA reads its neighbour's
//                            inputs, which must not have been overwritten).
//   b2_shift_state           state[slot of sequence i] = gnorm(x[last row of sequence i]; w): what the next portion or
//                            decode step of that sequence reads as `prev`.  Runs after b2_group_norm_step on the stream.
//                            A batch of one row per sequence (a decode step) needs no second launch: with
//                            `advance_state` b2_group_norm_step stores the row it has just normalised itself, since the
//                            thread that read a column of the slot is the one that overwrites it.
//   gnorm(v; w): v is cut into `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), times w.
// The residual and all statistics are fp32 whatever the activation type.  Reductions run in a fixed order: a row's result
// does not depend on the batch around it, and the in-kernel `prev` equals what b2_shift_state stores bit for bit.
#include "b2_act.cuh"

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;

// 1 / sqrt(mean(part^2) + eps) of every group of `row` (shared memory, D = groups * Dg floats) into ginv [groups].
// `part_sm` holds groups * kNormWarps floats.  Warps split a group when there are fewer groups than warps.  Ends with a
// barrier.
__device__ __forceinline__ void group_inverse_rms(const float* row, int groups, int Dg, float eps, float* part_sm, float* ginv) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int wpg = groups >= kNormWarps ? 1 : kNormWarps / groups;          // warps per group
    if (wpg == 1) {
        for (int g = wid; g < groups; g += kNormWarps) {
            const float* v = row + (size_t)g * Dg;
            float ss = 0.f;
            for (int i = lane; i < Dg; i += 32) ss = fmaf(v[i], v[i], ss);
            ss = b2::warp_sum(ss);
            if (lane == 0) ginv[g] = rsqrtf(ss / (float)Dg + eps);
        }
        __syncthreads();
        return;
    }
    if (wid < groups * wpg) {
        const int g = wid / wpg, part = wid % wpg;
        const float* v = row + (size_t)g * Dg;
        float ss = 0.f;
        for (int i = part * 32 + lane; i < Dg; i += wpg * 32) ss = fmaf(v[i], v[i], ss);
        ss = b2::warp_sum(ss);
        if (lane == 0) part_sm[g * kNormWarps + part] = ss;
    }
    __syncthreads();
    if (threadIdx.x < groups) {
        float ss = 0.f;
        for (int p = 0; p < wpg; ++p) ss += part_sm[threadIdx.x * kNormWarps + p];
        ginv[threadIdx.x] = rsqrtf(ss / (float)Dg + eps);
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kNormThreads)
embed_sinusoid_norm_kernel(float* __restrict__ x, const T* __restrict__ embed, const int64_t* __restrict__ tokens,
                           const int32_t* __restrict__ positions, int D, const double* __restrict__ freq,
                           const float* __restrict__ norm_w, int groups, float eps) {
    extern __shared__ __align__(16) float gn_sm[];   // row [D] | parts [groups * warps] | ginv [groups]
    float* row = gn_sm;
    float* part_sm = gn_sm + D;
    float* ginv = part_sm + groups * kNormWarps;
    const int t = blockIdx.x;
    const T* e = embed + (size_t)tokens[t] * D;
    const double p = (double)positions[t];
    for (int j = threadIdx.x; 2 * j < D; j += blockDim.x) {
        double a = p * freq[j];
        a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);     // into [-pi, pi]
        float s, c;
        sincosf((float)a, &s, &c);
        row[2 * j] = b2::ld(e + 2 * j) + s;
        if (2 * j + 1 < D) row[2 * j + 1] = b2::ld(e + 2 * j + 1) + c;
    }
    __syncthreads();
    float* xt = x + (size_t)t * D;
    if (!norm_w) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) xt[i] = row[i];
        return;
    }
    const int Dg = D / groups;
    group_inverse_rms(row, groups, Dg, eps, part_sm, ginv);
    for (int i = threadIdx.x; i < D; i += blockDim.x) xt[i] = row[i] * ginv[i / Dg] * norm_w[i];
}

// W = 4: every access is a 16-byte (fp32) or 8-byte (bf16) vector; W = 1: any width and alignment.  A CTA walks
// `rows_per_cta` consecutive rows: with a token shift the normalised row stays in shared memory as the next row's `prev`,
// so only the first row of a CTA normalises its predecessor a second time (from that row's inputs, never from x_out).
// A thread keeps to its own columns in every pass; only the group statistics look across threads.
template <typename T, int W>
__global__ void __launch_bounds__(kNormThreads)
group_norm_step_kernel(const float* __restrict__ x_in, float* __restrict__ x_out, int rows, int rows_per_cta, int D,
                       const T* __restrict__ y, int64_t y_stride, const float* __restrict__ y_scale,
                       const float* __restrict__ y_bias, const float* __restrict__ norm_w, int groups, float eps,
                       const float* __restrict__ shift_mu, const float* __restrict__ shift_state,
                       const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start,
                       const int32_t* __restrict__ state_slot, int n_seq, T* __restrict__ h, int64_t h_stride,
                       float* __restrict__ state_out) {
    extern __shared__ __align__(16) float gn_sm[];   // row [D] | second row [D] (shift) | parts | ginv
    float* cur = gn_sm;
    float* prv = gn_sm + D;
    float* part_sm = gn_sm + (shift_mu ? 2 : 1) * (size_t)D;
    float* ginv = part_sm + groups * kNormWarps;
    const int Dg = D / groups;
    const int step = blockDim.x * W;
    const bool write_out = x_out && (y || x_out != x_in);
    // x_in[t] + y_scale * (y[t] + y_bias) into dst; `store`: also into x_out
    auto load_row = [&](int t, float* dst, bool store) {
        for (int i = threadIdx.x * W; i < D; i += step) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(x_in + (size_t)t * D + i, v); else v[0] = x_in[(size_t)t * D + i];
            if (y) {
                float u[4] = {0.f, 0.f, 0.f, 0.f}, sc[4] = {1.f, 1.f, 1.f, 1.f}, bi[4] = {0.f, 0.f, 0.f, 0.f};
                if (W == 4) {
                    b2::ld4(y + (size_t)t * y_stride + i, u);
                    if (y_scale) b2::ld4(y_scale + i, sc);
                    if (y_bias) b2::ld4(y_bias + i, bi);
                } else {
                    u[0] = b2::ld(y + (size_t)t * y_stride + i);
                    if (y_scale) sc[0] = y_scale[i];
                    if (y_bias) bi[0] = y_bias[i];
                }
#pragma unroll
                for (int c = 0; c < W; ++c) v[c] = fmaf(sc[c], u[c] + bi[c], v[c]);
            }
#pragma unroll
            for (int c = 0; c < W; ++c) dst[i + c] = v[c];
            if (store) {
                if (W == 4) b2::st4(x_out + (size_t)t * D + i, v); else x_out[(size_t)t * D + i] = v[0];
            }
        }
    };
    // dst <- dst / rms of its group * w, in place (own columns)
    auto normalise = [&](float* dst) {
        for (int i = threadIdx.x * W; i < D; i += step) {
            float w[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(norm_w + i, w); else w[0] = norm_w[i];
#pragma unroll
            for (int c = 0; c < W; ++c) dst[i + c] = dst[i + c] * ginv[(i + c) / Dg] * w[c];
        }
    };
    const int t0 = blockIdx.x * rows_per_cta, t1 = min(t0 + rows_per_cta, rows);
    int seq = 0;
    if (shift_mu) {
        seq = b2::seq_of_row(cu_q, n_seq, t0);
        if (t0 - cu_q[seq] > 0 && ctx_start[seq] >= 0) {         // the row before the CTA's first: normalised once more
            load_row(t0 - 1, prv, false);
            __syncthreads();
            group_inverse_rms(prv, groups, Dg, eps, part_sm, ginv);
            normalise(prv);
        }
    }
    for (int t = t0; t < t1; ++t) {
        load_row(t, cur, write_out);
        if (!h) continue;
        __syncthreads();
        group_inverse_rms(cur, groups, Dg, eps, part_sm, ginv);
        T* ho = h + (size_t)t * h_stride;
        const float* pv = nullptr;
        float* keep = nullptr;                       // one row per sequence: the row's reader of the state also advances it
        if (shift_mu) {
            while (seq + 1 < n_seq && cu_q[seq + 1] <= t) ++seq;
            const int li = t - cu_q[seq], ctx = ctx_start[seq], slot = state_slot[seq];
            pv = (li > 0 && ctx >= 0) ? prv : ((li == 0 && ctx > 0 && slot >= 0) ? shift_state + (size_t)slot * D : nullptr);
            if (state_out && ctx >= 0 && slot >= 0) keep = state_out + (size_t)slot * D;
        }
        // one pass: normalise, keep the normalised row for the next row's blend, blend with the row before, store
        for (int i = threadIdx.x * W; i < D; i += step) {
            float w[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f}, mu[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
            if (W == 4) {
                b2::ld4(norm_w + i, w);
                if (pv) b2::ld4(pv + i, p);
                if (shift_mu) b2::ld4(shift_mu + i, mu);
            } else {
                w[0] = norm_w[i];
                if (pv) p[0] = pv[i];
                if (shift_mu) mu[0] = shift_mu[i];
            }
#pragma unroll
            for (int c = 0; c < W; ++c) {
                const float v = cur[i + c] * ginv[(i + c) / Dg] * w[c];
                if (shift_mu) cur[i + c] = v;
                o[c] = shift_mu ? fmaf(p[c] - v, mu[c], v) : v;
            }
            if (W == 4) b2::st4(ho + i, o); else b2::st(ho + i, o[0]);
            if (keep) {
                if (W == 4) b2::st4(keep + i, *reinterpret_cast<const float(*)[4]>(cur + i)); else keep[i] = cur[i];
            }
        }
        __syncthreads();                             // the statistics' readers are done before the next row lands
        if (shift_mu) {
            float* sw = cur;                         // this row is the next one's `prev`
            cur = prv;
            prv = sw;
        }
    }
}

__global__ void __launch_bounds__(kNormThreads)
shift_state_kernel(const float* __restrict__ x, int D, const float* __restrict__ norm_w, int groups, float eps,
                   const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start,
                   const int32_t* __restrict__ state_slot, float* __restrict__ shift_state) {
    extern __shared__ __align__(16) float gn_sm[];   // row [D] | parts | ginv
    float* row = gn_sm;
    float* part_sm = gn_sm + D;
    float* ginv = part_sm + groups * kNormWarps;
    const int seq = blockIdx.x;
    const int slot = state_slot[seq];
    const int n = cu_q[seq + 1] - cu_q[seq];
    if (ctx_start[seq] < 0 || slot < 0 || n <= 0) return;
    const float* xt = x + (size_t)(cu_q[seq + 1] - 1) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) row[i] = xt[i];
    __syncthreads();
    const int Dg = D / groups;
    group_inverse_rms(row, groups, Dg, eps, part_sm, ginv);
    float* st = shift_state + (size_t)slot * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) st[i] = row[i] * ginv[i / Dg] * norm_w[i];
}

}  // namespace

extern "C" int b2_embed_sinusoid_norm(float* x, const void* embed, int act_dtype, const int64_t* tokens,
                                      const int32_t* positions, int T, int D, const double* freq, const float* norm_w,
                                      int groups, float eps, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && groups >= 1 && D % groups == 0, B2_EINVAL, "embed_sinusoid_norm: bad sizes D=%d groups=%d", D,
               groups);
    if (T == 0) return B2_OK;
    B2_REQUIRE(x && embed && tokens && positions && freq, B2_EINVAL, "embed_sinusoid_norm: null pointer");
    const size_t smem = ((size_t)D + (size_t)groups * (kNormWarps + 1)) * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "embed_sinusoid_norm: width %d does not fit shared memory", D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, {
        auto kern = embed_sinusoid_norm_kernel<A>;
        if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<T, kNormThreads, smem, st>>>(x, static_cast<const A*>(embed), tokens, positions, D, freq, norm_w, groups, eps);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_group_norm_step(const float* x_in, float* x_out, int T, int D, const void* y, int64_t y_stride,
                                  const float* y_scale, const float* y_bias, const float* norm_w, int groups, float eps,
                                  const float* shift_mu, const float* shift_state, const int32_t* cu_q,
                                  const int32_t* ctx_start, const int32_t* state_slot, int n_seq, void* h, int64_t h_stride,
                                  int act_dtype, int advance_state, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0 && groups >= 1 && D % groups == 0, B2_EINVAL, "group_norm_step: bad sizes D=%d groups=%d", D, groups);
    if (T == 0 || (!y && !h && x_out == x_in)) return B2_OK;
    B2_REQUIRE(x_in, B2_EINVAL, "group_norm_step: null residual");
    B2_REQUIRE(!h || norm_w, B2_EINVAL, "group_norm_step: a read-out needs its norm weight");
    B2_REQUIRE(!y || x_out, B2_EINVAL, "group_norm_step: a sublayer output needs a residual to land in");
    B2_REQUIRE(!shift_mu || (h && cu_q && ctx_start && state_slot && shift_state && n_seq > 0), B2_EINVAL,
               "group_norm_step: a token shift needs the read-out, the sequences and the state");
    B2_REQUIRE(!advance_state || (shift_mu && T == n_seq), B2_EINVAL,
               "group_norm_step: the state is advanced in the same launch only for one row per sequence (%d rows, %d sequences)", T,
               n_seq);
    B2_REQUIRE(!(shift_mu && y && x_out == x_in), B2_EINVAL,
               "group_norm_step: with a sublayer output and a token shift the residual cannot be updated in place");
    const size_t smem = ((shift_mu ? 2 : 1) * (size_t)D + (size_t)groups * (kNormWarps + 1)) * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "group_norm_step: width %d does not fit shared memory", D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // long batches with a token shift: four rows a CTA, so that three of four rows find their predecessor in shared memory
    const int per = (shift_mu && T >= 2048) ? (T >= 8192 ? 8 : 4) : 1;
    const bool vec = D % 4 == 0 && b2_aligned16(x_in) && (!x_out || b2_aligned16(x_out)) &&
                     (!y || (y_stride % 4 == 0 && b2_aligned16(y))) && (!h || (h_stride % 4 == 0 && b2_aligned16(h))) &&
                     (!y_scale || b2_aligned16(y_scale)) && (!y_bias || b2_aligned16(y_bias)) && (!norm_w || b2_aligned16(norm_w)) &&
                     (!shift_mu || (b2_aligned16(shift_mu) && b2_aligned16(shift_state)));
#define B2_GROUP_NORM(W)                                                                                                    \
    do {                                                                                                                    \
        auto kern = group_norm_step_kernel<A, W>;                                                                           \
        if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<(T + per - 1) / per, kNormThreads, smem, st>>>(x_in, x_out, T, per, D, static_cast<const A*>(y), y_stride, y_scale, \
                                                              y_bias, norm_w, groups, eps, shift_mu, shift_state, cu_q, ctx_start, \
                                                              state_slot, n_seq, static_cast<A*>(h), h_stride,              \
                                                              advance_state ? const_cast<float*>(shift_state) : nullptr);   \
    } while (0)
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec) B2_GROUP_NORM(4);
        else B2_GROUP_NORM(1);
    });
#undef B2_GROUP_NORM
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_shift_state(const float* x, int D, const float* norm_w, int groups, float eps, const int32_t* cu_q,
                              const int32_t* ctx_start, const int32_t* state_slot, int n_seq, float* shift_state, void* stream) {
    B2_REQUIRE(D > 0 && groups >= 1 && D % groups == 0 && n_seq >= 0, B2_EINVAL, "shift_state: bad sizes D=%d groups=%d", D, groups);
    if (n_seq == 0) return B2_OK;
    B2_REQUIRE(x && norm_w && cu_q && ctx_start && state_slot && shift_state, B2_EINVAL, "shift_state: null pointer");
    const size_t smem = ((size_t)D + (size_t)groups * (kNormWarps + 1)) * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "shift_state: width %d does not fit shared memory", D);
    if (smem > 48 * 1024)
        B2_CUDA_OK(cudaFuncSetAttribute(shift_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    shift_state_kernel<<<n_seq, kNormThreads, smem, static_cast<cudaStream_t>(stream)>>>(x, D, norm_w, groups, eps, cu_q, ctx_start,
                                                                                        state_slot, shift_state);
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
