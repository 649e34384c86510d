// latent_attention.cu -- softmax attention whose keys and values are rebuilt from ONE low-rank latent per token that all
// heads share, plus one rotated key part that all heads share as well.  Per token the paged pool keeps a row
//   cache [num_blocks, bs, R + dr] = [ latent c (R, RMS-normed) | rotated key part (dr) ]        (activation type)
// and nothing per head.  With per-head up-projections K_h = W_uk[h] c and V_h = W_uv[h] c the score of head h is
//   s = scale * ( (W_uk[h]^T q_h) . c  +  q_rot_h . k_rot ),
// so a query that has been carried into the latent space ("absorbed": qa_h = [ W_uk[h]^T q_h | q_rot_h ], size R + dr) scores
// straight against the cache rows, and the head's output is W_uv[h] applied to sum_j p_j c_j.  Every head reads the same
// R + dr numbers per key: the op is multi-query attention with key size R + dr and value = the first R entries of the key.
//
//   b2_latent_prep        per token: the rotated parts of the query heads are rotated (pairs 2i, 2i+1 of the first
//                         `rot_dims` entries; angle and magnitude from a fp32 table [max_pos, rot_dims] = cos | sin halves)
//                         and written behind the absorbed part of qa; when the layer owns a down-projection its first R
//                         outputs are RMS-normed (plain weight) into the cache row at the token's slot and the last dr,
//                         rotated, behind them.  A layer that reads another layer's pool passes dkv_off < 0.
//   b2_latent_prep_rows   the same with the query heads and the down-projection in rows of two different buffers (a design
//                         whose queries come out of a second product, behind a query latent).
//   b2_latent_attention   o[t, h, :R] = gate[t, h] * sum_j softmax_j(s)[j] c_j over the visible keys: j <= i, and with a
//                         window W > 0 also i - j < W.  gate = sigmoid of a per-head column of the projection rows
//                         (gate NULL: 1).  Softmax state, scores and the accumulator are fp32.
// Sequences are described like everywhere in this library: rows cu_q[i] .. cu_q[i+1]-1, ctx_start[i] cached tokens before
// them (< 0: padding, output rows are zeroed), block_tables[i, :].
// Every sequence of a batch has at least one row; a batch with as many rows as sequences is therefore one row each (a
// decode step) and may take the decode kernel.  b2_latent_attention_workspace tells how much fp32 scratch a call can use
// to split the keys of a row over CTAs; without it the call runs unsplit.
#include "b2_act.cuh"

namespace {

constexpr int kMaxRPerLane = 32;                     // R <= 1024 in the warp kernel

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int64_t proj_stride, const T* __restrict__ kv, int64_t kv_stride,
                                   int H, int dn, int dr, int rot_dims, int R,
                                   int q_off, int dkv_off, const float* __restrict__ norm_w, float eps,
                                   const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, int max_pos,
                                   const int64_t* __restrict__ slots, int bs, T* __restrict__ qa, T* __restrict__ cache) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    const int Dc = R + dr, half = rot_dims / 2;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot_dims;
    // query heads: [dn | dr] -> the dr part, rotated, behind the R absorbed entries of qa[t, h]
    for (int idx = threadIdx.x; idx < H * dr; idx += blockDim.x) {
        const int hh = idx / dr, i = idx % dr;
        const T* src = row + q_off + (size_t)hh * (dn + dr) + dn;
        float v = b2::ld(src + i);
        if (i < rot_dims) {
            const int pr = i >> 1;
            const float c = cs[pr], s = cs[half + pr];
            const float other = b2::ld(src + (i ^ 1));
            v = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
        }
        b2::st(qa + ((size_t)t * H + hh) * Dc + R + i, v);
    }
    if (dkv_off < 0) return;
    const int64_t slot = slots[t];
    if (slot < 0) return;                            // uniform over the block
    T* dst = cache + (size_t)slot * Dc;
    const T* src = kv + (size_t)t * kv_stride + dkv_off;      // the down-projection may live in rows of its own
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = b2::ld(src + i);
        ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf(b2::block_sum(ss, red) / (float)R + eps);
    for (int i = threadIdx.x; i < R; i += blockDim.x) b2::st(dst + i, b2::ld(src + i) * inv * (norm_w ? norm_w[i] : 1.f));
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
        float v = b2::ld(src + R + i);
        if (i < rot_dims) {
            const int pr = i >> 1;
            const float c = cs[pr], s = cs[half + pr];
            const float other = b2::ld(src + R + (i ^ 1));
            v = (i & 1) ? fmaf(v, c, other * s) : fmaf(v, c, -other * s);
        }
        b2::st(dst + R + i, v);
    }
}

// The same with four elements per access (8 or 16 bytes) for row layouts whose offsets are all multiples of four.
template <typename T>
__global__ void latent_prep_vec_kernel(const T* __restrict__ proj, int64_t proj_stride, const T* __restrict__ kv,
                                       int64_t kv_stride, int H, int dn, int dr, int rot_dims, int R,
                                       int q_off, int dkv_off, const float* __restrict__ norm_w, float eps,
                                       const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, int max_pos,
                                       const int64_t* __restrict__ slots, T* __restrict__ qa, T* __restrict__ cache) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* row = proj + (size_t)t * proj_stride;
    const int Dc = R + dr, half = rot_dims / 2;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot_dims;
    auto turn = [&](float (&v)[4], int i) {          // entries i .. i+3 of a rotated part: two pairs
#pragma unroll
        for (int c = 0; c < 4; c += 2) {
            if (i + c < rot_dims) {
                const int pr = (i + c) >> 1;
                const float co = cs[pr], si = cs[half + pr], u = v[c], w = v[c + 1];
                v[c] = u * co - w * si;
                v[c + 1] = w * co + u * si;
            }
        }
    };
    for (int e = threadIdx.x * 4; e < H * dr; e += blockDim.x * 4) {
        const int hh = e / dr, i = e % dr;
        float v[4];
        b2::ld4(row + q_off + (size_t)hh * (dn + dr) + dn + i, v);
        turn(v, i);
        b2::st4(qa + ((size_t)t * H + hh) * Dc + R + i, v);
    }
    if (dkv_off < 0) return;
    const int64_t slot = slots[t];
    if (slot < 0) return;                            // uniform over the block
    T* dst = cache + (size_t)slot * Dc;
    const T* src = kv + (size_t)t * kv_stride + dkv_off;      // the down-projection may live in rows of its own
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < R; i += blockDim.x * 4) {
        float v[4];
        b2::ld4(src + i, v);
        ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
    const float inv = rsqrtf(b2::block_sum(ss, red) / (float)R + eps);
    for (int i = threadIdx.x * 4; i < R; i += blockDim.x * 4) {
        float v[4];
        b2::ld4(src + i, v);
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] *= inv * (norm_w ? norm_w[i + c] : 1.f);
        b2::st4(dst + i, v);
    }
    for (int i = threadIdx.x * 4; i < dr; i += blockDim.x * 4) {
        float v[4];
        b2::ld4(src + R + i, v);
        turn(v, i);
        b2::st4(dst + R + i, v);
    }
}

// One warp per (row, head): scores of 32 keys at a time (a lane per key), online softmax, P.C with a lane per latent column.
// Any sizes, both activation types; the tensor-core kernel below takes the bf16 shapes it is built for.
template <typename T>
__global__ void latent_attention_kernel(const T* __restrict__ qa, const T* __restrict__ cache,
                                        const int32_t* __restrict__ block_tables, int max_nb, const int32_t* __restrict__ cu_q,
                                        const int32_t* __restrict__ ctx_start, int n_seq, int rows, int H, int R, int dr, int bs,
                                        float scale, int window, const T* __restrict__ gate, int64_t gate_stride,
                                        T* __restrict__ out) {
    extern __shared__ float q_sm[];                  // [warps, R + dr]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int item = blockIdx.x * (blockDim.x >> 5) + wid;       // (row, head)
    if (item >= rows * H) return;
    const int row = item / H, hh = item % H;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int ctx = ctx_start[seq];
    const int Dc = R + dr;
    T* dst = out + (size_t)item * R;
    if (ctx < 0) {
        for (int i = lane; i < R; i += 32) b2::st(dst + i, 0.f);
        return;
    }
    const int pos = ctx + row - cu_q[seq];
    const int lo = window > 0 ? max(pos - window + 1, 0) : 0;
    float* qs = q_sm + (size_t)wid * Dc;
    const T* qv = qa + (size_t)item * Dc;
    for (int i = lane; i < Dc; i += 32) qs[i] = b2::ld(qv + i) * scale;
    __syncwarp();
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    float m = -INFINITY, l = 0.f;
    float acc[kMaxRPerLane];
#pragma unroll
    for (int c = 0; c < kMaxRPerLane; ++c) acc[c] = 0.f;
    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        size_t base = 0;
        if (j <= pos) {
            base = ((size_t)bt[j / bs] * bs + (j % bs)) * Dc;
            const T* kr = cache + base;
            float d0 = 0.f, d1 = 0.f;
            int i = 0;
            for (; i + 1 < Dc; i += 2) {
                d0 = fmaf(qs[i], b2::ld(kr + i), d0);
                d1 = fmaf(qs[i + 1], b2::ld(kr + i + 1), d1);
            }
            if (i < Dc) d0 = fmaf(qs[i], b2::ld(kr + i), d0);
            s = d0 + d1;
        }
        const float m_new = fmaxf(m, b2::warp_max(s));
        const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
        const float p = j <= pos ? __expf(s - m_new) : 0.f;
        l = l * corr + b2::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxRPerLane; ++c) acc[c] *= corr;
        const int nk = min(32, pos - j0 + 1);
        for (int kk = 0; kk < nk; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const size_t vb = __shfl_sync(0xffffffffu, (unsigned long long)base, kk);
            const T* vr = cache + vb;
#pragma unroll
            for (int c = 0; c < kMaxRPerLane; ++c) {
                const int i = lane + 32 * c;
                if (i < R) acc[c] = fmaf(pk, b2::ld(vr + i), acc[c]);
            }
        }
    }
    float f = l > 0.f ? 1.f / l : 0.f;
    if (gate) f *= b2::sigmoid_f(b2::ld(gate + (size_t)row * gate_stride + hh));
#pragma unroll
    for (int c = 0; c < kMaxRPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < R) b2::st(dst + i, acc[c] * f);
    }
}

// ------------------------------------------------------------------------------------------------- tensor-core kernel
// bf16, latent size R in {64, 128, 256, 512}, rotated part a multiple of 16.  All heads read the same cache rows, so the
// M side of the products is (token, head): one CTA takes kLQ = 64 rows = 64 / Hc consecutive tokens of one sequence x Hc
// heads (Hc = min(H, 64)).  A decode row (one token) and a prompt portion are the same case with another token count.
// Keys are walked 64 at a time from the first token's window start to the last token's position; a key tile is gathered
// from the pages into shared memory ONCE per CTA (cp.async, 16 bytes per copy, the next tile in flight while this one is
// multiplied when two tiles fit beside Q) and serves S = Q K^T over all R + dr columns
// and O += P V over its first R columns (the value of a key is the head of its own row).  Eight warps: four groups of 16
// rows x two halves of the R output columns; both halves compute the group's scores (mma.sync m16n8k16, ldmatrix operands)
// and keep the online softmax in registers (exp2 with the scale folded in).  The gate multiplies the normalised output.
constexpr int kLQ = 64, kLK = 64;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(b2::smem_u32(dst)), "l"(src) : "memory");
}

template <int RT>
__global__ void __launch_bounds__(256)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ qa, const __nv_bfloat16* __restrict__ cache,
                            const int32_t* __restrict__ block_tables, int max_nb, const int32_t* __restrict__ cu_q,
                            const int32_t* __restrict__ ctx_start, int n_seq, int H, int Hc, int dr, int bs, float scale_log2,
                            int window, int stages, const __nv_bfloat16* __restrict__ gate, int64_t gate_stride,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ ws_o, float* __restrict__ ws_ml) {
    constexpr int R = 16 * RT;
    const int Dc = R + dr, LD = Dc + 8, vecs = Dc / 8;
    extern __shared__ __align__(16) unsigned char lat_smem[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(lat_smem);       // [64][LD]
    __nv_bfloat16* k_sm = q_sm + kLQ * LD;                                  // [stages][64][LD]
    __shared__ int s_info[2];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, wm = w & 3, wn = w >> 2;
    const int Gt = kLQ / Hc;                                                // tokens per CTA
    if (tid == 0) {
        int want = blockIdx.x, found = -1, t0 = 0;
        for (int s = 0; s < n_seq; ++s) {
            const int nt = (cu_q[s + 1] - cu_q[s] + Gt - 1) / Gt;
            if (want < nt) { found = s; t0 = want * Gt; break; }
            want -= nt;
        }
        s_info[0] = found;
        s_info[1] = t0;
    }
    __syncthreads();
    const int seq = s_info[0], t0 = s_info[1];
    if (seq < 0) return;
    const int h0 = blockIdx.y * Hc, nh = min(Hc, H - h0);
    const int tok0 = cu_q[seq] + t0;                                        // batch row of the CTA's first token
    const int ntok = min(Gt, cu_q[seq + 1] - tok0);
    const int ctx = ctx_start[seq];
    const int nsplit = gridDim.z, zs = blockIdx.z;                          // the CTA's share of the key tiles (decode batches)
    if (ctx < 0 && nsplit > 1) {                                            // padding: the merge turns "no keys" into zero rows
        for (int rr = tid; rr < ntok * nh; rr += 256) {
            float* ml = ws_ml + (((size_t)(tok0 + rr / nh) * H + h0 + rr % nh) * nsplit + zs) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;
    }
    if (ctx < 0) {                                                          // padding: zero rows
        for (int idx = tid; idx < ntok * nh * (R / 8); idx += 256) {
            const int rr = idx / (R / 8), c = (idx % (R / 8)) * 8;
            *reinterpret_cast<uint4*>(out + ((size_t)(tok0 + rr / nh) * H + h0 + rr % nh) * R + c) = make_uint4(0, 0, 0, 0);
        }
        return;
    }
    const int p0 = ctx + t0, p_last = p0 + ntok - 1;
    const int klo = window > 0 ? max(p0 - window + 1, 0) : 0;
    const int32_t* bt = block_tables + (size_t)seq * max_nb;

    for (int idx = tid; idx < kLQ * vecs; idx += 256) {
        const int r = idx / vecs, c = (idx % vecs) * 8;
        const int tk = r / Hc, hd = r % Hc;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tk < ntok && hd < nh) v = *reinterpret_cast<const uint4*>(qa + ((size_t)(tok0 + tk) * H + h0 + hd) * Dc + c);
        *reinterpret_cast<uint4*>(q_sm + r * LD + c) = v;
    }
    const int gq = lane >> 2, tq = lane & 3;
    const int ra = wm * 16 + gq, rb = ra + 8;                               // this thread's two rows
    const int i0 = p0 + ra / Hc, i1 = p0 + rb / Hc;                         // their positions
    const int lo0 = window > 0 ? max(i0 - window + 1, 0) : 0, lo1 = window > 0 ? max(i1 - window + 1, 0) : 0;
    const int w_first = p0 + (wm * 16) / Hc, w_last = p0 + (wm * 16 + 15) / Hc;
    const int w_lo = window > 0 ? max(w_first - window + 1, 0) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[RT][4];
#pragma unroll
    for (int n = 0; n < RT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const uint32_t q_base = b2::smem_u32(q_sm), k_base0 = b2::smem_u32(k_sm);
    const int ksteps = Dc / 16;

    // a thread copies a quarter of one key row per tile: one page lookup, then 16-byte copies 64 bytes apart
    const int ld_key = tid >> 2, ld_sub = (tid & 3) * 8;
    auto issue = [&](int kv0, int buf) {
        const int j = kv0 + ld_key;
        __nv_bfloat16* dst = k_sm + (size_t)buf * kLK * LD + ld_key * LD;
        if (j <= p_last) {
            const __nv_bfloat16* src = cache + ((size_t)bt[j / bs] * bs + j % bs) * Dc;
            for (int c = ld_sub; c < Dc; c += 32) cp_async16(dst + c, src + c);
        } else {
            for (int c = ld_sub; c < Dc; c += 32) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const bool active = wm * 16 < ntok * Hc;                                // a row group without rows only helps to copy
    const int all_tiles = (p_last - klo) / kLK + 1, per = (all_tiles + nsplit - 1) / nsplit;
    const int t_begin = zs * per, ntiles = min(all_tiles, t_begin + per);
    if (t_begin < ntiles) issue(klo + t_begin * kLK, 0);
    for (int t = t_begin; t < ntiles; ++t) {
        const int kv0 = klo + t * kLK, buf = stages == 2 ? ((t - t_begin) & 1) : 0;
        if (stages == 2 && t + 1 < ntiles) {                                // the next tile streams in while this one is multiplied
            issue(kv0 + kLK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                                    // the tile (and, first time, Q) is in shared memory
        const uint32_t k_base = k_base0 + (uint32_t)buf * kLK * LD * 2u;
        if (active && !(kv0 > w_last || kv0 + kLK - 1 < w_lo)) {            // else no key of the tile is visible to the warp's rows
            float sc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll 2
            for (int kk = 0; kk < ksteps; ++kk) {
                uint32_t a0, a1, a2, a3;
                b2::ldmatrix_x4(q_base + 2u * ((wm * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
#pragma unroll
                for (int n2 = 0; n2 < 4; ++n2) {
                    uint32_t b0, b1, b2_, b3;
                    const int key = n2 * 16 + (lane >> 4) * 8 + (lane & 7), dim = kk * 16 + ((lane >> 3) & 1) * 8;
                    b2::ldmatrix_x4(k_base + 2u * (key * LD + dim), b0, b1, b2_, b3);
                    b2::mma_bf16_16816(sc[2 * n2], a0, a1, a2, a3, b0, b1);
                    b2::mma_bf16_16816(sc[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = kv0 + n * 8 + 2 * tq + (e & 1);
                    const bool ok = e < 2 ? (j >= lo0 && j <= i0) : (j >= lo1 && j <= i1);
                    sc[n][e] = ok ? sc[n][e] * scale_log2 : -INFINITY;
                }
                mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
            const float c0 = exp2f(m0 - mu0), c1 = exp2f(m1 - mu1);             // exp2(-inf) = 0: nothing accumulated yet
            m0 = mn0;
            m1 = mn1;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                sc[n][0] = exp2f(sc[n][0] - mu0);
                sc[n][1] = exp2f(sc[n][1] - mu0);
                sc[n][2] = exp2f(sc[n][2] - mu1);
                sc[n][3] = exp2f(sc[n][3] - mu1);
                s0 += sc[n][0] + sc[n][1];
                s1 += sc[n][2] + sc[n][3];
            }
            l0 = l0 * c0 + s0;
            l1 = l1 * c1 + s1;
#pragma unroll
            for (int n = 0; n < RT; ++n) {
                o[n][0] *= c0;
                o[n][1] *= c0;
                o[n][2] *= c1;
                o[n][3] *= c1;
            }
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t a0 = b2::pack_bf16x2(sc[2 * ks][0], sc[2 * ks][1]),
                               a1 = b2::pack_bf16x2(sc[2 * ks][2], sc[2 * ks][3]);
                const uint32_t a2 = b2::pack_bf16x2(sc[2 * ks + 1][0], sc[2 * ks + 1][1]),
                               a3 = b2::pack_bf16x2(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < RT / 2; ++n2) {
                    uint32_t b0, b1, b2_, b3;
                    const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = wn * (R / 2) + n2 * 16 + (lane >> 4) * 8;
                    b2::ldmatrix_x4_trans(k_base + 2u * (key * LD + col), b0, b1, b2_, b3);
                    b2::mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
                    b2::mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
                }
            }
        }
        __syncthreads();                                                    // the tile is consumed: its buffer may be refilled
        if (stages == 1 && t + 1 < ntiles) issue(kv0 + kLK, 0);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int ta = ra / Hc, ha = ra % Hc, tb = rb / Hc, hb = rb % Hc;
    const bool va = ta < ntok && ha < nh, vb = tb < ntok && hb < nh;
    if (nsplit > 1) {                                                       // partial (max, sum, unnormalised output) of this share
        const size_t ia = ((size_t)(tok0 + ta) * H + h0 + ha) * nsplit + zs, ib = ((size_t)(tok0 + tb) * H + h0 + hb) * nsplit + zs;
        if (wn == 0 && tq == 0) {
            if (va) { ws_ml[ia * 2] = m0; ws_ml[ia * 2 + 1] = l0; }
            if (vb) { ws_ml[ib * 2] = m1; ws_ml[ib * 2 + 1] = l1; }
        }
#pragma unroll
        for (int n = 0; n < RT; ++n) {
            const int col = wn * (R / 2) + n * 8 + 2 * tq;
            if (va) *reinterpret_cast<float2*>(ws_o + ia * R + col) = make_float2(o[n][0], o[n][1]);
            if (vb) *reinterpret_cast<float2*>(ws_o + ib * R + col) = make_float2(o[n][2], o[n][3]);
        }
        return;
    }
    float f0 = l0 > 0.f ? 1.f / l0 : 0.f, f1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (gate) {
        if (va) f0 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(tok0 + ta) * gate_stride + h0 + ha]));
        if (vb) f1 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(tok0 + tb) * gate_stride + h0 + hb]));
    }
    __nv_bfloat16* oa = out + ((size_t)(tok0 + ta) * H + h0 + ha) * R + wn * (R / 2);
    __nv_bfloat16* ob = out + ((size_t)(tok0 + tb) * H + h0 + hb) * R + wn * (R / 2);
#pragma unroll
    for (int n = 0; n < RT; ++n) {
        const int col = n * 8 + 2 * tq;
        if (va) *reinterpret_cast<uint32_t*>(oa + col) = b2::pack_bf16x2(o[n][0] * f0, o[n][1] * f0);
        if (vb) *reinterpret_cast<uint32_t*>(ob + col) = b2::pack_bf16x2(o[n][2] * f1, o[n][3] * f1);
    }
}

// ------------------------------------------------------------------------------------------------- decode rows
// bf16, R >= 128, every sequence of the batch has ONE row: a CTA takes one token x up to 16 heads (one m16 row group), so
// the eight warps cannot share rows -- they share the KEYS of a tile instead.  Warp w scores keys 8w .. 8w+7 of the 64-key
// tile against all 16 rows, the row maxima meet in shared memory, every warp writes its 16 x 8 slice of P (bf16) to a
// shared P tile, and then multiplies the whole P tile with ITS R / 8 output columns of the key rows.  No score is computed
// twice, and the chain of dependent instructions per tile is an eighth of what one warp per row group would run.
constexpr int kPLD = kLK + 8;

__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

template <int RT>
__global__ void __launch_bounds__(256)
latent_attention_decode_kernel(const __nv_bfloat16* __restrict__ qa, const __nv_bfloat16* __restrict__ cache,
                               const int32_t* __restrict__ block_tables, int max_nb, const int32_t* __restrict__ cu_q,
                               const int32_t* __restrict__ ctx_start, int H, int dr, int bs, float scale_log2, int window,
                               const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out,
                               float* __restrict__ ws_o, float* __restrict__ ws_ml) {
    constexpr int R = 16 * RT, CW = R / 8, NTO = CW / 8;                    // output columns / n-tiles per warp
    static_assert(CW % 16 == 0, "a warp owns whole pairs of n-tiles");
    const int Dc = R + dr, LD = Dc + 8, vecs = Dc / 8;
    extern __shared__ __align__(16) unsigned char lat_smem[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(lat_smem);       // [16][LD]
    __nv_bfloat16* k_sm = q_sm + 16 * LD;                                   // [2][64][LD]
    __nv_bfloat16* p_sm = k_sm + 2 * kLK * LD;                              // [16][kPLD]
    float* mx_sm = reinterpret_cast<float*>(p_sm + 16 * kPLD);              // [8][16]: row maxima, later row sums, per warp
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int seq = blockIdx.x, tok = cu_q[seq];
    const int h0 = blockIdx.y * 16, nh = min(16, H - h0);
    const int nsplit = gridDim.z, zs = blockIdx.z;
    const int ctx = ctx_start[seq];
    if (ctx < 0) {                                                          // padding
        if (nsplit > 1) {
            for (int rr = tid; rr < nh; rr += 256) {
                float* ml = ws_ml + (((size_t)tok * H + h0 + rr) * nsplit + zs) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
        } else {
            for (int idx = tid; idx < nh * (R / 8); idx += 256)
                *reinterpret_cast<uint4*>(out + ((size_t)tok * H + h0 + idx / (R / 8)) * R + (idx % (R / 8)) * 8) =
                    make_uint4(0, 0, 0, 0);
        }
        return;
    }
    const int pos = ctx;
    const int klo = window > 0 ? max(pos - window + 1, 0) : 0;
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    for (int idx = tid; idx < 16 * vecs; idx += 256) {
        const int r = idx / vecs, c = (idx % vecs) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nh) v = *reinterpret_cast<const uint4*>(qa + ((size_t)tok * H + h0 + r) * Dc + c);
        *reinterpret_cast<uint4*>(q_sm + r * LD + c) = v;
    }
    const int gq = lane >> 2, tq = lane & 3;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[NTO][4];
#pragma unroll
    for (int n = 0; n < NTO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const uint32_t q_base = b2::smem_u32(q_sm), k_base0 = b2::smem_u32(k_sm), p_base = b2::smem_u32(p_sm);
    const int ksteps = Dc / 16;
    const int ld_key = tid >> 2, ld_sub = (tid & 3) * 8;
    auto issue = [&](int kv0, int buf) {
        const int j = kv0 + ld_key;
        __nv_bfloat16* dst = k_sm + (size_t)buf * kLK * LD + ld_key * LD;
        if (j <= pos) {
            const __nv_bfloat16* src = cache + ((size_t)bt[j / bs] * bs + j % bs) * Dc;
            for (int c = ld_sub; c < Dc; c += 32) cp_async16(dst + c, src + c);
        } else {
            for (int c = ld_sub; c < Dc; c += 32) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int all_tiles = (pos - klo) / kLK + 1, per = (all_tiles + nsplit - 1) / nsplit;
    const int t_begin = zs * per, ntiles = min(all_tiles, t_begin + per);
    if (t_begin < ntiles) issue(klo + t_begin * kLK, 0);
    for (int t = t_begin; t < ntiles; ++t) {
        const int kv0 = klo + t * kLK, buf = (t - t_begin) & 1;
        if (t + 1 < ntiles) {
            issue(kv0 + kLK, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();                                                    // the tile (and, first time, Q) is in shared memory
        const uint32_t k_base = k_base0 + (uint32_t)buf * kLK * LD * 2u;
        float sc[4] = {0.f, 0.f, 0.f, 0.f};                                 // 16 rows x this warp's 8 keys
#pragma unroll 4
        for (int kk = 0; kk < ksteps; ++kk) {
            uint32_t a0, a1, a2, a3, b0, b1;
            b2::ldmatrix_x4(q_base + 2u * ((lane & 15) * LD + kk * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
            ldmatrix_x2(k_base + 2u * ((w * 8 + (lane & 7)) * LD + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1);
            b2::mma_bf16_16816(sc, a0, a1, a2, a3, b0, b1);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int j = kv0 + w * 8 + 2 * tq + (e & 1);
            sc[e] = (j >= klo && j <= pos) ? sc[e] * scale_log2 : -INFINITY;
        }
        float mx0 = fmaxf(sc[0], sc[1]), mx1 = fmaxf(sc[2], sc[3]);
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        if (tq == 0) {
            mx_sm[w * 16 + gq] = mx0;
            mx_sm[w * 16 + gq + 8] = mx1;
        }
        __syncthreads();                                                    // every warp's row maxima of this tile
        float mn0 = m0, mn1 = m1;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            mn0 = fmaxf(mn0, mx_sm[x * 16 + gq]);
            mn1 = fmaxf(mn1, mx_sm[x * 16 + gq + 8]);
        }
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2f(m0 - mu0), c1 = exp2f(m1 - mu1);
        m0 = mn0;
        m1 = mn1;
        sc[0] = exp2f(sc[0] - mu0);
        sc[1] = exp2f(sc[1] - mu0);
        sc[2] = exp2f(sc[2] - mu1);
        sc[3] = exp2f(sc[3] - mu1);
        l0 = l0 * c0 + sc[0] + sc[1];                                       // sums over this warp's keys only
        l1 = l1 * c1 + sc[2] + sc[3];
        *reinterpret_cast<uint32_t*>(p_sm + gq * kPLD + w * 8 + 2 * tq) = b2::pack_bf16x2(sc[0], sc[1]);
        *reinterpret_cast<uint32_t*>(p_sm + (gq + 8) * kPLD + w * 8 + 2 * tq) = b2::pack_bf16x2(sc[2], sc[3]);
#pragma unroll
        for (int n = 0; n < NTO; ++n) {
            o[n][0] *= c0;
            o[n][1] *= c0;
            o[n][2] *= c1;
            o[n][3] *= c1;
        }
        __syncthreads();                                                    // the P tile is complete
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t a0, a1, a2, a3;
            b2::ldmatrix_x4(p_base + 2u * ((lane & 15) * kPLD + ks * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
#pragma unroll
            for (int n2 = 0; n2 < NTO / 2; ++n2) {
                uint32_t b0, b1, b2_, b3;
                const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = w * CW + n2 * 16 + (lane >> 4) * 8;
                b2::ldmatrix_x4_trans(k_base + 2u * (key * LD + col), b0, b1, b2_, b3);
                b2::mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
                b2::mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
            }
        }
        __syncthreads();                                                    // the tile, P and the maxima are consumed
    }
    // the row sums of the eight key slices
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (tq == 0) {
        mx_sm[w * 16 + gq] = l0;
        mx_sm[w * 16 + gq + 8] = l1;
    }
    __syncthreads();
    l0 = l1 = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        l0 += mx_sm[x * 16 + gq];
        l1 += mx_sm[x * 16 + gq + 8];
    }
    const bool va = gq < nh, vb = gq + 8 < nh;
    const size_t ra = (size_t)tok * H + h0 + gq, rb = ra + 8;
    if (nsplit > 1) {
        if (w == 0 && tq == 0) {
            if (va) { ws_ml[(ra * nsplit + zs) * 2] = m0; ws_ml[(ra * nsplit + zs) * 2 + 1] = l0; }
            if (vb) { ws_ml[(rb * nsplit + zs) * 2] = m1; ws_ml[(rb * nsplit + zs) * 2 + 1] = l1; }
        }
#pragma unroll
        for (int n = 0; n < NTO; ++n) {
            const int col = w * CW + n * 8 + 2 * tq;
            if (va) *reinterpret_cast<float2*>(ws_o + (ra * nsplit + zs) * R + col) = make_float2(o[n][0], o[n][1]);
            if (vb) *reinterpret_cast<float2*>(ws_o + (rb * nsplit + zs) * R + col) = make_float2(o[n][2], o[n][3]);
        }
        return;
    }
    float f0 = l0 > 0.f ? 1.f / l0 : 0.f, f1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (gate) {
        if (va) f0 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)tok * gate_stride + h0 + gq]));
        if (vb) f1 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)tok * gate_stride + h0 + gq + 8]));
    }
#pragma unroll
    for (int n = 0; n < NTO; ++n) {
        const int col = w * CW + n * 8 + 2 * tq;
        if (va) *reinterpret_cast<uint32_t*>(out + ra * R + col) = b2::pack_bf16x2(o[n][0] * f0, o[n][1] * f0);
        if (vb) *reinterpret_cast<uint32_t*>(out + rb * R + col) = b2::pack_bf16x2(o[n][2] * f1, o[n][3] * f1);
    }
}

// ------------------------------------------------------------------------------------------------- prompt portions, per-head keys
// Long prompt portions are cheaper with keys and values rebuilt per head: a (query, key) pair then costs dn + dr + dv
// multiplications instead of 2 R + dr.  The latent rows a portion can see are gathered from the pages into one
// contiguous buffer per step (b2_latent_gather: for sequence i the positions k_lo[i] .. end, at rows cu_k[i] ..), the
// per-head keys and values come from two library GEMMs over that buffer, and b2_window_attention runs over them:
//   key of head h at gathered row g = [ kn[g, h, :dn] | kt[g, :dr] ]   (kt: the shared rotated part, a column slice of
//   the gathered rows), value v[g, h, :dv]; query = [ qn[t, h, :dn] | qr[t, h, :dr] ] from two buffers as well.
// One CTA = 64 consecutive rows of one sequence x one head, four warps of 16 rows, 64-key tiles staged through shared
// memory, mma.sync m16n8k16 with ldmatrix operands, online softmax in registers (exp2, scale folded in).  bf16; dn and dr
// multiples of 8, dn + dr and dv multiples of 16, dv <= 128.
constexpr int kWQ = 64, kWK = 64, kWMaxDVT = 8;

__global__ void latent_gather_kernel(const __nv_bfloat16* __restrict__ cache, const int32_t* __restrict__ block_tables, int max_nb,
                                     const int32_t* __restrict__ cu_k, const int32_t* __restrict__ k_lo, int n_seq, int bs, int Dc,
                                     __nv_bfloat16* __restrict__ out) {
    const int row = blockIdx.x;
    const int seq = b2::seq_of_row(cu_k, n_seq, row);
    const int j = k_lo[seq] + row - cu_k[seq];
    const __nv_bfloat16* src = cache + ((size_t)block_tables[(size_t)seq * max_nb + j / bs] * bs + j % bs) * Dc;
    __nv_bfloat16* dst = out + (size_t)row * Dc;
    for (int c = threadIdx.x * 8; c < Dc; c += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
}

__global__ void __launch_bounds__(128, 3)
window_attention_kernel(const __nv_bfloat16* __restrict__ qn, int64_t qn_row, int qn_head, const __nv_bfloat16* __restrict__ qr,
                        int64_t qr_row, int qr_head, const __nv_bfloat16* __restrict__ kn, const __nv_bfloat16* __restrict__ kt,
                        int64_t kt_row, const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ cu_q,
                        const int32_t* __restrict__ ctx_start, const int32_t* __restrict__ cu_k, const int32_t* __restrict__ k_lo,
                        int n_seq, int H, int dn, int dr, int dv, float scale_log2, int window,
                        const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out) {
    const int DK = dn + dr, LDK = DK + 8, LDV = dv + 8, dkt = DK / 16, dvt = dv / 16;
    extern __shared__ __align__(16) unsigned char lat_smem[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(lat_smem);       // [64][LDK]
    __nv_bfloat16* k_sm = q_sm + kWQ * LDK;                                 // [64][LDK]
    __nv_bfloat16* v_sm = k_sm + kWK * LDK;                                 // [64][LDV]
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    int seq = -1, t0 = 0;
    {
        int want = blockIdx.x;
        for (int s = 0; s < n_seq; ++s) {
            const int nt = (cu_q[s + 1] - cu_q[s] + kWQ - 1) / kWQ;
            if (want < nt) { seq = s; t0 = want * kWQ; break; }
            want -= nt;
        }
    }
    if (seq < 0) return;
    const int hh = blockIdx.y;
    const int r0 = cu_q[seq] + t0;
    const int rows = min(kWQ, cu_q[seq + 1] - r0);
    const int ctx = ctx_start[seq];
    if (ctx < 0) {
        for (int idx = tid; idx < rows * (dv / 8); idx += 128)
            *reinterpret_cast<uint4*>(out + ((size_t)(r0 + idx / (dv / 8)) * H + hh) * dv + (idx % (dv / 8)) * 8) = make_uint4(0, 0, 0, 0);
        return;
    }
    const int p0 = ctx + t0, p_last = p0 + rows - 1;
    const int first = k_lo[seq];                                            // position of the sequence's first gathered row
    const int klo = max(window > 0 ? max(p0 - window + 1, 0) : 0, first);
    const size_t g0 = (size_t)cu_k[seq];

    const int qv = DK / 8, nv8 = dn / 8;
    for (int idx = tid; idx < kWQ * qv; idx += 128) {
        const int r = idx / qv, c8 = idx % qv;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (r < rows) {
            x = c8 < nv8 ? *reinterpret_cast<const uint4*>(qn + (size_t)(r0 + r) * qn_row + (size_t)hh * qn_head + c8 * 8)
                         : *reinterpret_cast<const uint4*>(qr + (size_t)(r0 + r) * qr_row + (size_t)hh * qr_head + (c8 - nv8) * 8);
        }
        *reinterpret_cast<uint4*>(q_sm + r * LDK + c8 * 8) = x;
    }
    const int gq = lane >> 2, tq = lane & 3;
    const int i0 = p0 + w * 16 + gq, i1 = i0 + 8;
    const int lo0 = window > 0 ? max(i0 - window + 1, 0) : 0, lo1 = window > 0 ? max(i1 - window + 1, 0) : 0;
    const int w_first = p0 + w * 16, w_last = w_first + 15;
    const int w_lo = window > 0 ? max(w_first - window + 1, 0) : 0;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[2 * kWMaxDVT][4];
#pragma unroll
    for (int n = 0; n < 2 * kWMaxDVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const uint32_t q_base = b2::smem_u32(q_sm), k_base = b2::smem_u32(k_sm), v_base = b2::smem_u32(v_sm);
    const int vv = dv / 8;

    for (int kv0 = klo; kv0 <= p_last; kv0 += kWK) {
        __syncthreads();                                                    // the previous tile is consumed (and Q is stored)
        {                                                                   // two threads per key row: one address, then 16-byte copies
            const int key = tid >> 1, half = tid & 1, j = kv0 + key;
            __nv_bfloat16* kd = k_sm + key * LDK;
            __nv_bfloat16* vd = v_sm + key * LDV;
            if (j <= p_last) {
                const size_t g = g0 + (size_t)(j - first);
                const __nv_bfloat16* ks = kn + (g * H + hh) * dn;
                const __nv_bfloat16* ts = kt + g * kt_row;
                const __nv_bfloat16* vs = v + (g * H + hh) * dv;
                for (int c8 = half; c8 < nv8; c8 += 2) cp_async16(kd + c8 * 8, ks + c8 * 8);
                for (int c8 = half; c8 < qv - nv8; c8 += 2) cp_async16(kd + (nv8 + c8) * 8, ts + c8 * 8);
                for (int c8 = half; c8 < vv; c8 += 2) cp_async16(vd + c8 * 8, vs + c8 * 8);
            } else {
                for (int c8 = half; c8 < qv; c8 += 2) *reinterpret_cast<uint4*>(kd + c8 * 8) = make_uint4(0, 0, 0, 0);
                for (int c8 = half; c8 < vv; c8 += 2) *reinterpret_cast<uint4*>(vd + c8 * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (kv0 > w_last || kv0 + kWK - 1 < w_lo) continue;                 // no key of the tile is visible to the warp's rows
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll 4
        for (int kk = 0; kk < dkt; ++kk) {
            uint32_t a0, a1, a2, a3;
            b2::ldmatrix_x4(q_base + 2u * ((w * 16 + (lane & 15)) * LDK + kk * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
#pragma unroll
            for (int n2 = 0; n2 < 4; ++n2) {
                uint32_t b0, b1, b2_, b3;
                const int key = n2 * 16 + (lane >> 4) * 8 + (lane & 7), dim = kk * 16 + ((lane >> 3) & 1) * 8;
                b2::ldmatrix_x4(k_base + 2u * (key * LDK + dim), b0, b1, b2_, b3);
                b2::mma_bf16_16816(sc[2 * n2], a0, a1, a2, a3, b0, b1);
                b2::mma_bf16_16816(sc[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = kv0 + n * 8 + 2 * tq + (e & 1);
                const bool ok = e < 2 ? (j >= lo0 && j <= i0) : (j >= lo1 && j <= i1);
                sc[n][e] = ok ? sc[n][e] * scale_log2 : -INFINITY;
            }
            mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2f(m0 - mu0), c1 = exp2f(m1 - mu1);
        m0 = mn0;
        m1 = mn1;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            sc[n][0] = exp2f(sc[n][0] - mu0);
            sc[n][1] = exp2f(sc[n][1] - mu0);
            sc[n][2] = exp2f(sc[n][2] - mu1);
            sc[n][3] = exp2f(sc[n][3] - mu1);
            s0 += sc[n][0] + sc[n][1];
            s1 += sc[n][2] + sc[n][3];
        }
        l0 = l0 * c0 + s0;
        l1 = l1 * c1 + s1;
#pragma unroll
        for (int n = 0; n < 2 * kWMaxDVT; ++n) {
            o[n][0] *= c0;
            o[n][1] *= c0;
            o[n][2] *= c1;
            o[n][3] *= c1;
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a0 = b2::pack_bf16x2(sc[2 * ks][0], sc[2 * ks][1]),
                           a1 = b2::pack_bf16x2(sc[2 * ks][2], sc[2 * ks][3]);
            const uint32_t a2 = b2::pack_bf16x2(sc[2 * ks + 1][0], sc[2 * ks + 1][1]),
                           a3 = b2::pack_bf16x2(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < kWMaxDVT; ++n2) {
                if (n2 < dvt) {
                    uint32_t b0, b1, b2_, b3;
                    const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = n2 * 16 + (lane >> 4) * 8;
                    b2::ldmatrix_x4_trans(v_base + 2u * (key * LDV + col), b0, b1, b2_, b3);
                    b2::mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
                    b2::mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
                }
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int ra = w * 16 + gq, rb = ra + 8;
    float f0 = l0 > 0.f ? 1.f / l0 : 0.f, f1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (gate) {
        if (ra < rows) f0 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(r0 + ra) * gate_stride + hh]));
        if (rb < rows) f1 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(r0 + rb) * gate_stride + hh]));
    }
#pragma unroll
    for (int n = 0; n < 2 * kWMaxDVT; ++n) {
        const int col = n * 8 + 2 * tq;
        if (col < dv) {
            if (ra < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(r0 + ra) * H + hh) * dv + col) = b2::pack_bf16x2(o[n][0] * f0, o[n][1] * f0);
            if (rb < rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(r0 + rb) * H + hh) * dv + col) = b2::pack_bf16x2(o[n][2] * f1, o[n][3] * f1);
        }
    }
}

// out[row, :] = gate * sum_z o_z 2^(m_z - M) / sum_z l_z 2^(m_z - M) over the shares of a (token, head) row
__global__ void latent_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, int nsplit, int R, int H,
                                    const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out) {
    const int row = blockIdx.x;                                             // token * H + head
    const float* ml = ws_ml + (size_t)row * nsplit * 2;
    float M = -INFINITY;
    for (int z = 0; z < nsplit; ++z) M = fmaxf(M, ml[2 * z]);
    float L = 0.f;
    if (M > -INFINITY)
        for (int z = 0; z < nsplit; ++z) L += ml[2 * z + 1] * (ml[2 * z] == -INFINITY ? 0.f : exp2f(ml[2 * z] - M));
    float f = L > 0.f ? 1.f / L : 0.f;
    if (gate) f *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(row / H) * gate_stride + row % H]));
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float a = 0.f;
        if (L > 0.f)
            for (int z = 0; z < nsplit; ++z)
                if (ml[2 * z] > -INFINITY) a = fmaf(ws_o[((size_t)row * nsplit + z) * R + c], exp2f(ml[2 * z] - M), a);
        out[(size_t)row * R + c] = __float2bfloat16_rn(a * f);
    }
}

inline int latent_sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    return sms;
}

// Which kernel and how many shares of the key tiles per CTA row: a batch that cannot fill the GPU (decode rows) splits its
// keys over CTAs.  decode: every sequence has one row and the latent is wide enough for eight column slices.
struct LatentPlan {
    bool decode;
    int nsplit;
};
inline LatentPlan latent_plan(int T, int n_seq, int H, int R, int window, int max_nb, int bs) {
    LatentPlan p;
    p.decode = T == n_seq && R >= 128;
    const int Hc = H < kLQ ? H : kLQ, Gt = kLQ / Hc;
    const long ctas = p.decode ? (long)T * ((H + 15) / 16) : (long)(T < T / Gt + n_seq ? T : T / Gt + n_seq) * ((H + Hc - 1) / Hc);
    long keys = (long)max_nb * bs;
    const int span = p.decode ? 1 : Gt;
    if (window > 0 && window + span < keys) keys = window + span;
    const long tiles = (keys + kLK - 1) / kLK;
    long n = latent_sm_count() / (ctas > 0 ? ctas : 1);
    if (n > tiles / 2) n = tiles / 2;
    if (n > 16) n = 16;
    p.nsplit = n < 1 ? 1 : (int)n;
    return p;
}

template <int RT>
int launch_latent_mma(void* out, const void* qa, const void* cache, const int32_t* block_tables, int max_nb, const int32_t* cu_q,
                      const int32_t* ctx_start, int n_seq, int T, int H, int dr, int bs, float scale, int window, const void* gate,
                      int64_t gate_stride, bool decode, int nsplit, float* ws, cudaStream_t st) {
    const int Dc = 16 * RT + dr, Hc = H < kLQ ? H : kLQ, Gt = kLQ / Hc;
    const size_t tile = (size_t)kLK * (Dc + 8) * sizeof(__nv_bfloat16);
    const int stages = 3 * tile <= 227 * 1024 - 64 ? 2 : 1;                 // two key tiles in flight when they fit beside Q
    const size_t smem = (size_t)(1 + stages) * tile;
    auto kern = latent_attention_mma_kernel<RT>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int tiles = T < T / Gt + n_seq ? T : T / Gt + n_seq;   // upper bound on sum(ceil(len / Gt)); spare CTAs leave at once
    float* ws_o = ws;
    float* ws_ml = ws ? ws + (size_t)T * H * nsplit * 16 * RT : nullptr;
    if constexpr (RT >= 8) {
        if (decode) {
            const size_t dsm = (size_t)(16 + 2 * kLK) * (Dc + 8) * sizeof(__nv_bfloat16) + 16 * kPLD * sizeof(__nv_bfloat16) +
                               128 * sizeof(float);
            auto dk = latent_attention_decode_kernel<RT>;
            if (dsm > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(dk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dsm));
            dk<<<dim3(T, (H + 15) / 16, nsplit), 256, dsm, st>>>(
                static_cast<const __nv_bfloat16*>(qa), static_cast<const __nv_bfloat16*>(cache), block_tables, max_nb, cu_q, ctx_start,
                H, dr, bs, scale * 1.4426950408889634f, window, static_cast<const __nv_bfloat16*>(gate), gate_stride,
                static_cast<__nv_bfloat16*>(out), ws_o, ws_ml);
            if (nsplit > 1)
                latent_merge_kernel<<<T * H, 128, 0, st>>>(ws_o, ws_ml, nsplit, 16 * RT, H, static_cast<const __nv_bfloat16*>(gate),
                                                           gate_stride, static_cast<__nv_bfloat16*>(out));
            B2_CUDA_OK(cudaGetLastError());
            return B2_OK;
        }
    }
    kern<<<dim3(tiles, (H + Hc - 1) / Hc, nsplit), 256, smem, st>>>(
        static_cast<const __nv_bfloat16*>(qa), static_cast<const __nv_bfloat16*>(cache), block_tables, max_nb, cu_q, ctx_start,
        n_seq, H, Hc, dr, bs, scale * 1.4426950408889634f, window, stages, static_cast<const __nv_bfloat16*>(gate), gate_stride,
        static_cast<__nv_bfloat16*>(out), ws_o, ws_ml);
    if (nsplit > 1)
        latent_merge_kernel<<<T * H, 128, 0, st>>>(ws_o, ws_ml, nsplit, 16 * RT, H, static_cast<const __nv_bfloat16*>(gate),
                                                   gate_stride, static_cast<__nv_bfloat16*>(out));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

inline bool latent_mma_ok(int act_dtype, int R, int dr, const void* qa, const void* cache, const void* out) {
    return act_dtype == B2_ACT_BF16 && (R == 64 || R == 128 || R == 256 || R == 512) && dr % 16 == 0 && b2_aligned16(qa) &&
           b2_aligned16(cache) && b2_aligned16(out) && (size_t)(kLQ + kLK) * (R + dr + 8) * 2 <= 227 * 1024;
}

}  // namespace

// fp32 scratch (in floats) b2_latent_attention wants for this call; 0 when it needs none
extern "C" int64_t b2_latent_attention_workspace(int act_dtype, int T, int n_seq, int H, int R, int dr, int bs, int window,
                                                 int max_nb) {
    if (T <= 0 || n_seq <= 0 || H <= 0 || !latent_mma_ok(act_dtype, R, dr, nullptr, nullptr, nullptr)) return 0;
    const int n = latent_plan(T, n_seq, H, R, window, max_nb, bs).nsplit;
    return n > 1 ? (int64_t)T * H * n * (R + 2) : 0;
}

extern "C" int b2_latent_prep(const void* proj, int64_t proj_stride, int act_dtype, int T, int H, int dn, int dr, int rot_dims,
                              int R, int q_off, int dkv_off, const float* norm_w, float eps, const int32_t* positions,
                              const float* cos_sin, int max_pos, const int64_t* slots, int bs, void* qa, void* cache,
                              void* stream) {
    return b2_latent_prep_rows(proj, proj_stride, proj, proj_stride, act_dtype, T, H, dn, dr, rot_dims, R, q_off, dkv_off, norm_w,
                               eps, positions, cos_sin, max_pos, slots, bs, qa, cache, stream);
}

extern "C" int b2_latent_prep_rows(const void* q, int64_t q_stride, const void* kv, int64_t kv_stride, int act_dtype, int T, int H,
                                   int dn, int dr, int rot_dims, int R, int q_off, int dkv_off, const float* norm_w, float eps,
                                   const int32_t* positions, const float* cos_sin, int max_pos, const int64_t* slots, int bs,
                                   void* qa, void* cache, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && dn >= 0 && dr >= 0 && R > 0 && bs > 0 && q_off >= 0 && rot_dims >= 0 && rot_dims <= dr &&
                   rot_dims % 2 == 0 && max_pos > 0, B2_EINVAL, "latent_prep: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(q && positions && qa && (rot_dims == 0 || cos_sin), B2_EINVAL, "latent_prep: null pointer");
    B2_REQUIRE(dkv_off < 0 || (slots && cache && kv), B2_EINVAL,
               "latent_prep: a layer with a down-projection needs its rows, slots and its pool");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int work = H * dr > R ? H * dr : R;
    const int threads = work >= 2048 ? 256 : 128;
    const bool vec = q_stride % 4 == 0 && q_off % 4 == 0 && dn % 4 == 0 && dr % 4 == 0 && R % 4 == 0 && rot_dims % 4 == 0 &&
                     (dkv_off < 0 || (dkv_off % 4 == 0 && kv_stride % 4 == 0 && b2_aligned16(kv))) && b2_aligned16(q) &&
                     b2_aligned16(qa) && (dkv_off < 0 || b2_aligned16(cache));
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec)
            latent_prep_vec_kernel<A><<<T, threads, 0, st>>>(static_cast<const A*>(q), q_stride, static_cast<const A*>(kv), kv_stride,
                                                             H, dn, dr, rot_dims, R, q_off, dkv_off, norm_w, eps, positions,
                                                             cos_sin, max_pos, slots, static_cast<A*>(qa), static_cast<A*>(cache));
        else
            latent_prep_kernel<A><<<T, threads, 0, st>>>(static_cast<const A*>(q), q_stride, static_cast<const A*>(kv), kv_stride, H,
                                                         dn, dr, rot_dims, R, q_off, dkv_off, norm_w, eps, positions, cos_sin,
                                                         max_pos, slots, bs, static_cast<A*>(qa), static_cast<A*>(cache));
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_latent_attention(void* out, const void* qa, const void* cache, int act_dtype, const int32_t* block_tables,
                                   int max_nb, const int32_t* cu_q, const int32_t* ctx_start, int n_seq, int T, int H, int R,
                                   int dr, int bs, float scale, int window, const void* gate, int64_t gate_stride,
                                   float* workspace, int64_t workspace_floats, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && R > 0 && dr >= 0 && bs > 0 && window >= 0, B2_EINVAL, "latent_attention: bad sizes");
    B2_REQUIRE(R <= 32 * kMaxRPerLane, B2_EUNSUPPORTED, "latent_attention: latent size %d above %d", R, 32 * kMaxRPerLane);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && qa && cache && block_tables && cu_q && ctx_start, B2_EINVAL, "latent_attention: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (latent_mma_ok(act_dtype, R, dr, qa, cache, out)) {
        const LatentPlan plan = latent_plan(T, n_seq, H, R, window, max_nb, bs);
        int nsplit = plan.nsplit;
        if (nsplit > 1 && (!workspace || workspace_floats < (int64_t)T * H * nsplit * (R + 2))) nsplit = 1;
#define B2_LAT(RT)                                                                                                            \
    return launch_latent_mma<RT>(out, qa, cache, block_tables, max_nb, cu_q, ctx_start, n_seq, T, H, dr, bs, scale, window, gate, \
                                 gate_stride, plan.decode, nsplit, nsplit > 1 ? workspace : nullptr, st)
        if (R == 64) B2_LAT(4);
        if (R == 128) B2_LAT(8);
        if (R == 256) B2_LAT(16);
        B2_LAT(32);
#undef B2_LAT
    }
    const int warps = 4;
    const size_t smem = (size_t)warps * (R + dr) * sizeof(float);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "latent_attention: key size %d too large", R + dr);
    const int items = T * H, blocks = (items + warps - 1) / warps;
    B2_DISPATCH_ACT(act_dtype, A, (latent_attention_kernel<A><<<blocks, warps * 32, smem, st>>>(
        static_cast<const A*>(qa), static_cast<const A*>(cache), block_tables, max_nb, cu_q, ctx_start, n_seq, T, H, R, dr, bs,
        scale, window, static_cast<const A*>(gate), gate_stride, static_cast<A*>(out))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_latent_gather(void* out, const void* cache, const int32_t* block_tables, int max_nb, const int32_t* cu_k,
                                const int32_t* k_lo, int n_seq, int N, int bs, int Dc, void* stream) {
    B2_REQUIRE(N >= 0 && n_seq >= 0 && bs > 0 && Dc > 0 && Dc % 8 == 0, B2_EINVAL, "latent_gather: bad sizes (row width %d)", Dc);
    if (N == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && cache && block_tables && cu_k && k_lo && b2_aligned16(out) && b2_aligned16(cache), B2_EINVAL,
               "latent_gather: null or unaligned pointer");
    latent_gather_kernel<<<N, 64, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(cache), block_tables, max_nb, cu_k, k_lo, n_seq, bs, Dc, static_cast<__nv_bfloat16*>(out));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_window_attention(void* out, const void* qn, int64_t qn_row, int qn_head, const void* qr, int64_t qr_row,
                                   int qr_head, const void* kn, const void* kt, int64_t kt_row, const void* v,
                                   const int32_t* cu_q, const int32_t* ctx_start, const int32_t* cu_k, const int32_t* k_lo,
                                   int n_seq, int T, int H, int dn, int dr, int dv, float scale, int window, const void* gate,
                                   int64_t gate_stride, void* stream) {
    B2_REQUIRE(T >= 0 && n_seq >= 0 && H > 0 && dn >= 0 && dr >= 0 && dv > 0 && window >= 0, B2_EINVAL, "window_attention: bad sizes");
    B2_REQUIRE(dn % 8 == 0 && dr % 8 == 0 && (dn + dr) % 16 == 0 && dn + dr > 0 && dv % 16 == 0 && dv <= 16 * kWMaxDVT, B2_EUNSUPPORTED,
               "window_attention: head sizes %d + %d / %d", dn, dr, dv);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && qn && qr && kn && kt && v && cu_q && ctx_start && cu_k && k_lo, B2_EINVAL, "window_attention: null pointer");
    B2_REQUIRE(b2_aligned16(out) && b2_aligned16(qn) && b2_aligned16(qr) && b2_aligned16(kn) && b2_aligned16(kt) && b2_aligned16(v) &&
                   qn_row % 8 == 0 && qn_head % 8 == 0 && qr_row % 8 == 0 && qr_head % 8 == 0 && kt_row % 8 == 0, B2_EINVAL,
               "window_attention: pointers and strides must keep 16-byte alignment");
    const size_t smem = (size_t)((kWQ + kWK) * (dn + dr + 8) + kWK * (dv + 8)) * sizeof(__nv_bfloat16);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "window_attention: key size %d too large", dn + dr);
    if (smem > 48 * 1024)
        B2_CUDA_OK(cudaFuncSetAttribute(window_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int tiles = T / kWQ + n_seq;
    window_attention_kernel<<<dim3(tiles, H), 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(qn), qn_row, qn_head, static_cast<const __nv_bfloat16*>(qr), qr_row, qr_head,
        static_cast<const __nv_bfloat16*>(kn), static_cast<const __nv_bfloat16*>(kt), kt_row, static_cast<const __nv_bfloat16*>(v), cu_q,
        ctx_start, cu_k, k_lo, n_seq, H, dn, dr, dv, scale * 1.4426950408889634f, window, static_cast<const __nv_bfloat16*>(gate),
        gate_stride, static_cast<__nv_bfloat16*>(out));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
