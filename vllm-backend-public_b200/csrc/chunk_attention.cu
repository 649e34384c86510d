// chunk_attention.cu -- softmax attention without a rotation over a paged cache, with three parameters that other
// designs can set independently:
//   * per-head RMS norm of queries and keys (a plain weight of size dk shared by the heads),
//   * a block-local causal mask: position i sees j <= i with floor(j / chunk) == floor(i / chunk), blocks counted from
//     position 0 of the sequence (chunk = 0: plain causal),
//   * a sink: `sink` is added to the softmax denominator as exp(sink_logit - max), a key with no value (sink = 0: none;
//     sink = 1 with logit 0 gives p_j = exp(s_j) / (1 + sum exp(s))); the logit may also be one learned number per
//     query head (sink_logits [H], not scaled),
//   * a sliding window that keeps the first tokens: position i sees j <= i with i - j < window or j < keep_first
//     (window = 0: no window).  A query then reads the kept keys and its window's keys and nothing between them,
//   * a sigmoid gate per (token, head) on the head's output.
// Key size dk and value size dv are independent; K and V live in separate paged pools
//   k_cache [num_blocks, G, bs, dk],  v_cache [num_blocks, G, bs, dv]      (activation type).
//
//   b2_qknorm_cache      per token: q heads normalised into q_out; k heads normalised and written to the K pool, v copied
//                        to the V pool, through the token's slot (slot < 0 skips the write).
//   b2_qk_prep_cache     the same pass with the norm optional and a query temperature: the query of the token at position p
//                        is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) (fp32), so queries sharpen as the
//                        context grows in steps of `every` positions (coef = 0: none).
//   b2_qk_rope_cache     rows [q | k] or [q | k | v]: the first rot_dims entries of every q and k head are rotated by the
//                        token's position (pairs (i, i + rot_dims/2) or (2i, 2i + 1); fp32 table [max_pos, rot_dims] =
//                        cos | sin halves), q to q_out, rotated k to the K pool; the V pool receives v, or, for designs
//                        whose values ARE the keys, the k heads as projected (before the rotation).
//   b2_chunk_attention   per (token, head) one warp: scores of 32 keys at a time (a lane per key), online softmax in fp32
//                        seeded with the sink, P.V with a lane per value column.  With the mask a query touches at most
//                        `chunk` keys wherever it stands, so prompt chunks and decode rows run the same kernel; a decode
//                        row is a sequence with one query.
// Sequences are described like everywhere in this library: rows cu_q[i] .. cu_q[i+1]-1, ctx_start[i] cached tokens
// before them (< 0: padding, output rows are zeroed), block_tables[i, :].
#include "b2_act.cuh"

namespace {

constexpr int kMaxDvPerLane = 16;                    // dv <= 512

// The keys a query at position `pos` may see, as one compact index range [0, n): first the kept keys lo .. lo+nfirst-1
// (the sequence's first tokens that lie before the window), then wlo .. pos.  Without a window nfirst = 0 and wlo = lo.
struct KeySpan {
    int lo, nfirst, wlo, n;
    __device__ __forceinline__ int key(int c) const { return c < nfirst ? lo + c : wlo + (c - nfirst); }
};
__device__ __forceinline__ KeySpan key_span(int pos, int last, int chunk, int window, int keep_first) {
    KeySpan s;
    s.lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    s.wlo = window > 0 ? max(s.lo, pos - window + 1) : s.lo;
    s.nfirst = (window > 0 && keep_first > s.lo) ? max(0, min(keep_first, s.wlo) - s.lo) : 0;
    s.n = s.nfirst + (last - s.wlo + 1);
    return s;
}
// what the masks leave of key j for the query at position i
__device__ __forceinline__ bool key_visible(int i, int j, int lo_i, int window, int keep_first) {
    return j <= i && j >= lo_i && (window <= 0 || i - j < window || j < keep_first);
}

// Rows [q | k] (+ [v]): partial rotation of the q and k heads, K (rotated) and V pool writes; see the file comment.
template <typename T>
__global__ void qk_rope_cache_kernel(const T* __restrict__ qkv, int64_t qkv_stride, int H, int G, int dk, int dv, bool v_from_k,
                                     int rot_dims, bool interleaved, const int32_t* __restrict__ positions,
                                     const float* __restrict__ cos_sin, int max_pos, const int64_t* __restrict__ slots, int bs,
                                     T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache) {
    const int row = blockIdx.x;
    const T* src = qkv + (size_t)row * qkv_stride;
    int pos = positions[row];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot_dims;
    const int half = rot_dims / 2;
    const int64_t slot = slots[row];
    const int64_t blk = slot >= 0 ? slot / bs : 0;
    const int off = slot >= 0 ? (int)(slot % bs) : 0;
    // q and k heads: element i of a head
    for (int idx = threadIdx.x; idx < (H + G) * dk; idx += blockDim.x) {
        const int hd = idx / dk, i = idx % dk;
        if (hd >= H && slot < 0) continue;
        const T* v = src + (size_t)hd * dk;
        float x = b2::ld(v + i);
        if (i < rot_dims) {
            int pr, partner;
            bool second;
            if (interleaved) { pr = i >> 1; partner = i ^ 1; second = i & 1; }
            else { second = i >= half; pr = second ? i - half : i; partner = second ? i - half : i + half; }
            const float c = cs[pr], sn = cs[half + pr], other = b2::ld(v + partner);
            x = second ? fmaf(x, c, other * sn) : fmaf(x, c, -other * sn);
        }
        T* dst = hd < H ? q_out + ((size_t)row * H + hd) * dk : k_cache + (((size_t)blk * G + (hd - H)) * bs + off) * dk;
        b2::st(dst + i, x);
    }
    if (slot < 0) return;
    const T* vsrc = v_from_k ? src + (size_t)H * dk : src + (size_t)(H + G) * dk;
    for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) {
        const int g = idx / dv, i = idx % dv;
        v_cache[(((size_t)blk * G + g) * bs + off) * dv + i] = vsrc[idx];
    }
}

// The same with four entries per access (8 or 16 bytes): every size a multiple of four, the rotated entries a multiple of
// eight in the (i, i + rot_dims/2) layout so that a group of four and its partners never straddle the halves.
template <typename T>
__global__ void __launch_bounds__(256)
qk_rope_cache_vec_kernel(const T* __restrict__ qkv, int64_t qkv_stride, int H, int G, int dk, int dv, bool v_from_k, int rot_dims,
                         bool interleaved, const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, int max_pos,
                         const int64_t* __restrict__ slots, int bs, T* __restrict__ q_out, T* __restrict__ k_cache,
                         T* __restrict__ v_cache) {
    const int row = blockIdx.x;
    const T* src = qkv + (size_t)row * qkv_stride;
    int pos = positions[row];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float* cs = cos_sin + (size_t)pos * rot_dims;
    const int half = rot_dims / 2;
    const int64_t slot = slots[row];
    const int64_t blk = slot >= 0 ? slot / bs : 0;
    const int off = slot >= 0 ? (int)(slot % bs) : 0;
    const int per = dk / 4, nqk = (slot >= 0 ? H + G : H) * per;
    for (int idx = threadIdx.x; idx < nqk; idx += blockDim.x) {
        const int hd = idx / per, i = (idx % per) * 4;
        const T* v = src + (size_t)hd * dk;
        float x[4];
        b2::ld4(v + i, x);
        if (i < rot_dims) {
            if (interleaved) {
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    const float co = cs[(i + c) >> 1], si = cs[half + ((i + c) >> 1)], a = x[c], b = x[c + 1];
                    x[c] = fmaf(a, co, -b * si);
                    x[c + 1] = fmaf(b, co, a * si);
                }
            } else {
                const bool second = i >= half;
                const int pr = second ? i - half : i;
                float y[4];
                b2::ld4(v + (second ? i - half : i + half), y);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float co = cs[pr + c], si = cs[half + pr + c];
                    x[c] = second ? fmaf(x[c], co, y[c] * si) : fmaf(x[c], co, -y[c] * si);
                }
            }
        }
        T* dst = hd < H ? q_out + ((size_t)row * H + hd) * dk : k_cache + (((size_t)blk * G + (hd - H)) * bs + off) * dk;
        b2::st4(dst + i, x);
    }
    if (slot < 0) return;
    const T* vsrc = v_from_k ? src + (size_t)H * dk : src + (size_t)(H + G) * dk;
    const int pv = dv / 4;
    for (int idx = threadIdx.x; idx < G * pv; idx += blockDim.x) {
        const int g = idx / pv, i = (idx % pv) * 4;
        float x[4];
        b2::ld4(vsrc + (size_t)g * dv + i, x);
        b2::st4(v_cache + (((size_t)blk * G + g) * bs + off) * dv + i, x);
    }
}

template <typename T>
__global__ void qknorm_cache_kernel(const T* __restrict__ qkv, int64_t qkv_stride, int H, int G, int dk, int dv,
                                    const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                    const int64_t* __restrict__ slots, int bs, T* __restrict__ q_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, bool norm,
                                    const int32_t* __restrict__ positions, float temp_coef, int temp_every) {
    const int row = blockIdx.x;
    float q_factor = 1.f;
    if (positions && temp_coef != 0.f) q_factor = 1.f + temp_coef * logf((float)((positions[row] + 1) / temp_every + 1));
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const T* src = qkv + (size_t)row * qkv_stride;
    const int64_t slot = slots[row];
    const int64_t blk = slot >= 0 ? slot / bs : 0;
    const int off = slot >= 0 ? (int)(slot % bs) : 0;
    for (int hd = wid; hd < H + 2 * G; hd += nw) {
        if (hd < H + G) {                            // q or k head: x / sqrt(mean(x^2) + eps) * w
            const T* v = src + (size_t)hd * dk;
            float inv = hd < H ? q_factor : 1.f;
            if (norm) {
                float ss = 0.f;
                for (int i = lane; i < dk; i += 32) {
                    const float x = b2::ld(v + i);
                    ss = fmaf(x, x, ss);
                }
                inv = rsqrtf(b2::warp_sum(ss) / (float)dk + eps) * (hd < H ? q_factor : 1.f);
            }
            T* dst;
            const float* w;
            if (hd < H) {
                dst = q_out + ((size_t)row * H + hd) * dk;
                w = q_w;
            } else {
                if (slot < 0) continue;
                dst = k_cache + (((size_t)blk * G + (hd - H)) * bs + off) * dk;
                w = k_w;
            }
            for (int i = lane; i < dk; i += 32) b2::st(dst + i, b2::ld(v + i) * inv * (w ? w[i] : 1.f));
        } else {
            if (slot < 0) continue;
            const int g = hd - H - G;
            const T* v = src + (size_t)(H + G) * dk + (size_t)g * dv;
            T* dst = v_cache + (((size_t)blk * G + g) * bs + off) * dv;
            for (int i = lane; i < dv; i += 32) dst[i] = v[i];
        }
    }
}

template <typename T>
__global__ void chunk_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                       const int32_t* __restrict__ block_tables, int max_nb,
                                       const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start, int n_seq,
                                       int rows, int H, int G, int dk, int dv, int bs, float scale, int chunk, int window,
                                       int keep_first, float sink, float sink_logit, const float* __restrict__ sink_logits,
                                       const T* __restrict__ gate, int64_t gate_stride, int skip_rows_from,
                                       T* __restrict__ out) {
    extern __shared__ float q_sm[];                  // [warps, dk]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int item = blockIdx.x * (blockDim.x >> 5) + wid;       // (row, head)
    if (item >= rows * H) return;
    const int row = item / H, hh = item % H;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int ctx = ctx_start[seq];
    T* dst = out + (size_t)item * dv;
    if (skip_rows_from > 0 && ctx >= 0 && cu_q[seq + 1] - cu_q[seq] >= skip_rows_from) return;    // the tile kernel's
    if (ctx < 0) {
        for (int i = lane; i < dv; i += 32) b2::st(dst + i, 0.f);
        return;
    }
    const int pos = ctx + row - cu_q[seq];
    const KeySpan span = key_span(pos, pos, chunk, window, keep_first);
    const int g = hh / (H / G);
    float* qs = q_sm + (size_t)wid * dk;
    const T* qv = q + (size_t)item * dk;
    for (int i = lane; i < dk; i += 32) qs[i] = b2::ld(qv + i) * scale;
    __syncwarp();
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    float m = sink > 0.f ? (sink_logits ? sink_logits[hh] : sink_logit) : -INFINITY, l = sink;      // the sink seeds the running maximum and denominator
    float acc[kMaxDvPerLane];
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] = 0.f;
    for (int c0 = 0; c0 < span.n; c0 += 32) {
        const bool in = c0 + lane < span.n;
        const int j = span.key(c0 + lane);
        float s = -INFINITY;
        size_t vbase = 0;
        if (in) {
            const size_t tile = ((size_t)bt[j / bs] * G + g) * bs + (j % bs);
            const T* kr = k_cache + tile * dk;
            vbase = tile * dv;
            float d = 0.f;
            for (int i = 0; i < dk; ++i) d = fmaf(qs[i], b2::ld(kr + i), d);
            s = d;
        }
        const float m_new = fmaxf(m, b2::warp_max(s));
        const float corr = m == -INFINITY ? 0.f : __expf(m - m_new);
        const float p = in ? __expf(s - m_new) : 0.f;
        l = l * corr + b2::warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] *= corr;
        const int nk = min(32, span.n - c0);
        for (int kk = 0; kk < nk; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const size_t vb = __shfl_sync(0xffffffffu, (unsigned long long)vbase, kk);
            const T* vr = v_cache + vb;
#pragma unroll
            for (int c = 0; c < kMaxDvPerLane; ++c) {
                const int i = lane + 32 * c;
                if (i < dv) acc[c] = fmaf(pk, b2::ld(vr + i), acc[c]);
            }
        }
    }
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (gate) inv *= b2::sigmoid_f(b2::ld(gate + (size_t)row * gate_stride + hh));
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) b2::st(dst + i, acc[c] * inv);
    }
}

// ------------------------------------------------------------------------------------------------- grouped decode kernel
// bf16 rows that the tiled kernel does not take (decode rows, short portions): one CTA per (row, kv head) serves ALL the
// query heads of that kv head, so K and V are read once per group instead of once per head.  Four warps share the visible
// keys 32 at a time (a lane per key, 16-byte loads of its K row, one dot product per query head), keep an online softmax
// per head, accumulate P.V with a lane per pair of value columns, and merge through shared memory; the sink enters
// through warp 0's initial state.  Up to kGroupMaxHeads query heads per pass (more: further passes over the keys).
constexpr int kGroupMaxHeads = 8, kGroupMaxPairs = 4;      // dv <= 256

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(b2::smem_u32(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(128)
chunk_attention_group_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                             const __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ block_tables, int max_nb,
                             const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start, int n_seq, int H, int G,
                             int dk, int dv, int bs, float scale, int chunk, int window, int keep_first, float sink,
                             float sink_logit, const float* __restrict__ sink_logits, const __nv_bfloat16* __restrict__ gate,
                             int64_t gate_stride, int skip_rows_from, __nv_bfloat16* __restrict__ out) {
    // q [QH][dk] | per warp: m [QH], l [QH], acc [QH][dv] | per warp: K tile [32][dk + 8], V tile [32][dv] (bf16)
    extern __shared__ __align__(16) float grp_sm[];
    const int row = blockIdx.x, g = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int seq = b2::seq_of_row(cu_q, n_seq, row);
    const int ctx = ctx_start[seq];
    const int QHall = H / G;
    if (skip_rows_from > 0 && ctx >= 0 && cu_q[seq + 1] - cu_q[seq] >= skip_rows_from) return;    // the tile kernel's
    if (ctx < 0) {
        for (int i = tid; i < QHall * dv; i += 128) out[((size_t)row * H + (size_t)g * QHall) * dv + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = ctx + row - cu_q[seq];
    const KeySpan span = key_span(pos, pos, chunk, window, keep_first);
    const int32_t* bt = block_tables + (size_t)seq * max_nb;
    const int npairs = dv / 2;
    for (int h0 = 0; h0 < QHall; h0 += kGroupMaxHeads) {
        const int QH = min(kGroupMaxHeads, QHall - h0);
        float* qs = grp_sm;
        float* part = grp_sm + kGroupMaxHeads * dk;
        const int ldk = dk + 8;                            // 16 bytes of padding: the lanes' rows spread over the banks
        __nv_bfloat16* kt = reinterpret_cast<__nv_bfloat16*>(part + 4 * kGroupMaxHeads * (2 + dv)) + (size_t)w * 32 * (ldk + dv);
        __nv_bfloat16* vt = kt + 32 * ldk;
        __syncthreads();                                   // a previous pass is done with the shared memory
        for (int i = tid; i < QH * dk; i += 128)
            qs[i] = __bfloat162float(q[((size_t)row * H + (size_t)g * QHall + h0) * dk + i]) * scale;
        __syncthreads();
        float m[kGroupMaxHeads], l[kGroupMaxHeads], acc[kGroupMaxHeads][kGroupMaxPairs][2];
#pragma unroll
        for (int h = 0; h < kGroupMaxHeads; ++h) {
            m[h] = (w == 0 && sink > 0.f) ? (sink_logits ? sink_logits[g * QHall + h0 + min(h, QH - 1)] : sink_logit) : -INFINITY;
            l[h] = w == 0 ? sink : 0.f;
#pragma unroll
            for (int c = 0; c < kGroupMaxPairs; ++c) acc[h][c][0] = acc[h][c][1] = 0.f;
        }
        for (int c0 = w * 32; c0 < span.n; c0 += 128) {
            const bool valid = c0 + lane < span.n;
            float sc[kGroupMaxHeads];
#pragma unroll
            for (int h = 0; h < kGroupMaxHeads; ++h) sc[h] = 0.f;
            // the warp's 32 keys: K and V rows gathered from the pages with every 16-byte copy in flight at once
            const int nk = min(32, span.n - c0);
            __syncwarp();                                  // the previous tile has been read
            for (int idx = lane; idx < nk * (dk / 8); idx += 32) {
                const int key = idx / (dk / 8), c = (idx % (dk / 8)) * 8, jk = span.key(c0 + key);
                cp_async16(kt + key * ldk + c, k_cache + (((size_t)bt[jk / bs] * G + g) * bs + jk % bs) * dk + c);
            }
            for (int idx = lane; idx < nk * (dv / 8); idx += 32) {
                const int key = idx / (dv / 8), c = (idx % (dv / 8)) * 8, jk = span.key(c0 + key);
                cp_async16(vt + key * dv + c, v_cache + (((size_t)bt[jk / bs] * G + g) * bs + jk % bs) * dv + c);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            if (valid) {
                const __nv_bfloat16* kr = kt + lane * ldk;
                for (int c = 0; c < dk; c += 8) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(kr + c);
                    const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
                    float kf[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        kf[2 * e] = __uint_as_float(wds[e] << 16);
                        kf[2 * e + 1] = __uint_as_float(wds[e] & 0xffff0000u);
                    }
#pragma unroll
                    for (int h = 0; h < kGroupMaxHeads; ++h) {
                        if (h < QH) {
                            const float4 qa = *reinterpret_cast<const float4*>(qs + h * dk + c);
                            const float4 qb = *reinterpret_cast<const float4*>(qs + h * dk + c + 4);
                            sc[h] = fmaf(qa.x, kf[0], sc[h]); sc[h] = fmaf(qa.y, kf[1], sc[h]);
                            sc[h] = fmaf(qa.z, kf[2], sc[h]); sc[h] = fmaf(qa.w, kf[3], sc[h]);
                            sc[h] = fmaf(qb.x, kf[4], sc[h]); sc[h] = fmaf(qb.y, kf[5], sc[h]);
                            sc[h] = fmaf(qb.z, kf[6], sc[h]); sc[h] = fmaf(qb.w, kf[7], sc[h]);
                        }
                    }
                }
            }
            float pr[kGroupMaxHeads];
#pragma unroll
            for (int h = 0; h < kGroupMaxHeads; ++h) {
                pr[h] = 0.f;
                if (h < QH) {
                    const float x = valid ? sc[h] : -INFINITY;
                    const float mn = fmaxf(m[h], b2::warp_max(x));          // finite: the tile has at least one key
                    const float corr = m[h] == -INFINITY ? 0.f : __expf(m[h] - mn);
                    pr[h] = valid ? __expf(x - mn) : 0.f;
                    l[h] = l[h] * corr + b2::warp_sum(pr[h]);
                    m[h] = mn;
#pragma unroll
                    for (int c = 0; c < kGroupMaxPairs; ++c) {
                        acc[h][c][0] *= corr;
                        acc[h][c][1] *= corr;
                    }
                }
            }
            for (int kk = 0; kk < nk; ++kk) {
                float vx[kGroupMaxPairs], vy[kGroupMaxPairs];
#pragma unroll
                for (int c = 0; c < kGroupMaxPairs; ++c) {
                    const int pi = lane + 32 * c;
                    vx[c] = vy[c] = 0.f;
                    if (pi < npairs) {
                        const uint32_t wd = *reinterpret_cast<const uint32_t*>(vt + kk * dv + 2 * pi);
                        vx[c] = __uint_as_float(wd << 16);
                        vy[c] = __uint_as_float(wd & 0xffff0000u);
                    }
                }
#pragma unroll
                for (int h = 0; h < kGroupMaxHeads; ++h) {
                    if (h < QH) {
                        const float ph = __shfl_sync(0xffffffffu, pr[h], kk);
#pragma unroll
                        for (int c = 0; c < kGroupMaxPairs; ++c) {
                            acc[h][c][0] = fmaf(ph, vx[c], acc[h][c][0]);
                            acc[h][c][1] = fmaf(ph, vy[c], acc[h][c][1]);
                        }
                    }
                }
            }
        }
        // merge the four warps
        float* mine = part + (size_t)w * kGroupMaxHeads * (2 + dv);
#pragma unroll
        for (int h = 0; h < kGroupMaxHeads; ++h) {
            if (h < QH) {
                if (lane == 0) {
                    mine[h * (2 + dv)] = m[h];
                    mine[h * (2 + dv) + 1] = l[h];
                }
#pragma unroll
                for (int c = 0; c < kGroupMaxPairs; ++c) {
                    const int pi = lane + 32 * c;
                    if (pi < npairs) {
                        mine[h * (2 + dv) + 2 + 2 * pi] = acc[h][c][0];
                        mine[h * (2 + dv) + 3 + 2 * pi] = acc[h][c][1];
                    }
                }
            }
        }
        __syncthreads();
        for (int i = tid; i < QH * dv; i += 128) {
            const int h = i / dv, col = i % dv;
            float M = -INFINITY;
            for (int x = 0; x < 4; ++x) M = fmaxf(M, part[((size_t)x * kGroupMaxHeads + h) * (2 + dv)]);
            float L = 0.f, O = 0.f;
            if (M > -INFINITY) {
                for (int x = 0; x < 4; ++x) {
                    const float* px = part + ((size_t)x * kGroupMaxHeads + h) * (2 + dv);
                    const float f = px[0] == -INFINITY ? 0.f : __expf(px[0] - M);
                    L = fmaf(px[1], f, L);
                    O = fmaf(px[2 + col], f, O);
                }
            }
            float res = L > 0.f ? O / L : 0.f;
            if (gate) res *= b2::sigmoid_f(__bfloat162float(gate[(size_t)row * gate_stride + (size_t)g * QHall + h0 + h]));
            out[((size_t)row * H + (size_t)g * QHall + h0 + h) * dv + col] = __float2bfloat16_rn(res);
        }
    }
}

// ------------------------------------------------------------------------------------------------- tiled prompt kernel
// bf16, dk and dv multiples of 16: one CTA = 64 consecutive query rows of one sequence x one head, four warps of 16 rows.
// Keys are walked 64 at a time from the first row's block start to the last row's position (at most chunk + 63 keys
// with a mask, the whole prefix without): K and V tiles are gathered from the pages into shared memory, S = Q K^T and
// O += P V run on mma.sync m16n8k16 with ldmatrix operands, the online softmax lives in the accumulator registers
// (exp2 with the scale folded in, the sink seeding the running maximum and denominator).  Sequences with fewer than
// kTileMinRows rows (decode rows) are left to the warp kernel above.
constexpr int kTQ = 64, kTK = 64, kTileMinRows = 16;

template <int DKT, int DVT>
__global__ void __launch_bounds__(128)
chunk_attention_tile_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                            const __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ block_tables, int max_nb,
                            const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_start, int n_seq, int H, int G,
                            int bs, float scale_log2, int chunk, int window, int keep_first, float sink,
                            float sink_logit_log2, const float* __restrict__ sink_logits,
                            const __nv_bfloat16* __restrict__ gate, int64_t gate_stride, __nv_bfloat16* __restrict__ out) {
    constexpr int DK = 16 * DKT, DV = 16 * DVT, LDK = DK + 8, LDV = DV + 8;
    extern __shared__ __align__(16) unsigned char tile_smem[];
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(tile_smem);      // [64][LDK]
    __nv_bfloat16* k_sm = q_sm + kTQ * LDK;                                 // [64][LDK]
    __nv_bfloat16* v_sm = k_sm + kTK * LDK;                                 // [64][LDV]
    __shared__ int s_info[2];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    if (tid == 0) {
        int want = blockIdx.x, found = -1, t0 = 0;
        for (int s = 0; s < n_seq; ++s) {
            const int len = cu_q[s + 1] - cu_q[s];
            if (len < kTileMinRows || ctx_start[s] < 0) continue;
            const int nt = (len + kTQ - 1) / kTQ;
            if (want < nt) { found = s; t0 = want * kTQ; break; }
            want -= nt;
        }
        s_info[0] = found;
        s_info[1] = t0;
    }
    __syncthreads();
    const int seq = s_info[0], t0 = s_info[1];
    if (seq < 0) return;
    const int hh = blockIdx.y, g = hh / (H / G);
    const int r0 = cu_q[seq] + t0;
    const int rows = min(kTQ, cu_q[seq + 1] - r0);
    const int p0 = ctx_start[seq] + t0, p_last = p0 + rows - 1;
    // the union of what the tile's rows see, as one compact range: kept first keys, then the first row's window .. p_last
    const KeySpan span = key_span(p0, p_last, chunk, window, keep_first);
    const int32_t* bt = block_tables + (size_t)seq * max_nb;

    for (int idx = tid; idx < kTQ * (DK / 8); idx += 128) {
        const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(r0 + r) * H + hh) * DK + c);
        *reinterpret_cast<uint4*>(q_sm + r * LDK + c) = v;
    }
    const int gq = lane >> 2, tq = lane & 3;
    const int i0 = p0 + w * 16 + gq, i1 = i0 + 8;                           // positions of this thread's two rows
    const int lo0 = chunk > 0 ? (i0 / chunk) * chunk : 0, lo1 = chunk > 0 ? (i1 / chunk) * chunk : 0;
    const int w_first = p0 + w * 16, w_last = w_first + 15;
    const int w_clo = chunk > 0 ? (w_first / chunk) * chunk : 0;
    const int w_lo = window > 0 ? max(w_clo, w_first - window + 1) : w_clo;   // the lowest key of the warp's rows' windows
    if (sink_logits) sink_logit_log2 = sink_logits[hh] * 1.4426950408889634f;
    float m0 = sink > 0.f ? sink_logit_log2 : -INFINITY, m1 = m0;
    float l0 = tq == 0 ? sink : 0.f, l1 = l0;                               // partial sums per lane; the sink counted once
    float o[2 * DVT][4];
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    const uint32_t q_base = b2::smem_u32(q_sm), k_base = b2::smem_u32(k_sm), v_base = b2::smem_u32(v_sm);

    for (int kv0 = 0; kv0 < span.n; kv0 += kTK) {                           // kv0: compact key index of the tile's first key
        __syncthreads();                                                    // the previous tile is consumed (and Q is stored)
        for (int idx = tid; idx < kTK * (DK / 8); idx += 128) {
            const int key = idx / (DK / 8), c = (idx % (DK / 8)) * 8, j = span.key(kv0 + key);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j <= p_last) v = *reinterpret_cast<const uint4*>(k_cache + (((size_t)bt[j / bs] * G + g) * bs + j % bs) * DK + c);
            *reinterpret_cast<uint4*>(k_sm + key * LDK + c) = v;
        }
        for (int idx = tid; idx < kTK * (DV / 8); idx += 128) {
            const int key = idx / (DV / 8), c = (idx % (DV / 8)) * 8, j = span.key(kv0 + key);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j <= p_last) v = *reinterpret_cast<const uint4*>(v_cache + (((size_t)bt[j / bs] * G + g) * bs + j % bs) * DV + c);
            *reinterpret_cast<uint4*>(v_sm + key * LDV + c) = v;
        }
        __syncthreads();
        {   // nothing in this tile is visible to the warp's rows: all keys after them, or all before their windows and not kept
            const int j_min = span.key(kv0), j_max = span.key(min(kv0 + kTK, span.n) - 1);
            if (j_min > w_last || (j_max < w_lo && (window <= 0 || j_min >= keep_first))) continue;
        }
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < DKT; ++kk) {
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
                const int j = span.key(kv0 + n * 8 + 2 * tq + (e & 1));
                const bool ok = e < 2 ? key_visible(i0, j, lo0, window, keep_first) : key_visible(i1, j, lo1, window, keep_first);
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
        for (int n = 0; n < 2 * DVT; ++n) {
            o[n][0] *= c0;
            o[n][1] *= c0;
            o[n][2] *= c1;
            o[n][3] *= c1;
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a0 = b2::pack_bf16x2(sc[2 * ks][0], sc[2 * ks][1]), a1 = b2::pack_bf16x2(sc[2 * ks][2], sc[2 * ks][3]);
            const uint32_t a2 = b2::pack_bf16x2(sc[2 * ks + 1][0], sc[2 * ks + 1][1]),
                           a3 = b2::pack_bf16x2(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
            for (int n2 = 0; n2 < DVT; ++n2) {
                uint32_t b0, b1, b2_, b3;
                const int key = ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), col = n2 * 16 + (lane >> 4) * 8;
                b2::ldmatrix_x4_trans(v_base + 2u * (key * LDV + col), b0, b1, b2_, b3);
                b2::mma_bf16_16816(o[2 * n2], a0, a1, a2, a3, b0, b1);
                b2::mma_bf16_16816(o[2 * n2 + 1], a0, a1, a2, a3, b2_, b3);
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int ra = w * 16 + gq, rb = ra + 8;
    if (gate) {
        if (ra < rows) inv0 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(r0 + ra) * gate_stride + hh]));
        if (rb < rows) inv1 *= b2::sigmoid_f(__bfloat162float(gate[(size_t)(r0 + rb) * gate_stride + hh]));
    }
#pragma unroll
    for (int n = 0; n < 2 * DVT; ++n) {
        const int col = n * 8 + 2 * tq;
        if (ra < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(r0 + ra) * H + hh) * DV + col) = b2::pack_bf16x2(o[n][0] * inv0, o[n][1] * inv0);
        if (rb < rows)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(r0 + rb) * H + hh) * DV + col) = b2::pack_bf16x2(o[n][2] * inv1, o[n][3] * inv1);
    }
}

template <int DKT, int DVT>
int launch_tile(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_tables, int max_nb,
                const int32_t* cu_q, const int32_t* ctx_start, int n_seq, int T, int H, int G, int bs, float scale, int chunk,
                int window, int keep_first, float sink, float sink_logit, const float* sink_logits, const void* gate,
                int64_t gate_stride, void* out, cudaStream_t st) {
    constexpr int DK = 16 * DKT, DV = 16 * DVT;
    const size_t smem = (size_t)(kTQ * (DK + 8) + kTK * (DK + 8) + kTK * (DV + 8)) * sizeof(__nv_bfloat16);
    auto kern = chunk_attention_tile_kernel<DKT, DVT>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int tiles = (T + kTQ - 1) / kTQ + n_seq;          // upper bound on sum(ceil(len / 64)); spare CTAs leave at once
    kern<<<dim3(tiles, H), 128, smem, st>>>(static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
                                           static_cast<const __nv_bfloat16*>(v_cache), block_tables, max_nb, cu_q, ctx_start,
                                           n_seq, H, G, bs, scale * 1.4426950408889634f, chunk, window, keep_first, sink,
                                           sink_logit * 1.4426950408889634f, sink_logits,
                                           static_cast<const __nv_bfloat16*>(gate), gate_stride, static_cast<__nv_bfloat16*>(out));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

}  // namespace

extern "C" int b2_qknorm_cache(const void* qkv, int64_t qkv_stride, int act_dtype, int T, int H, int G, int dk, int dv,
                               const float* q_w, const float* k_w, float eps, const int64_t* slots, int bs, void* q_out,
                               void* k_cache, void* v_cache, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0, B2_EINVAL, "qknorm_cache: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(qkv && slots && q_out && k_cache && v_cache, B2_EINVAL, "qknorm_cache: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = H + 2 * G < 8 ? H + 2 * G : 8;
    B2_DISPATCH_ACT(act_dtype, A, (qknorm_cache_kernel<A><<<T, warps * 32, 0, st>>>(
        static_cast<const A*>(qkv), qkv_stride, H, G, dk, dv, q_w, k_w, eps, slots, bs, static_cast<A*>(q_out),
        static_cast<A*>(k_cache), static_cast<A*>(v_cache), true, nullptr, 0.f, 1)));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_qk_prep_cache(const void* qkv, int64_t qkv_stride, int act_dtype, int T, int H, int G, int dk, int dv,
                                int norm, const float* q_w, const float* k_w, float eps, const int32_t* positions,
                                float temp_coef, int temp_every, const int64_t* slots, int bs, void* q_out, void* k_cache,
                                void* v_cache, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0, B2_EINVAL, "qk_prep_cache: bad sizes");
    B2_REQUIRE(temp_coef == 0.f || (positions && temp_every >= 1), B2_EINVAL,
               "qk_prep_cache: a query temperature needs positions and a period of at least 1");
    if (T == 0) return B2_OK;
    B2_REQUIRE(qkv && slots && q_out && k_cache && v_cache, B2_EINVAL, "qk_prep_cache: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = H + 2 * G < 8 ? H + 2 * G : 8;
    B2_DISPATCH_ACT(act_dtype, A, (qknorm_cache_kernel<A><<<T, warps * 32, 0, st>>>(
        static_cast<const A*>(qkv), qkv_stride, H, G, dk, dv, q_w, k_w, eps, slots, bs, static_cast<A*>(q_out),
        static_cast<A*>(k_cache), static_cast<A*>(v_cache), norm != 0, positions, temp_coef, temp_every > 0 ? temp_every : 1)));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_qk_rope_cache(const void* qkv, int64_t qkv_stride, int act_dtype, int T, int H, int G, int dk, int dv,
                                int v_from_k, int rot_dims, int interleaved, const int32_t* positions, const float* cos_sin,
                                int max_pos, const int64_t* slots, int bs, void* q_out, void* k_cache, void* v_cache,
                                void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0, B2_EINVAL, "qk_rope_cache: bad sizes");
    B2_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= dk, B2_EINVAL,
               "qk_rope_cache: %d rotated entries in heads of %d", rot_dims, dk);
    B2_REQUIRE(!v_from_k || dv == dk, B2_EINVAL, "qk_rope_cache: values taken from the keys need dv == dk");
    B2_REQUIRE(rot_dims == 0 || max_pos > 0, B2_EINVAL, "qk_rope_cache: empty rotation table");
    if (T == 0) return B2_OK;
    B2_REQUIRE(qkv && slots && q_out && k_cache && v_cache && positions && (cos_sin || rot_dims == 0), B2_EINVAL,
               "qk_rope_cache: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t esz = act_dtype == B2_ACT_BF16 ? 2 : 4;
    auto al = [&](const void* p) { return reinterpret_cast<uintptr_t>(p) % (4 * esz) == 0; };
    const bool vec = dk % 4 == 0 && dv % 4 == 0 && qkv_stride % 4 == 0 && rot_dims % (interleaved ? 4 : 8) == 0 && al(qkv) && al(q_out) &&
                     al(k_cache) && al(v_cache);
    const int work = (H + G) * dk / (vec ? 4 : 1);
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec)
            qk_rope_cache_vec_kernel<A><<<T, threads, 0, st>>>(
                static_cast<const A*>(qkv), qkv_stride, H, G, dk, dv, v_from_k != 0, rot_dims, interleaved != 0, positions, cos_sin,
                max_pos > 0 ? max_pos : 1, slots, bs, static_cast<A*>(q_out), static_cast<A*>(k_cache), static_cast<A*>(v_cache));
        else
            qk_rope_cache_kernel<A><<<T, threads, 0, st>>>(
                static_cast<const A*>(qkv), qkv_stride, H, G, dk, dv, v_from_k != 0, rot_dims, interleaved != 0, positions, cos_sin,
                max_pos > 0 ? max_pos : 1, slots, bs, static_cast<A*>(q_out), static_cast<A*>(k_cache), static_cast<A*>(v_cache));
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_chunk_attention(void* out, const void* q, const void* k_cache, const void* v_cache, int act_dtype,
                                  const int32_t* block_tables, int max_nb, const int32_t* cu_q, const int32_t* ctx_start,
                                  int n_seq, int T, int H, int G, int dk, int dv, int bs, float scale, int chunk, float sink,
                                  float sink_logit, void* stream) {
    return b2_masked_attention(out, q, k_cache, v_cache, act_dtype, block_tables, max_nb, cu_q, ctx_start, n_seq, T, H, G, dk, dv,
                               bs, scale, chunk, 0, 0, sink, sink_logit, nullptr, nullptr, 0, stream);
}

extern "C" int b2_masked_attention(void* out, const void* q, const void* k_cache, const void* v_cache, int act_dtype,
                                   const int32_t* block_tables, int max_nb, const int32_t* cu_q, const int32_t* ctx_start,
                                   int n_seq, int T, int H, int G, int dk, int dv, int bs, float scale, int chunk, int window,
                                   int keep_first, float sink, float sink_logit, const float* sink_logits, const void* gate,
                                   int64_t gate_stride, void* stream) {
    B2_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && bs > 0 && chunk >= 0 && sink >= 0.f && window >= 0 &&
               keep_first >= 0, B2_EINVAL, "masked_attention: bad sizes");
    B2_REQUIRE(!gate || gate_stride >= H, B2_EINVAL, "masked_attention: gate rows shorter than the heads");
    B2_REQUIRE(dv <= 32 * kMaxDvPerLane, B2_EUNSUPPORTED, "chunk_attention: value size %d above %d", dv, 32 * kMaxDvPerLane);
    if (T == 0 || n_seq == 0) return B2_OK;
    B2_REQUIRE(out && q && k_cache && v_cache && block_tables && cu_q && ctx_start, B2_EINVAL, "chunk_attention: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int warps = 4;
    const size_t smem = (size_t)warps * dk * sizeof(float);
    B2_REQUIRE(smem <= 48 * 1024, B2_EUNSUPPORTED, "chunk_attention: key size %d too large", dk);
    const int items = T * H, blocks = (items + warps - 1) / warps;
    // prompt chunks of bf16 models with tensor-core friendly head sizes go to the tiled kernel (a sequence needs at least
    // kTileMinRows rows, so a batch of T rows over n_seq sequences can only hold one when T - n_seq >= kTileMinRows - 1)
    int skip_from = 0;
    if (act_dtype == B2_ACT_BF16 && T - n_seq >= kTileMinRows - 1 && dk % 32 == 0 && dv % 32 == 0 && dk <= 128 && dv <= 128 &&
        b2_aligned16(q) && b2_aligned16(k_cache) && b2_aligned16(v_cache) && b2_aligned16(out)) {
        skip_from = kTileMinRows;
        int rc = B2_OK;
#define B2_TILE(a, b)                                                                                                     \
    if (dk == 16 * a && dv == 16 * b)                                                                                     \
        rc = launch_tile<a, b>(q, k_cache, v_cache, block_tables, max_nb, cu_q, ctx_start, n_seq, T, H, G, bs, scale, chunk, \
                               window, keep_first, sink, sink_logit, sink_logits, gate, gate_stride, out, st);
        B2_TILE(2, 2) B2_TILE(2, 4) B2_TILE(2, 6) B2_TILE(2, 8) B2_TILE(4, 2) B2_TILE(4, 4) B2_TILE(4, 6) B2_TILE(4, 8)
        B2_TILE(6, 2) B2_TILE(6, 4) B2_TILE(6, 6) B2_TILE(6, 8) B2_TILE(8, 2) B2_TILE(8, 4) B2_TILE(8, 6) B2_TILE(8, 8)
#undef B2_TILE
        if (rc != B2_OK) return rc;
    }
    if (act_dtype == B2_ACT_BF16 && dk % 8 == 0 && dv % 8 == 0 && dv <= 64 * kGroupMaxPairs && b2_aligned16(q) &&
        b2_aligned16(k_cache) && b2_aligned16(v_cache) && b2_aligned16(out)) {
        const size_t gsm = (size_t)(kGroupMaxHeads * dk + 4 * kGroupMaxHeads * (2 + dv)) * sizeof(float) +
                           (size_t)4 * 32 * (dk + 8 + dv) * sizeof(__nv_bfloat16);
        if (gsm <= 160 * 1024) {
            auto kern = chunk_attention_group_kernel;
            if (gsm > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gsm));
            kern<<<dim3(T, G), 128, gsm, st>>>(static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
                                               static_cast<const __nv_bfloat16*>(v_cache), block_tables, max_nb, cu_q, ctx_start,
                                               n_seq, H, G, dk, dv, bs, scale, chunk, window, keep_first, sink, sink_logit,
                                               sink_logits, static_cast<const __nv_bfloat16*>(gate), gate_stride, skip_from,
                                               static_cast<__nv_bfloat16*>(out));
            B2_CUDA_OK(cudaGetLastError());
            return B2_OK;
        }
    }
    B2_DISPATCH_ACT(act_dtype, A, (chunk_attention_kernel<A><<<blocks, warps * 32, smem, st>>>(
        static_cast<const A*>(q), static_cast<const A*>(k_cache), static_cast<const A*>(v_cache), block_tables, max_nb, cu_q,
        ctx_start, n_seq, T, H, G, dk, dv, bs, scale, chunk, window, keep_first, sink, sink_logit, sink_logits,
        static_cast<const A*>(gate), gate_stride, skip_from, static_cast<A*>(out))));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
