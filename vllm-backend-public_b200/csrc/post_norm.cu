// post_norm.cu -- the residual path of a decoder that normalises every sublayer on both sides ("sandwich" norms), and
// the element-wise pieces of its feed-forwards and output:
//
//   b2_sandwich_norm   one pass over the fp32 residual rows x [T, D]:
//                      (1) when y is given: the sublayer output is normalised and added, x' = x + norm(y; post_w, post_b)
//                          (post_w NULL: plain x' = x + y);
//                      (2) when h is given: the next sublayer's input is normalised out, h = norm(x'; pre_w, pre_b).
//                      norm = layer norm (B2_NORM_LAYER, bias optional) or RMS norm (B2_NORM_RMS), eps inside the root.
//                      The write-back and the next read-out touch the same row, so the op moves D*4 in, D*4 out for the
//                      residual plus one activation row each way.  With post_w = NULL it is residual add + pre-norm.
//   b2_row_norm        out[t, :] = in[t, :] / sqrt(mean(in[t, :]^2) + eps) * w over activation rows of any width (row strides
//                      of their own: a column range of a wider projection is fine); the statistics in fp32.  The norm of a
//                      low-rank latent between its two projections.
//   b2_relu_sq         out = max(in, 0)^2
//   b2_glu_and_mul     out[t, i] = glu(in[t, i], in[t, I + i]) for rows [gate | up]: SiLU(g) * u (B2_GLU_SILU) or the bounded
//                      unit g' * sigmoid(alpha g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit) (B2_GLU_CLAMPED)
//                      or gelu_tanh(g) * u, gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) (B2_GLU_GELU_TANH)
//   b2_gate_mul        out[t, i] = x[t, i] * act(gate[t, i]) * scale with act = sigmoid (B2_GATE_SIGMOID) or SiLU
//                      (B2_GATE_SILU): an output gate on concatenated head outputs, the three rows with strides of their own
//   b2_softcap         z <- cap * tanh(z / cap) in place
// The residual and all statistics are fp32 whatever the activation type.
#include "b2_act.cuh"

namespace {

// W = 4: every access is a 16-byte (fp32) or 8-byte (bf16) vector; W = 1: any width and alignment.  A thread keeps to its
// own columns in every pass, so the row in shared memory needs no barrier beyond those of the reductions.
template <typename T, int W>
__global__ void __launch_bounds__(512)
sandwich_norm_kernel(float* __restrict__ x, int D, const T* __restrict__ y, int64_t y_stride, const float* __restrict__ post_w,
                     const float* __restrict__ post_b, const float* __restrict__ pre_w, const float* __restrict__ pre_b, float eps,
                     int norm_kind, T* __restrict__ h, int64_t h_stride) {
    extern __shared__ __align__(16) float row_sm[];  // [D]
    __shared__ float red[33];
    const int t = blockIdx.x;
    float* xt = x + (size_t)t * D;
    const int step = blockDim.x * W;
    float sum = 0.f;
    if (y) {
        const T* yt = y + (size_t)t * y_stride;
        for (int d = threadIdx.x * W; d < D; d += step) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(yt + d, v); else v[0] = b2::ld(yt + d);
#pragma unroll
            for (int c = 0; c < W; ++c) {
                row_sm[d + c] = v[c];
                sum += v[c];
            }
        }
        float mean = 0.f, inv = 1.f;
        if (post_w) {
            if (norm_kind == B2_NORM_LAYER) mean = b2::block_sum(sum, red) / (float)D;
            float sq = 0.f;
            for (int d = threadIdx.x * W; d < D; d += step) {
#pragma unroll
                for (int c = 0; c < W; ++c) {
                    const float e = row_sm[d + c] - mean;
                    sq = fmaf(e, e, sq);
                }
            }
            inv = rsqrtf(b2::block_sum(sq, red) / (float)D + eps);
        }
        sum = 0.f;
        for (int d = threadIdx.x * W; d < D; d += step) {
            float r[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(xt + d, r); else r[0] = xt[d];
#pragma unroll
            for (int c = 0; c < W; ++c) {
                float v = row_sm[d + c];
                if (post_w) v = (v - mean) * inv * post_w[d + c] + (post_b ? post_b[d + c] : 0.f);
                r[c] += v;
                row_sm[d + c] = r[c];
                sum += r[c];
            }
            if (W == 4) b2::st4(xt + d, r); else xt[d] = r[0];
        }
    } else {
        for (int d = threadIdx.x * W; d < D; d += step) {
            float r[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(xt + d, r); else r[0] = xt[d];
#pragma unroll
            for (int c = 0; c < W; ++c) {
                row_sm[d + c] = r[c];
                sum += r[c];
            }
        }
    }
    if (!h) return;
    float mean = 0.f;
    if (norm_kind == B2_NORM_LAYER) mean = b2::block_sum(sum, red) / (float)D;
    float sq = 0.f;
    for (int d = threadIdx.x * W; d < D; d += step) {
#pragma unroll
        for (int c = 0; c < W; ++c) {
            const float e = row_sm[d + c] - mean;
            sq = fmaf(e, e, sq);
        }
    }
    const float inv = rsqrtf(b2::block_sum(sq, red) / (float)D + eps);
    T* ho = h + (size_t)t * h_stride;
    for (int d = threadIdx.x * W; d < D; d += step) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < W; ++c) v[c] = (row_sm[d + c] - mean) * inv * pre_w[d + c] + (pre_b ? pre_b[d + c] : 0.f);
        if (W == 4) b2::st4(ho + d, v); else b2::st(ho + d, v[0]);
    }
}

// W = 4: 16-byte (fp32) or 8-byte (bf16) accesses, the row kept in registers between the two passes when it fits (up to
// kRowNormKeep accesses a thread); W = 1: any width and alignment.
constexpr int kRowNormKeep = 4;

template <typename T, int W>
__global__ void __launch_bounds__(256)
row_norm_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ in, int64_t in_stride, int n,
                const float* __restrict__ w, float eps) {
    __shared__ float red[33];
    const T* src = in + (size_t)blockIdx.x * in_stride;
    T* dst = out + (size_t)blockIdx.x * out_stride;
    const int step = blockDim.x * W;
    const bool keep = n <= kRowNormKeep * step;
    float held[kRowNormKeep][4];
    float ss = 0.f;
    if (keep) {
#pragma unroll
        for (int r = 0; r < kRowNormKeep; ++r) {
            const int i = threadIdx.x * W + r * step;
            held[r][0] = held[r][1] = held[r][2] = held[r][3] = 0.f;
            if (i < n) {
                if (W == 4) b2::ld4(src + i, held[r]); else held[r][0] = b2::ld(src + i);
            }
#pragma unroll
            for (int c = 0; c < W; ++c) ss = fmaf(held[r][c], held[r][c], ss);
        }
    } else {
        for (int i = threadIdx.x * W; i < n; i += step) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(src + i, v); else v[0] = b2::ld(src + i);
#pragma unroll
            for (int c = 0; c < W; ++c) ss = fmaf(v[c], v[c], ss);
        }
    }
    const float inv = rsqrtf(b2::block_sum(ss, red) / (float)n + eps);
    if (keep) {
#pragma unroll
        for (int r = 0; r < kRowNormKeep; ++r) {
            const int i = threadIdx.x * W + r * step;
            if (i < n) {
#pragma unroll
                for (int c = 0; c < W; ++c) held[r][c] *= inv * (w ? w[i + c] : 1.f);
                if (W == 4) b2::st4(dst + i, held[r]); else b2::st(dst + i, held[r][0]);
            }
        }
    } else {
        for (int i = threadIdx.x * W; i < n; i += step) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (W == 4) b2::ld4(src + i, v); else v[0] = b2::ld(src + i);
#pragma unroll
            for (int c = 0; c < W; ++c) v[c] *= inv * (w ? w[i + c] : 1.f);
            if (W == 4) b2::st4(dst + i, v); else b2::st(dst + i, v[0]);
        }
    }
}

template <typename T, int W>
__global__ void relu_sq_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ in, int64_t in_stride, int I) {
    const int t = blockIdx.x;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * W; i < I; i += gridDim.y * blockDim.x * W) {
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (W == 4) b2::ld4(in + (size_t)t * in_stride + i, v); else v[0] = b2::ld(in + (size_t)t * in_stride + i);
#pragma unroll
        for (int c = 0; c < W; ++c) {
            v[c] = fmaxf(v[c], 0.f);
            v[c] *= v[c];
        }
        if (W == 4) b2::st4(out + (size_t)t * out_stride + i, v); else b2::st(out + (size_t)t * out_stride + i, v[0]);
    }
}

template <typename T, int W>
__global__ void glu_and_mul_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ in, int64_t in_stride, int I,
                                   int glu, float alpha, float limit) {
    const int t = blockIdx.x;
    const T* r = in + (size_t)t * in_stride;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * W; i < I; i += gridDim.y * blockDim.x * W) {
        float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
        if (W == 4) {
            b2::ld4(r + i, g);
            b2::ld4(r + I + i, u);
        } else {
            g[0] = b2::ld(r + i);
            u[0] = b2::ld(r + I + i);
        }
#pragma unroll
        for (int c = 0; c < W; ++c) {
            if (glu == B2_GLU_CLAMPED) v[c] = b2::glu_clamped_f(g[c], u[c], alpha, limit);
            else if (glu == B2_GLU_GELU_TANH) v[c] = b2::gelu_tanh_f(g[c]) * u[c];
            else v[c] = b2::silu_f(g[c]) * u[c];
        }
        if (W == 4) b2::st4(out + (size_t)t * out_stride + i, v); else b2::st(out + (size_t)t * out_stride + i, v[0]);
    }
}

template <typename T, int W>
__global__ void gate_mul_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x, int64_t x_stride,
                                const T* __restrict__ gate, int64_t gate_stride, int I, int kind, float scale) {
    const int t = blockIdx.x;
    for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * W; i < I; i += gridDim.y * blockDim.x * W) {
        float z[4] = {0.f, 0.f, 0.f, 0.f}, a[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
        if (W == 4) {
            b2::ld4(gate + (size_t)t * gate_stride + i, z);
            b2::ld4(x + (size_t)t * x_stride + i, a);
        } else {
            z[0] = b2::ld(gate + (size_t)t * gate_stride + i);
            a[0] = b2::ld(x + (size_t)t * x_stride + i);
        }
#pragma unroll
        for (int c = 0; c < W; ++c) v[c] = a[c] * (kind == B2_GATE_SIGMOID ? b2::sigmoid_f(z[c]) : b2::silu_f(z[c])) * scale;
        if (W == 4) b2::st4(out + (size_t)t * out_stride + i, v); else b2::st(out + (size_t)t * out_stride + i, v[0]);
    }
}

template <typename T>
__global__ void softcap_kernel(T* __restrict__ z, int64_t stride, int V, float cap) {
    const int t = blockIdx.x;
    const float inv = 1.f / cap;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < V; i += gridDim.y * blockDim.x) {
        T* p = z + (size_t)t * stride + i;
        b2::st(p, cap * tanhf(b2::ld(p) * inv));
    }
}

inline dim3 rows_grid(int cols, int rows) {
    int gx = (cols + 255) / 256;
    if (gx > 64) gx = 64;
    return dim3(rows, gx);
}

}  // namespace

extern "C" int b2_sandwich_norm(float* x, int T, int D, const void* y, int64_t y_stride, const float* post_w,
                                const float* post_b, const float* pre_w, const float* pre_b, float eps, int norm_kind, void* h,
                                int64_t h_stride, int act_dtype, void* stream) {
    B2_REQUIRE(T >= 0 && D > 0, B2_EINVAL, "sandwich_norm: bad sizes T=%d D=%d", T, D);
    if (T == 0 || (!y && !h)) return B2_OK;
    B2_REQUIRE(x, B2_EINVAL, "sandwich_norm: null residual");
    B2_REQUIRE(!h || pre_w, B2_EINVAL, "sandwich_norm: a read-out needs its norm weight");
    B2_REQUIRE(norm_kind == B2_NORM_LAYER || norm_kind == B2_NORM_RMS, B2_EINVAL, "sandwich_norm: unknown norm kind %d", norm_kind);
    const size_t smem = (size_t)D * sizeof(float);
    B2_REQUIRE(smem <= 200 * 1024, B2_EUNSUPPORTED, "sandwich_norm: width %d does not fit shared memory", D);
    B2_REQUIRE(b2_aligned16(x), B2_EINVAL, "sandwich_norm: the residual must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int threads = D >= 8192 ? 512 : (D >= 1024 ? 256 : 128);
    const bool vec = D % 4 == 0 && (!y || (y_stride % 4 == 0 && b2_aligned16(y))) && (!h || (h_stride % 4 == 0 && b2_aligned16(h)));
#define B2_SANDWICH(W)                                                                                                      \
    do {                                                                                                                    \
        auto kern = sandwich_norm_kernel<A, W>;                                                                             \
        if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<T, threads, smem, st>>>(x, D, static_cast<const A*>(y), y_stride, post_w, post_b, pre_w, pre_b, eps, norm_kind, \
                                       static_cast<A*>(h), h_stride);                                                       \
    } while (0)
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec) B2_SANDWICH(4);
        else B2_SANDWICH(1);
    });
#undef B2_SANDWICH
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_row_norm(void* out, int64_t out_stride, const void* in, int64_t in_stride, int act_dtype, int T, int n,
                           const float* w, float eps, void* stream) {
    B2_REQUIRE(T >= 0 && n > 0 && out_stride >= n && in_stride >= n, B2_EINVAL, "row_norm: bad sizes");
    if (T == 0) return B2_OK;
    B2_REQUIRE(out && in, B2_EINVAL, "row_norm: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t esz = act_dtype == B2_ACT_BF16 ? 2 : 4;
    const bool vec = n % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && reinterpret_cast<uintptr_t>(in) % (4 * esz) == 0 &&
                     reinterpret_cast<uintptr_t>(out) % (4 * esz) == 0;
    const int per = vec ? 4 : 1;
    const int threads = n >= 1024 * per ? 256 : (n >= 256 * per ? 128 : 64);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec)
            row_norm_kernel<A, 4><<<T, threads, 0, st>>>(static_cast<A*>(out), out_stride, static_cast<const A*>(in), in_stride, n, w, eps);
        else
            row_norm_kernel<A, 1><<<T, threads, 0, st>>>(static_cast<A*>(out), out_stride, static_cast<const A*>(in), in_stride, n, w, eps);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_relu_sq(void* out, int64_t out_stride, const void* in, int64_t in_stride, int act_dtype, int T, int I,
                          void* stream) {
    B2_REQUIRE(T >= 0 && I > 0, B2_EINVAL, "relu_sq: bad sizes T=%d I=%d", T, I);
    if (T == 0) return B2_OK;
    B2_REQUIRE(out && in, B2_EINVAL, "relu_sq: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = I % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && b2_aligned16(in) && b2_aligned16(out);
    B2_DISPATCH_ACT(act_dtype, A, {
        A* o = static_cast<A*>(out);
        const A* i = static_cast<const A*>(in);
        if (vec) relu_sq_kernel<A, 4><<<rows_grid(I / 4, T), 256, 0, st>>>(o, out_stride, i, in_stride, I);
        else relu_sq_kernel<A, 1><<<rows_grid(I, T), 256, 0, st>>>(o, out_stride, i, in_stride, I);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_glu_and_mul(void* out, int64_t out_stride, const void* gate_up, int64_t in_stride, int act_dtype, int T, int I,
                              int glu, float alpha, float limit, void* stream) {
    B2_REQUIRE(T >= 0 && I > 0, B2_EINVAL, "glu_and_mul: bad sizes T=%d I=%d", T, I);
    B2_REQUIRE(glu == B2_GLU_SILU || glu == B2_GLU_CLAMPED || glu == B2_GLU_GELU_TANH, B2_EINVAL,
               "glu_and_mul: unknown gated activation %d", glu);
    if (T == 0) return B2_OK;
    B2_REQUIRE(out && gate_up, B2_EINVAL, "glu_and_mul: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = I % 4 == 0 && in_stride % 4 == 0 && out_stride % 4 == 0 && b2_aligned16(gate_up) && b2_aligned16(out);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec) glu_and_mul_kernel<A, 4><<<rows_grid(I / 4, T), 256, 0, st>>>(static_cast<A*>(out), out_stride,
                                                                              static_cast<const A*>(gate_up), in_stride, I, glu,
                                                                              alpha, limit);
        else glu_and_mul_kernel<A, 1><<<rows_grid(I, T), 256, 0, st>>>(static_cast<A*>(out), out_stride,
                                                                      static_cast<const A*>(gate_up), in_stride, I, glu, alpha, limit);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_gate_mul(void* out, int64_t out_stride, const void* x, int64_t x_stride, const void* gate, int64_t gate_stride,
                           int act_dtype, int T, int I, int kind, float scale, void* stream) {
    B2_REQUIRE(T >= 0 && I > 0, B2_EINVAL, "gate_mul: bad sizes T=%d I=%d", T, I);
    B2_REQUIRE(kind == B2_GATE_SILU || kind == B2_GATE_SIGMOID, B2_EINVAL, "gate_mul: unknown gate %d", kind);
    if (T == 0) return B2_OK;
    B2_REQUIRE(out && x && gate, B2_EINVAL, "gate_mul: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = I % 4 == 0 && x_stride % 4 == 0 && gate_stride % 4 == 0 && out_stride % 4 == 0 && b2_aligned16(x) &&
                     b2_aligned16(gate) && b2_aligned16(out);
    B2_DISPATCH_ACT(act_dtype, A, {
        if (vec) gate_mul_kernel<A, 4><<<rows_grid(I / 4, T), 256, 0, st>>>(static_cast<A*>(out), out_stride, static_cast<const A*>(x),
                                                                           x_stride, static_cast<const A*>(gate), gate_stride, I,
                                                                           kind, scale);
        else gate_mul_kernel<A, 1><<<rows_grid(I, T), 256, 0, st>>>(static_cast<A*>(out), out_stride, static_cast<const A*>(x),
                                                                   x_stride, static_cast<const A*>(gate), gate_stride, I, kind, scale);
    });
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}

extern "C" int b2_softcap(void* z, int64_t stride, int act_dtype, int T, int V, float cap, void* stream) {
    B2_REQUIRE(T >= 0 && V > 0 && cap > 0.f, B2_EINVAL, "softcap: bad sizes T=%d V=%d cap=%g", T, V, cap);
    if (T == 0) return B2_OK;
    B2_REQUIRE(z, B2_EINVAL, "softcap: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    B2_DISPATCH_ACT(act_dtype, A, (softcap_kernel<A><<<rows_grid(V, T), 256, 0, st>>>(static_cast<A*>(z), stride, V, cap)));
    B2_CUDA_OK(cudaGetLastError());
    return B2_OK;
}
