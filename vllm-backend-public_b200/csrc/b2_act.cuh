// b2_act.cuh -- element access for kernels that are instantiated for two activation types:
// __nv_bfloat16 (serving) and float (the all-32-bit mode).  Math is always fp32; only loads and stores differ.
#pragma once
#include "b2_common.cuh"

#ifdef __CUDACC__
namespace b2 {

__device__ __forceinline__ float ld(const float* p) { return *p; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st(float* p, float v) { *p = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over the block; `red` is 33 floats of shared memory.  Every thread gets the result.  May be called repeatedly.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                      // protects `red` against the previous call's readers
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
// gated unit with both inputs bounded: g' = min(g, limit), u' = clamp(u, -limit, limit); g' * sigmoid(alpha g') * (u' + 1)
__device__ __forceinline__ float glu_clamped_f(float g, float u, float alpha, float limit) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoid_f(alpha * g) * (u + 1.f);
}
// tanh form of GELU: z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float relu_sq_f(float z) {
    z = fmaxf(z, 0.f);
    return z * z;
}
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// four consecutive elements of an activation row (8 or 16 bytes, aligned)
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]));
}

// Sequence of batch row `row` when rows are grouped by cu[0..n] (cu[0] = 0, cu[n] = rows in the batch).
__device__ __forceinline__ int seq_of_row(const int32_t* cu, int n, int row) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (cu[mid] <= row) lo = mid; else hi = mid - 1;
    }
    return lo;
}

}  // namespace b2
#endif

// activation type selector of the C ABI
#define B2_DISPATCH_ACT(act_dtype, T, ...)                                  \
    do {                                                                    \
        if ((act_dtype) == B2_ACT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else { using T = float; __VA_ARGS__; }                              \
    } while (0)
