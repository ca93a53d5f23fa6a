// Small device helpers shared by the kernels: typed 8-element vector access, warp sums,
// activation math.
#pragma once
#include "common.h"
#include <math_constants.h>

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }
// Value as the activation type would store it (a BF16 round trip, or the identity).
template <class T> __device__ __forceinline__ float rounded(float v) { return to_float(from_float<T>(v)); }

// 8 consecutive elements; the pointer must be 16-byte aligned (BF16) / 32-byte aligned (FP32).
__device__ __forceinline__ void load8(const bf16 *p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4 *>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&h);
}
__device__ __forceinline__ void store8(bf16 *p, const float (&v)[8]) {
    uint4 u;
    u.x = pack_bf16(v[0], v[1]);
    u.y = pack_bf16(v[2], v[3]);
    u.z = pack_bf16(v[4], v[5]);
    u.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4 *>(p) = u;
}
__device__ __forceinline__ void store8(float *p, const float (&v)[8]) {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int k = 16; k; k >>= 1)
        x += __shfl_xor_sync(0xffffffffu, x, k);
    return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int k = 16; k; k >>= 1)
        x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, k));
    return x;
}
// Sum over the block, same value returned to every thread; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float x, float *scratch) {
    x = warp_sum(x);
    __syncthreads();
    if (threadIdx.x % 32 == 0)
        scratch[threadIdx.x / 32] = x;
    __syncthreads();
    float total = 0;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w)
        total += scratch[w];
    return total;
}

__device__ __forceinline__ float sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
// Exact (erf) GELU and its derivative (reference cuda/attention.cuh:60-66 uses the same forms).
__device__ __forceinline__ float gelu(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865475f)); }
__device__ __forceinline__ float gelu_derivative(float x) {
    return 0.5f * (1.f + erff(x * 0.7071067811865475f)) + x * 0.3989422804014327f * expf(-0.5f * x * x);
}

// Exact FP32 master weight from its two 16-bit halves (reference cuda/ops.cuh:6-14).
__device__ __forceinline__ float join_weight(bf16 high, uint16_t low) {
    return __uint_as_float((unsigned(__bfloat16_as_ushort(high)) << 16) | low);
}
