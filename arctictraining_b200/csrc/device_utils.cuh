// SPDX-License-Identifier: Apache-2.0
// Device-side helpers shared by the kernels of this library: 16-byte bf16 vectors and warp / block reductions.
// This header depends on the CUDA toolkit only (no framework headers).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace atb {

using bf16 = __nv_bfloat16;
using bf162 = __nv_bfloat162;

constexpr int kNumSMs = 148;

struct alignas(16) bf16x8 {
    bf162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& in, float (&out)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(in.v[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

__device__ __forceinline__ bf16x8 pack8(const float (&in)[8]) {
    bf16x8 out;
#pragma unroll
    for (int i = 0; i < 4; ++i) out.v[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    return out;
}

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

// Block-wide sum; every thread gets the result.  `scratch` holds at least 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

}  // namespace atb
