// SPDX-License-Identifier: Apache-2.0
// RMSNorm backward kernel, shared by the tensor-based operator and the allocation-free C entry point.
#pragma once

#include "device_utils.cuh"

namespace atb {

// RMSNorm backward.  Each CTA walks rows blockIdx.x, +gridDim.x, ... and keeps the weight-gradient
// partial of the columns its threads own in registers; partials go to dw_partial[gridDim.x, H].
template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                          const bf16* __restrict__ w, const float* __restrict__ rstd,
                                                          bf16* __restrict__ dx, float* __restrict__ dw_partial,
                                                          int64_t T, int H) {
    __shared__ float scratch[32];
    const int nvec = H >> 3;
    float wreg[VPT][8];
    float dwacc[VPT][8];
    const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * 256;
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[v][j] = 0.f;
        if (i < nvec) unpack8(wr[i], wreg[v]);
    }
    // the raw vectors of the next row are requested before the current row's block-wide reduction, so that memory
    // latency overlaps the barriers
    bf16x8 xc[VPT], gc[VPT], xn[VPT], gn[VPT];
    if ((int64_t)blockIdx.x < T) {
        const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (int64_t)blockIdx.x * H);
        const bf16x8* gr = reinterpret_cast<const bf16x8*>(dy + (int64_t)blockIdx.x * H);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 256;
            if (i < nvec) { xc[v] = xr[i]; gc[v] = gr[i]; }
        }
    }
    for (int64_t row = blockIdx.x; row < T; row += gridDim.x) {
        const int64_t next = row + gridDim.x;
        if (next < T) {
            const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + next * H);
            const bf16x8* gr = reinterpret_cast<const bf16x8*>(dy + next * H);
#pragma unroll
            for (int v = 0; v < VPT; ++v) {
                const int i = threadIdx.x + v * 256;
                if (i < nvec) { xn[v] = xr[i]; gn[v] = gr[i]; }
            }
        }
        bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + row * H);
        const float r = rstd[row];
        float xf[VPT][8], gf[VPT][8];
        float dot = 0.f;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 256;
            if (i < nvec) {
                unpack8(xc[v], xf[v]);
                unpack8(gc[v], gf[v]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    dwacc[v][j] += gf[v][j] * xf[v][j] * r;
                    gf[v][j] *= wreg[v][j];
                    dot += gf[v][j] * xf[v][j];
                }
            }
        }
        dot = block_sum(dot, scratch);
        const float c = dot * r * r / (float)H;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * 256;
            if (i < nvec) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = r * (gf[v][j] - xf[v][j] * c);
                dxr[i] = pack8(o);
            }
        }
#pragma unroll
        for (int v = 0; v < VPT; ++v) { xc[v] = xn[v]; gc[v] = gn[v]; }
    }
    float* out = dw_partial + (int64_t)blockIdx.x * H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * 256;
        if (i < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) out[i * 8 + j] = dwacc[v][j];
        }
    }
}

}  // namespace atb
