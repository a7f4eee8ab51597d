// SPDX-License-Identifier: Apache-2.0
// Allocation-free RMSNorm backward: see rmsnorm_bwd_noalloc.h for the contract.
//
// The partial sums of the weight gradient go to a file-scope device array instead of a freshly allocated tensor.
// In host code the name of that array is only a handle for the runtime, not an address a kernel can use, so the
// device address is queried once per device with cudaGetSymbolAddress and passed to the kernels as a pointer.

#include "rmsnorm_bwd_noalloc.h"

#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "rmsnorm_kernels.cuh"

namespace {

constexpr int kMaxDevices = 64;

// 148 blocks x 8192 columns of fp32 partial sums; held by every GPU that loads this library.
static __device__ __align__(256) float g_dw_partials[ATB_NOALLOC_MAX_BLOCKS * ATB_NOALLOC_MAX_HIDDEN];

float* g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Sum the per-block partials in block order (deterministic) into dw.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partials, int nblk, int H,
                                                              float* __restrict__ dw) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= H) return;
    float acc = 0.f;
    for (int b = 0; b < nblk; ++b) acc += partials[(long long)b * H + col];
    dw[col] = acc;
}

int fail(int code, char* err, unsigned long err_len, const char* msg) {
    if (err != nullptr && err_len > 0) {
        strncpy(err, msg, err_len - 1);
        err[err_len - 1] = '\0';
    }
    return code;
}

int fail_cuda(cudaError_t e, const char* what, char* err, unsigned long err_len) {
    char buf[256];
    snprintf(buf, sizeof(buf), "%s: %s", what, cudaGetErrorString(e));
    return fail(2, err, err_len, buf);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// A pointer the kernels may dereference on device `dev`: device (or managed) memory that belongs to that device.
// Queries the driver's address map; allocates nothing.
bool on_device(const void* p, int dev) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (a.type == cudaMemoryTypeManaged) return true;
    return a.type == cudaMemoryTypeDevice && a.device == dev;
}

}  // namespace

extern "C" int atb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                                       long long rows, int hidden, void* cuda_stream, char* err, unsigned long err_len) {
    if (!dy || !x || !w || !rstd || !dx || !dw) return fail(1, err, err_len, "rmsnorm_bwd_noalloc: null pointer argument");
    if (rows <= 0) return fail(1, err, err_len, "rmsnorm_bwd_noalloc: rows must be positive");
    if (hidden <= 0 || hidden % 8 != 0)
        return fail(1, err, err_len, "rmsnorm_bwd_noalloc: hidden must be a positive multiple of 8");
    if (hidden > ATB_NOALLOC_MAX_HIDDEN) {
        char buf[160];
        snprintf(buf, sizeof(buf), "rmsnorm_bwd_noalloc: hidden=%d exceeds the built-in scratch limit of %d columns", hidden,
                 ATB_NOALLOC_MAX_HIDDEN);
        return fail(1, err, err_len, buf);
    }
    if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx))
        return fail(1, err, err_len, "rmsnorm_bwd_noalloc: dy, x, w and dx must be 16-byte aligned");

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice", err, err_len);
    if (dev < 0 || dev >= kMaxDevices) return fail(1, err, err_len, "rmsnorm_bwd_noalloc: device index out of range");
    // the scratch array that is used is the current device's: operands that live elsewhere (another GPU, host memory)
    // would fault in the kernel or, where the GPU can reach them, silently mix devices
    const void* ptrs[6] = {dy, x, w, rstd, dx, dw};
    for (const void* p : ptrs)
        if (!on_device(p, dev))
            return fail(1, err, err_len, "rmsnorm_bwd_noalloc: every operand must be device memory of the current device");
    float* partials = nullptr;
    {
        // set-up, once per device, with that device current: resolve the device address of the scratch array
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (g_partials_addr[dev] == nullptr) {
            float* addr = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_dw_partials);
            if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(scratch)", err, err_len);
            g_partials_addr[dev] = addr;
        }
        partials = g_partials_addr[dev];
    }

    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const int nblk = (int)(rows < ATB_NOALLOC_MAX_BLOCKS ? rows : ATB_NOALLOC_MAX_BLOCKS);
    const int nvec = hidden / 8;
    const int vpt = (nvec + 255) / 256;
    const atb::bf16* dyp = static_cast<const atb::bf16*>(dy);
    const atb::bf16* xp = static_cast<const atb::bf16*>(x);
    const atb::bf16* wp = static_cast<const atb::bf16*>(w);
    atb::bf16* dxp = static_cast<atb::bf16*>(dx);
    if (vpt <= 1) atb::rmsnorm_bwd_kernel<1><<<nblk, 256, 0, stream>>>(dyp, xp, wp, rstd, dxp, partials, rows, hidden);
    else if (vpt <= 2) atb::rmsnorm_bwd_kernel<2><<<nblk, 256, 0, stream>>>(dyp, xp, wp, rstd, dxp, partials, rows, hidden);
    else atb::rmsnorm_bwd_kernel<4><<<nblk, 256, 0, stream>>>(dyp, xp, wp, rstd, dxp, partials, rows, hidden);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "launch of rmsnorm_bwd_kernel", err, err_len);
    reduce_partials_kernel<<<(hidden + 255) / 256, 256, 0, stream>>>(partials, nblk, hidden, dw);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "launch of reduce_partials_kernel", err, err_len);
    return 0;
}
