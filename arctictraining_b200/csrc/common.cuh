// SPDX-License-Identifier: Apache-2.0
// Shared device/host helpers for the sm_100a kernels of this library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "device_utils.cuh"

#define ATB_CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define ATB_CHECK_CONTIG(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define ATB_CHECK_DTYPE(x, dt) TORCH_CHECK((x).scalar_type() == (dt), #x " has the wrong dtype")
#define ATB_CHECK_ALIGNED16(x) \
    TORCH_CHECK((reinterpret_cast<uintptr_t>((x).data_ptr()) & 15) == 0, #x " must be 16-byte aligned")
#define ATB_LAUNCH_CHECK() C10_CUDA_KERNEL_LAUNCH_CHECK()

namespace atb {

inline cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace atb
