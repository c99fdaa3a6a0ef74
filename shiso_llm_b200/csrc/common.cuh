// Shared by every kernel file: element types, conversions, reductions, launch checks.
//
// Activations and weights are float (the true 32-bit path) or __nv_bfloat16.
// Sums, norm statistics, softmax, rotation angles and the residual stream are
// always float.  No file is built with --use_fast_math: expf, sinf, cosf and
// rsqrtf below are the accurate library entries, as the reference keeps them for
// its attention and rotation kernels (kernels/cuda/dense/KERNEL.toml:20-36).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SHISO_API extern "C" __attribute__((visibility("default")))

// Element type codes passed across the C boundary.
enum { SHISO_F32 = 0, SHISO_BF16 = 1 };

// Error codes returned by launchers in addition to cudaError_t values (which are < 1000).
enum {
    SHISO_OK = 0,
    SHISO_ERR_DTYPE = 1001,
    SHISO_ERR_SHAPE = 1002,
    SHISO_ERR_ALIGN = 1003,
    SHISO_ERR_UNSUPPORTED = 1004,
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
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

// Sum over a block of up to 1024 threads; every thread gets the result.  The order
// of additions depends only on blockDim, so a row's statistic does not depend on
// what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < nwarps) ? scratch[lane] : 0.0f;
    total = warp_sum(total);
    return total;
}

static inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

static inline unsigned ceil_div_u(long long a, long long b) { return (unsigned)((a + b - 1) / b); }
