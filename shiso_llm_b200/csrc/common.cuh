// Shared by every kernel file: element types, conversions, reductions, launch checks.
//
// Activations and weights are float (the true 32-bit path) or __nv_bfloat16.
// Sums, norm statistics, softmax, rotation angles and the residual stream are
// always float.  No file is built with --use_fast_math: expf, sinf, cosf and
// rsqrtf below are the accurate library entries, as the reference keeps them for
// its attention and rotation kernels (kernels/cuda/dense/KERNEL.toml:20-36).  The exceptions
// say so where they stand: exponentials of the tensor-memory prompt attention, and silu_times.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

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

// silu(g) * u in the epilogue of a bfloat16 gate/up product, with the exponential and the
// reciprocal from the special-function unit (relative error about 2^-22, far below the bfloat16
// the result is rounded to).  The library's expf and an IEEE division took 8.7 us for the last
// 128 x 128 tile of a CTA of the prompt kernels: one warp to a scheduler, and nothing to hide
// their latency behind.  (The float32 path keeps expf and the division.)
__device__ __forceinline__ float silu_times(float g, float u) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(g * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r * u;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel is launched so that it may start while its predecessor in the stream is still
// finishing.  It waits for the predecessor to complete and flush (griddepcontrol.wait) before
// it touches anything a predecessor may have written; work that depends on no predecessor -
// address arithmetic, loads of weights - goes before the wait.  It says when its own successor
// may be scheduled (griddepcontrol.launch_dependents): small row kernels say so at once
// (pdl_begin), kernels that fill the SMs only after their main loop (pdl_trigger), because a
// successor that is resident early only spins in its wait and takes registers and shared
// memory from the CTAs that still have work to do.  The wait is a no-op for a kernel launched
// without the attribute.  SHISO_PDL=0 turns the attribute off.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_begin() {
    pdl_trigger();
    pdl_wait();
}

bool shiso_pdl_enabled();  // defined in elementwise.cu

// The word in device memory that a kernel sets when one of its bounded waits ran out
// (defined in gemm_tcgen05.cu).  The token-picking kernels hand it to the host with their
// picks: they read it and set it back to zero.
int* shiso_tc_status_word();

template <typename... KArgs, typename... Args>
static inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // errors surface in launch_status()
}

static inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return (int)e;
}

static inline unsigned ceil_div_u(long long a, long long b) { return (unsigned)((a + b - 1) / b); }
