// Y[T, N] = X[T, K] * W[N, K]^T (+ bias) with float accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path and the product for any
// combination of element types the tensor-core kernels do not take (a matrix kept in
// 32-bit beside 16-bit activations).  Every output element is accumulated by one
// thread over k = 0 .. K-1 in ascending order with fused multiply-adds, so a row's
// result does not depend on how many rows share the launch or where the row lies in
// it - the property the reference calls row-exact
// (crates/shiso-engine/src/projection.rs:972-978).  Any T, N, K >= 1.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename WT, typename XT, typename OT>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(const XT* __restrict__ x, const WT* __restrict__ w, const float* __restrict__ bias,
                   OT* __restrict__ y, int T, int N, int K) {
    pdl_wait();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int ty = tid / (BN / TN), tx = tid % (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = tid; e < BM * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gr = row0 + r, gk = k0 + c;
            xs[c][r] = (gr < T && gk < K) ? to_f32(x[(size_t)gr * K + gk]) : 0.0f;
        }
#pragma unroll
        for (int e = tid; e < BN * BK; e += 256) {
            const int r = e / BK, c = e % BK;
            const int gn = col0 + r, gk = k0 + c;
            ws[c][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gr = row0 + ty * TM + i;
        if (gr >= T) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = col0 + tx * TN + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[gn];
            y[(size_t)gr * N + gn] = from_f32<OT>(v);
        }
    }
}

template <typename WT, typename XT, typename OT>
int launch(const void* x, const void* w, const float* bias, void* y, int T, int N, int K, cudaStream_t stream) {
    dim3 grid(ceil_div_u(N, BN), ceil_div_u(T, BM));
    launch_kernel(gemm_simple_kernel<WT, XT, OT>, grid, 256, 0, stream, (const XT*)x, (const WT*)w, bias, (OT*)y, T, N, K);
    return launch_status();
}

}  // namespace

SHISO_API int shiso_gemm_simple(const void* x, int x_dtype, const void* w, int w_dtype, const float* bias,
                                void* y, int y_dtype, int T, int N, int K, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (K <= 0) return SHISO_ERR_SHAPE;
    using bf = __nv_bfloat16;
    const int code = x_dtype * 4 + w_dtype * 2 + y_dtype;
    switch (code) {
        case 0: return launch<float, float, float>(x, w, bias, y, T, N, K, stream);
        case 1: return launch<float, float, bf>(x, w, bias, y, T, N, K, stream);
        case 2: return launch<bf, float, float>(x, w, bias, y, T, N, K, stream);
        case 3: return launch<bf, float, bf>(x, w, bias, y, T, N, K, stream);
        case 4: return launch<float, bf, float>(x, w, bias, y, T, N, K, stream);
        case 5: return launch<float, bf, bf>(x, w, bias, y, T, N, K, stream);
        case 6: return launch<bf, bf, float>(x, w, bias, y, T, N, K, stream);
        case 7: return launch<bf, bf, bf>(x, w, bias, y, T, N, K, stream);
        default: return SHISO_ERR_DTYPE;
    }
}
