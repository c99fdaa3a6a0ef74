// Y[T, N] = X[T, K] * W[N, K]^T for a handful of rows (T <= 64), bfloat16: the decode step's
// matrix products, which are weight streaming.  (Up to 16 rows the persistent kernel of
// gemm_stream.cu runs them; this one-shot kernel takes 17 to 64.)
//
// At these sizes a product is over in a few microseconds, so what counts is how soon the
// weight bytes are in flight and how little else happens: no tensor map, no tensor memory,
// no cluster.  A CTA owns 16 output features (or 8 gate + 8 up rows of a SwiGLU pair); its
// 8 or 16 warps split K and every lane streams its 16-byte pieces of two weight rows straight
// from global memory, all of a round in flight at once, into mma.sync m16n8k16 (weights are the M operand,
// tokens the N operand).  A lane's 8 consecutive k values feed two MMAs as (k0..k3 | k4..k7);
// the activation fragment is loaded with the same permutation, so the sum over k is the same
// set of products.  The partial tiles are summed through shared memory in warp order,
// so the result does not depend on timing.
//
// What follows the product is folded into the epilogue, because at these sizes every extra
// kernel costs more than its arithmetic:
//   GLU       the weight is a [2 * inter, K] gate-over-up pair; a CTA takes 8 gate rows and
//             their 8 up rows and writes silu(gate) * up (kernels/cuda/generic/glu.cuh:35-57);
// (Two more fusions were built, measured inside a captured step and dropped.  Folding in the
// residual add and the next RMS norm - the CTA that finishes last normalising all rows - cost
// 10.5 us against 6.1 us for product + row kernel: fence, ticket and a single-CTA tail.  Running
// the gated short convolution in the input projection's epilogue won 0.9 us in isolation and
// lost 3 us per layer in the whole step, because its thin tail delays the grid's completion,
// which is what the next product's activations wait for.)
//
// The reference's decode products are matvec kernels that re-read the weights per row block
// (crates/shiso-engine/src/projection.rs:972-1069).
#include "common.cuh"

namespace {


__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Weights are never written while the engine runs: the read-only path may fetch them at any
// time, also before this grid's predecessor has finished.
__device__ __forceinline__ uint4 load_weight16(const __nv_bfloat16* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) v = __ldg(reinterpret_cast<const uint4*>(p));
    return v;
}

// Activations were written by a predecessor grid that may still have been running when this
// grid started: an ordinary (coherent) load, which the compiler keeps after the dependency wait.
// The read-only path (ld.global.nc) must not be used here - it may be hoisted above the wait
// and is not guaranteed to see the predecessor's writes.
__device__ __forceinline__ uint4 load_activation16(const __nv_bfloat16* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) {
        asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    }
    return v;
}

enum { MODE_PLAIN = 0, MODE_GLU = 1 };

struct SkinnyArgs {
    const __nv_bfloat16* x;  // [T, K]
    const __nv_bfloat16* w;  // [N, K]
    const float* bias;       // [N] or null (plain products only)
    void* y;                 // plain [T, N]; GLU [T, inter]
    int T, N, K, inter, out_f32, mode;
};

// NT = 8-token tiles (1, 2, 4 or 8); WARPS_K = warps that split K; UNROLL = 64-wide k blocks per
// warp whose loads (weights and activations) are all issued before the first MMA.
template <int NT, int WARPS_K, int UNROLL>
__global__ void __launch_bounds__(WARPS_K * 32)
gemm_skinny_kernel(SkinnyArgs a) {
    __shared__ float partial[WARPS_K][NT][32][4];
    bool waited = false;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int mode = a.mode;
    // the two rows of the 16 x K weight tile this lane streams: tile rows g and g + 8
    int rows[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        if (mode == MODE_GLU) {
            rows[h] = (h ? a.inter : 0) + blockIdx.x * 8 + g;  // gate row, and its up row
            row_ok[h] = blockIdx.x * 8 + g < a.inter;
        } else {
            rows[h] = blockIdx.x * 16 + r;
            row_ok[h] = rows[h] < a.N;
        }
    }
    const __nv_bfloat16* w_lo = a.w + (size_t)(row_ok[0] ? rows[0] : 0) * a.K;
    const __nv_bfloat16* w_hi = a.w + (size_t)(row_ok[1] ? rows[1] : 0) * a.K;

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;

    // warp w takes the 64-wide k blocks w, w + WARPS_K, ...; a lane owns 16 consecutive k of a block
    for (int k0 = warp * 64; k0 < a.K; k0 += WARPS_K * 64 * UNROLL) {
        uint4 wl[UNROLL][2], wh[UNROLL][2], xv[UNROLL][NT][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = k0 + u * WARPS_K * 64 + t4 * 16;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const bool in = k + h * 8 < a.K;
                wl[u][h] = load_weight16(w_lo + k + h * 8, in && row_ok[0]);
                wh[u][h] = load_weight16(w_hi + k + h * 8, in && row_ok[1]);
            }
        }
        if (!waited) {
            // The weights above depend on no predecessor and are already on their way; the
            // activations below were written by one.
            pdl_wait();
            waited = true;
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = k0 + u * WARPS_K * 64 + t4 * 16;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int token = n * 8 + g;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    xv[u][n][h] = load_activation16(a.x + (size_t)token * a.K + k + h * 8, token < a.T && k + h * 8 < a.K);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    mma_bf16(acc[n], wl[u][h].x, wh[u][h].x, wl[u][h].y, wh[u][h].y, xv[u][n][h].x, xv[u][n][h].y);
                    mma_bf16(acc[n], wl[u][h].z, wh[u][h].z, wl[u][h].w, wh[u][h].w, xv[u][n][h].z, xv[u][n][h].w);
                }
            }
        }
    }

    pdl_trigger();            // the weights are read: the successor may start fetching its own
    if (!waited) pdl_wait();  // a warp whose K range is empty still orders its writes after the predecessor
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) partial[warp][n][lane][e] = acc[n][e];
    __syncthreads();
    for (int i = threadIdx.x; i < NT * 128; i += WARPS_K * 32) {  // one (n, lane, e) element per thread and pass
        const int n = i / 128, l = (i / 4) % 32, e = i % 4;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS_K; ++w) sum += partial[w][n][l][e];
        partial[0][n][l][e] = sum;  // only this thread touches this element
    }
    __syncthreads();
    // In a lane's registers: c0: (row g, token 2t), c1: (row g, token 2t+1), c2/c3: row g + 8.
    if (warp == 0) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int token = n * 8 + t4 * 2 + e;
                if (token >= a.T) continue;
                const float lo = partial[0][n][lane][e], hi = partial[0][n][lane][2 + e];
                if (mode == MODE_GLU) {
                    if (row_ok[0]) {
                        const float v = lo / (1.0f + expf(-lo)) * hi;
                        const size_t at = (size_t)token * a.inter + blockIdx.x * 8 + g;
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                } else {
                    if (row_ok[0]) {
                        const float v = lo + (a.bias ? a.bias[rows[0]] : 0.0f);
                        const size_t at = (size_t)token * a.N + rows[0];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                    if (row_ok[1]) {
                        const float v = hi + (a.bias ? a.bias[rows[1]] : 0.0f);
                        const size_t at = (size_t)token * a.N + rows[1];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
}

int launch_skinny(const SkinnyArgs& a, unsigned blocks, cudaStream_t stream) {
    // enough warps per CTA that one round of loads covers the CTA's whole K range
    const bool deep = a.K > 3072;
#define SHISO_LAUNCH(NT_, WK_, UN_) launch_kernel(gemm_skinny_kernel<NT_, WK_, UN_>, blocks, WK_ * 32, 0, stream, a)
    if (a.T <= 8) {
        if (deep) SHISO_LAUNCH(1, 16, 4);
        else SHISO_LAUNCH(1, 8, 4);
    } else if (a.T <= 16) {
        if (deep) SHISO_LAUNCH(2, 16, 4);
        else SHISO_LAUNCH(2, 8, 4);
    } else if (a.T <= 32) {
        if (deep) SHISO_LAUNCH(4, 16, 2);
        else SHISO_LAUNCH(4, 8, 2);
    } else {
        SHISO_LAUNCH(8, 8, 1);  // 16 warps would need more static shared memory than a CTA may have
    }
#undef SHISO_LAUNCH
    return launch_status();
}

}  // namespace

// x [T, K] bf16 (T <= 64), w [N, K] bf16, K a multiple of 8, pointers 16-byte aligned.
// inter == 0: y[T, N] = x w^T (+ bias).  inter > 0: N == 2 * inter, y[T, inter] = silu(x gate^T) * (x up^T).
SHISO_API int shiso_gemm_skinny(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T, int N,
                                int K, int inter, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (T > 64 || K % 8 != 0 || K <= 0) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return SHISO_ERR_ALIGN;
    if (inter > 0 && (N != 2 * inter || bias)) return SHISO_ERR_SHAPE;
    SkinnyArgs a = {};
    a.x = (const __nv_bfloat16*)x;
    a.w = (const __nv_bfloat16*)w;
    a.bias = bias;
    a.y = y;
    a.T = T;
    a.N = N;
    a.K = K;
    a.inter = inter;
    a.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    a.mode = inter > 0 ? MODE_GLU : MODE_PLAIN;
    return launch_skinny(a, inter > 0 ? ceil_div_u(inter, 8) : ceil_div_u(N, 16), stream);
}
