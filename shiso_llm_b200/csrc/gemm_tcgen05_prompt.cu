// Y[T, N] = X[T, K] * W[N, K]^T for prompt-sized T (>= 128 rows), bfloat16: a persistent,
// warp-specialised tcgen05 kernel.
//
// Tile: 128 tokens (the MMA's M operand) x 256 weight rows (its N operand) x 64 k per stage;
// the accumulator is 128 TMEM lanes x 256 float columns and there are two of them (all 512
// columns), so the epilogue of one tile runs while the tensor core works on the next.
// One CTA per SM walks the tiles (token tiles fastest, so CTAs running together share a
// weight tile in L2).  Six warps: warp 0 issues the TMA loads (one lane), warp 1 allocates
// TMEM and issues tcgen05.mma (one lane), warps 2-5 are the epilogue: each owns 32 TMEM lanes
// = 32 tokens, reads 16 columns at a time with tcgen05.ld and stores 32 contiguous bytes of a
// token's row.  Four mbarrier families hand work around: full/empty per shared-memory stage
// (TMA -> MMA -> TMA), acc_full/acc_empty per accumulator (MMA -> epilogue -> MMA).
//
// With `inter > 0` the 256 weight rows of a tile are 128 gate rows and the matching 128 up
// rows of a [2 * inter, K] pair (two TMA boxes, adjacent in shared memory, one MMA), and the
// epilogue writes silu(gate) * up: the [T, 2 * inter] intermediate never exists.
//
// No multicast.  Every wait is bounded by a clock limit and reports through the status word.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int TILE_M = 128;   // tokens
constexpr int TILE_N = 256;   // weight rows (features, or 128 gate + 128 up)
constexpr int STAGES = 4;
constexpr int THREADS = 192;
constexpr int A_BYTES = TILE_M * BK * 2;
constexpr int B_BYTES = TILE_N * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct PromptParams {
    void* y;
    const float* bias;
    int* status;
    int T, N, K;     // N: rows of y
    int inter;       // > 0: gate/up pair, N == inter
    int out_f32;
    int m_tiles, n_tiles;
    // SCALED, as in gemm_tcgen05_pair.cu: row t of x lacks the factor rsqrt(sum over c < scale_count
    // of scale_partials[c * scale_stride + t] / K + scale_eps); it is applied to the accumulators
    const float* scale_partials;
    int scale_count, scale_stride;
    float scale_eps;
};

__device__ __forceinline__ void store16(const PromptParams& p, int token, int feature, const float* v) {
    // 16 consecutive features of one token; rows of y are 16-byte aligned (N % 8 == 0 is checked on the host)
    if (feature + 16 <= p.N) {
        if (p.out_f32) {
            float4* dst = reinterpret_cast<float4*>((float*)p.y + (size_t)token * p.N + feature);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            uint4 lo, hi;
            __nv_bfloat162* l = reinterpret_cast<__nv_bfloat162*>(&lo);
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&hi);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                l[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                h[i] = __floats2bfloat162_rn(v[8 + 2 * i], v[8 + 2 * i + 1]);
            }
            uint4* dst = reinterpret_cast<uint4*>((__nv_bfloat16*)p.y + (size_t)token * p.N + feature);
            dst[0] = lo;
            dst[1] = hi;
        }
    } else {
        for (int i = 0; i < 16 && feature + i < p.N; ++i) {
            const size_t at = (size_t)token * p.N + feature + i;
            if (p.out_f32) ((float*)p.y)[at] = v[i];
            else ((__nv_bfloat16*)p.y)[at] = __float2bfloat16_rn(v[i]);
        }
    }
}

template <bool GLU>
__global__ void __launch_bounds__(THREADS, 1)
gemm_prompt_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, PromptParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;    // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    int* failed = (int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int num_tiles = p.m_tiles * p.n_tiles;
    const int out_per_tile = GLU ? TILE_N / 2 : TILE_N;  // output features a tile produces

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * TILE_M;
                const int n0 = (tile / p.m_tiles) * out_per_tile;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
                        *failed = 1;
                        ok = false;
                        break;
                    }
                    uint8_t* a = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int k = kb * BK;
                    if (GLU) {
                        tma_load_2d(a + A_BYTES, &map_w, k, n0, &full[s]);
                        tma_load_2d(a + A_BYTES + B_BYTES / 2, &map_w, k, p.inter + n0, &full[s]);
                    } else {
                        tma_load_2d(a + A_BYTES, &map_w, k, n0, &full[s]);
                    }
                    if (it == 0) pdl_wait();  // weights depend on no predecessor; the activations do
                    tma_load_2d(a, &map_x, k, m0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            const uint32_t idesc = umma_idesc(TILE_M, TILE_N);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int acc = local & 1;
                if (local >= 2 && !mbar_wait(&acc_empty[acc], ((local >> 1) - 1) & 1)) {
                    *failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * TILE_N;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
                        *failed = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(d_tmem, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty[s]);
                }
                umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---- epilogue warps 2..5: TMEM lanes (warp % 4) * 32 .., one token per thread
        pdl_wait();
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int acc = local & 1;
            const int m0 = (tile % p.m_tiles) * TILE_M;
            const int n0 = (tile / p.m_tiles) * out_per_tile;
            const int token = m0 + quarter * 32 + lane;
            float row_scale = 1.0f;
            if (p.scale_partials) {  // asked for before the accumulator is waited for
                float sum = 0.0f;
                if (token < p.T) {
                    const float* mine = p.scale_partials + token;
                    int c = 0;
                    for (; c + 8 <= p.scale_count; c += 8) {  // eight loads in flight, added in index order
                        float part[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) part[u] = mine[(size_t)(c + u) * p.scale_stride];
#pragma unroll
                        for (int u = 0; u < 8; ++u) sum += part[u];
                    }
                    for (; c < p.scale_count; ++c) sum += mine[(size_t)c * p.scale_stride];
                }
                row_scale = rsqrtf(sum / (float)p.K + p.scale_eps);
            }
            if (!mbar_wait(&acc_full[acc], (local >> 1) & 1)) {
                *failed = 1;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * TILE_N;
            // Four TMEM loads are in flight before the one wait: 64 columns a round (32 gate and
            // 32 up for the pair), so the round trip to TMEM is paid 4 times a tile, not 16.
            constexpr int ROUND = GLU ? 32 : 64;
#pragma unroll 1
            for (int c = 0; c < out_per_tile; c += ROUND) {
                uint32_t r[4][16];
                if (GLU) {
                    tmem_ld16_issue(taddr + c, r[0]);
                    tmem_ld16_issue(taddr + c + 16, r[1]);
                    tmem_ld16_issue(taddr + TILE_N / 2 + c, r[2]);
                    tmem_ld16_issue(taddr + TILE_N / 2 + c + 16, r[3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) tmem_ld16_issue(taddr + c + 16 * q, r[q]);
                }
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) tmem_ld_pin(r[q]);
#pragma unroll
                for (int q = 0; q < (GLU ? 2 : 4); ++q) {
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[q][i]) * row_scale;
                    const int feature = n0 + c + 16 * q;
                    if (GLU) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = silu_times(v[i], __uint_as_float(r[q + 2][i]) * row_scale);
                    } else if (p.bias) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (feature + i < p.N) v[i] += p.bias[feature + i];
                    }
                    if (token < p.T && feature < p.N) store16(p, token, feature, v);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }
    pdl_trigger();
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*failed != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, 1);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

template <bool GLU>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const PromptParams& p, int sm_count, cudaStream_t stream) {
    auto kernel = gemm_prompt_kernel<GLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = p.m_tiles * p.n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles < sm_count ? tiles : sm_count);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, mx, mw, p);
}

}  // namespace

namespace {

int run_prompt(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T, int N, int K, int inter,
               const float* partials, int partial_count, int partial_stride, float eps, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (K % 8 != 0 || K < 8 || N % 8 != 0) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return SHISO_ERR_ALIGN;
    if (inter > 0 && (N != inter || bias)) return SHISO_ERR_SHAPE;
    if (tc::encode_fn() == nullptr) return SHISO_ERR_UNSUPPORTED;
    PromptParams p = {};
    p.y = y;
    p.bias = bias;
    p.status = shiso_tc_status_word();
    p.T = T;
    p.N = N;
    p.K = K;
    p.inter = inter;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    p.m_tiles = (T + TILE_M - 1) / TILE_M;
    const int out_per_tile = inter > 0 ? TILE_N / 2 : TILE_N;
    p.n_tiles = (N + out_per_tile - 1) / out_per_tile;
    p.scale_partials = partials;
    p.scale_count = partial_count;
    p.scale_stride = partial_stride;
    p.scale_eps = eps;
    CUtensorMap mx, mw;
    const int w_rows = inter > 0 ? 2 * inter : N;
    if (!tc::tensor_map(x, T, K, TILE_M, &mx) || !tc::tensor_map(w, w_rows, K, out_per_tile, &mw)) return SHISO_ERR_UNSUPPORTED;
    if (inter > 0) return launch<true>(mx, mw, p, sm_count, stream);
    return launch<false>(mx, mw, p, sm_count, stream);
}

}  // namespace

// x [T, K] bf16, w [N, K] (inter == 0) or [2 * inter, K] gate over up (inter > 0, N == inter), y [T, N].
// K and N multiples of 8, pointers 16-byte aligned.
SHISO_API int shiso_gemm_tcgen05_prompt(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T,
                                        int N, int K, int inter, int sm_count, cudaStream_t stream) {
    return run_prompt(x, w, bias, y, y_dtype, T, N, K, inter, nullptr, 0, 0, 0.0f, sm_count, stream);
}

// The same for rows x that lack their RMS scale (see PromptParams).
SHISO_API int shiso_gemm_tcgen05_prompt_scaled(const void* x, const float* partials, int partial_count, int partial_stride,
                                               float eps, const void* w, void* y, int y_dtype, int T, int N, int K,
                                               int inter, int sm_count, cudaStream_t stream) {
    if (!partials || partial_count <= 0 || partial_stride < T) return SHISO_ERR_UNSUPPORTED;
    return run_prompt(x, w, nullptr, y, y_dtype, T, N, K, inter, partials, partial_count, partial_stride, eps, sm_count, stream);
}
