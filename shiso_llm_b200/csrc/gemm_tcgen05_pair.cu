// Y[T, N] = X[T, K] * W[N, K]^T for long prompts (T >= 256 rows), bfloat16: the persistent
// warp-specialised kernel of gemm_tcgen05_prompt.cu on pairs of SMs (tcgen05 cta_group::2).
//
// Why pairs.  A 128 x 256 tile per SM needs 48 KB of operands per 64-wide k step, and the tensor
// core finishes a step in about 270 ns: all SMs together would have to pull some 26 TB/s out of
// L2, which it does not deliver, so the single-SM kernel runs at about half the tensor rate.
// Two CTAs of a cluster working on one 256-token x 256-row tile load 128 tokens and 128 weight
// rows each (32 KB a step per SM); the MMA of the leader CTA reads both halves of the weight
// operand across the pair.  The smaller stage also lets six of them fit, which covers more
// latency.
//
// Roles in each CTA (192 threads): warp 0 lane 0 issues this CTA's TMA loads, whose bytes are
// counted on the LEADER's full barrier; warp 1 allocates TMEM (both CTAs, collectively) and,
// in the leader only, issues the MMAs and commits to the barriers of both CTAs; warps 2-5 are
// the epilogue of this CTA's 128 tokens.  Barriers: full[s] (leader: TMA bytes of both CTAs),
// empty[s] (each CTA: its stage may be refilled), acc_full[a] (each CTA: accumulator a is
// complete), acc_empty[a] (leader: the epilogue warps of both CTAs have drained a).
//
// With `inter > 0` the leader CTA loads 128 gate rows and its peer the matching 128 up rows, so
// the accumulator's columns 0..127 are gate and 128..255 up, and the epilogue writes
// silu(gate) * up.
//
// Measured and dropped: dealing the work out as equal shares of all k blocks of all tiles laid
// end to end, so that no wave of tiles is left part empty (96 tiles on 74 pairs), with the pair
// that has a tile's first k block adding the partial accumulators the others leave in global
// memory.  Right results, slower products: 2,048 x 6144 x 2048 took 50.0 us against 38.6,
// 2,048 x 2048 x 2048 31.8 against 17.3 - every pair then ends with a tile it has to wait and
// add for, the 19 MB of partial sums go through the L2 that already bounds the main loop, and
// the pairs no longer walk the k blocks of neighbouring tiles in step.
//
// (Also measured and dropped: bfloat16 results leaving through shared memory and TMA stores of
// 32 rows x 64 columns instead of a thread writing 32-byte pieces of its own row - 17.0 against
// 17.3 us for 2,048 x 2048 x 2048, 38.7 against 38.6 for 6144 features: the epilogue's time is
// not in how its stores are shaped.)
//
// (Measured and dropped: the residual add and the first half of the next RMS norm in this
// epilogue, as the kernels for a few rows have them.  A product of 2,048 x 2,048 features is one
// tile a pair, so its whole epilogue stands at the kernel's end; reading and writing the float
// stream there took the tail from 3.1 to 14.8 us - more than the 10 us of the norm kernel it
// would replace - and even as whole lines the 42 MB would all move in that tail.)
//
// (Measured and dropped: pair tiles narrower than 256 weight rows where that saves a wave -
// 72 tiles of 240 for 2,048 features instead of 64 of 256 on 74 pairs, 128 tiles of 192 for
// 3,072 features instead of 96 of 256.  The prompt step took 3.26 ms either way; with 240 rows for
// every product 3.29 ms, with 192 rows 3.87 ms: a narrower tile brings less arithmetic per byte
// it loads, and that costs what the fuller waves save.)
//
// The loads carry no multicast qualifier.  Every wait is bounded by a clock limit; a CTA that
// gives up sets the status word, and all CTAs still meet at the cluster barrier before TMEM is
// freed.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int HALF_M = 128;    // tokens per CTA
constexpr int TILE_N = 256;    // weight rows per pair tile
constexpr int HALF_N = 128;    // weight rows each CTA loads
constexpr int STAGES = 6;
constexpr int THREADS = 192;
constexpr int A_BYTES = HALF_M * BK * 2;
constexpr int B_BYTES = HALF_N * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct PairParams {
    void* y;
    const float* bias;
    int* status;
    int T, N, K;
    int inter;  // > 0: gate/up pair, N == inter
    int out_f32;
    int m_tiles, n_tiles;  // pair tiles: 256 tokens x (256 rows, or 128 outputs of a gate/up pair)
    // SCALED: the rows of x lack their RMS scale (they are what a product into the stream left:
    // gemm_tcgen05.cu); row t is scaled by rsqrt(sum over c < scale_count of
    // scale_partials[c * scale_stride + t] / K + scale_eps), applied to the accumulators - a
    // thread owns a row here, so it is one factor a thread and tile
    const float* scale_partials;
    int scale_count, scale_stride;
    float scale_eps;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// The shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank`.
__device__ __forceinline__ uint32_t peer_address(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// TMA load into this CTA's shared memory whose bytes are counted on a barrier that may live in
// the peer CTA (`bar_cluster` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// mbar_wait for a barrier that threads of the peer CTA arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    const unsigned long long start = clock64();
    while (true) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (clock64() - start > WAIT_LIMIT_CYCLES) return false;
    }
}

// 32 bytes in one store: a whole sector per thread.  (With two 16-byte stores per sector the last
// 128 x 256 tile of a CTA - every CTA writes its last tile at the same time - took 3.6 to 5.0 us
// from the last MMA to the last store, 1.5 us with the stores taken out and 3.1 us with these.
// Turning a warp's rows through shared memory so that every store instruction writes whole
// 128-byte lines was no faster, 3.3 to 3.6 us: what is left is the 9 MB that all CTAs write at once.)
__device__ __forceinline__ void store32(void* dst, const uint32_t* r) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(dst), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void store16(const PairParams& p, int token, int feature, const float* v) {
    // 16 consecutive features of one token; rows of y are 16-byte aligned (N % 8 == 0 is checked on the host)
    if (feature + 16 <= p.N) {
        if (p.out_f32) {
            float* dst = (float*)p.y + (size_t)token * p.N + feature;
            if (((uintptr_t)dst & 31) == 0) {
                store32(dst, reinterpret_cast<const uint32_t*>(v));
                store32(dst + 8, reinterpret_cast<const uint32_t*>(v + 8));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            }
        } else {
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t*>(&pair);
            }
            __nv_bfloat16* dst = (__nv_bfloat16*)p.y + (size_t)token * p.N + feature;
            if (((uintptr_t)dst & 31) == 0) {
                store32(dst, packed);
            } else {
                reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (feature + i < p.N) {
                const size_t at = (size_t)token * p.N + feature + i;
                if (p.out_f32) ((float*)p.y)[at] = v[i];
                else ((__nv_bfloat16*)p.y)[at] = __float2bfloat16_rn(v[i]);
            }
        }
    }
}

template <bool GLU>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;    // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    int* failed = (int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int k_blocks = (p.K + BK - 1) / BK;
    const int num_tiles = p.m_tiles * p.n_tiles;
    const int out_per_tile = GLU ? TILE_N / 2 : TILE_N;
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);   // the leader's arrive.expect_tx; bytes come from both CTAs
            mbar_init(&empty[s], 1);  // one commit
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);   // one commit
            mbar_init(&acc_empty[i], 8);  // four epilogue warps in each CTA (used in the leader)
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is signalled on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer of this CTA's halves
            int it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                const int m0 = (tile % p.m_tiles) * (2 * HALF_M) + (int)rank * HALF_M;
                const int n_tile0 = (tile / p.m_tiles) * out_per_tile;
                const int w_row = GLU ? (leader ? n_tile0 : p.inter + n_tile0) : n_tile0 + (int)rank * HALF_N;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
                        *failed = 1;
                        ok = false;
                        break;
                    }
                    uint8_t* a = smem + s * STAGE_BYTES;
                    const uint32_t bar = peer_address(smem_u32(&full[s]), 0);
                    if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                    const int k = kb * BK;
                    tma_load_2d_pair(a + A_BYTES, &map_w, k, w_row, bar);
                    if (it == 0) pdl_wait();  // weights depend on no predecessor; the activations do
                    tma_load_2d_pair(a, &map_x, k, m0, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---- MMA issuer of the pair
            const uint32_t idesc = umma_idesc(2 * HALF_M, TILE_N);
            int it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
                const int acc = local & 1;
                if (local >= 2 && !mbar_wait_cluster(&acc_empty[acc], ((local >> 1) - 1) & 1)) {
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
                        umma_bf16_pair(d_tmem, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                umma_commit_pair(&acc_full[acc]);
            }
        }
    } else {
        // ---- epilogue warps 2..5: TMEM lanes (warp % 4) * 32 .., one token per thread
        pdl_wait();
        const int quarter = warp & 3;
        const uint32_t empty_bar[2] = {peer_address(smem_u32(&acc_empty[0]), 0), peer_address(smem_u32(&acc_empty[1]), 0)};
        int local = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++local) {
            const int acc = local & 1;
            const int m0 = (tile % p.m_tiles) * (2 * HALF_M) + (int)rank * HALF_M;
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
            // four TMEM loads in flight before the one wait (32 gate and 32 up columns for the pair)
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
            if (lane == 0) mbar_arrive_cluster(empty_bar[acc]);
        }
    }
    pdl_trigger();
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*failed != 0 && threadIdx.x == 0 && p.status) atomicExch(p.status, 1);
    cluster_sync_all();  // nobody signals into, or frees, a CTA that a peer still uses
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

template <bool GLU>
int launch(const CUtensorMap& mx, const CUtensorMap& mw, const PairParams& p, int sm_count, cudaStream_t stream) {
    auto kernel = gemm_pair_kernel<GLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = p.m_tiles * p.n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count & ~1);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    // The tiles are dealt out to the clusters in advance, so every cluster must be running from
    // the start: the grid is as many pairs as the device can hold at once (SMs of a pair share
    // a GPC, so this can be fewer than half the SMs).
    static int resident_pairs = 0;
    if (resident_pairs == 0) {
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            return SHISO_ERR_UNSUPPORTED;
        }
        resident_pairs = clusters < sm_count / 2 ? clusters : sm_count / 2;
    }
    cfg.gridDim = dim3(2 * (tiles < resident_pairs ? tiles : resident_pairs));
    return (int)cudaLaunchKernelEx(&cfg, kernel, mx, mw, p);
}

}  // namespace

namespace {

int run_pair(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T, int N, int K, int inter,
             const float* partials, int partial_count, int partial_stride, float eps, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (K % 8 != 0 || K < 8 || N % 8 != 0 || sm_count < 2) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return SHISO_ERR_ALIGN;
    if (inter > 0 && (N != inter || bias)) return SHISO_ERR_SHAPE;
    if (tc::encode_fn() == nullptr) return SHISO_ERR_UNSUPPORTED;
    PairParams p = {};
    p.y = y;
    p.bias = bias;
    p.status = shiso_tc_status_word();
    p.T = T;
    p.N = N;
    p.K = K;
    p.inter = inter;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    p.m_tiles = (T + 2 * HALF_M - 1) / (2 * HALF_M);
    const int out_per_tile = inter > 0 ? TILE_N / 2 : TILE_N;
    p.n_tiles = (N + out_per_tile - 1) / out_per_tile;
    p.scale_partials = partials;
    p.scale_count = partial_count;
    p.scale_stride = partial_stride;
    p.scale_eps = eps;
    CUtensorMap mx, mw;
    const int w_rows = inter > 0 ? 2 * inter : N;
    if (!tc::tensor_map(x, T, K, HALF_M, &mx) || !tc::tensor_map(w, w_rows, K, HALF_N, &mw)) return SHISO_ERR_UNSUPPORTED;
    if (inter > 0) return launch<true>(mx, mw, p, sm_count, stream);
    return launch<false>(mx, mw, p, sm_count, stream);
}

}  // namespace

// x [T, K] bf16, w [N, K] (inter == 0) or [2 * inter, K] gate over up (inter > 0, N == inter), y [T, N].
// K and N multiples of 8, pointers 16-byte aligned.
SHISO_API int shiso_gemm_tcgen05_pair(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T,
                                      int N, int K, int inter, int sm_count, cudaStream_t stream) {
    return run_pair(x, w, bias, y, y_dtype, T, N, K, inter, nullptr, 0, 0, 0.0f, sm_count, stream);
}

// The same for rows x that lack their RMS scale (see PairParams): row t is scaled by
// rsqrt(sum over c < partial_count of partials[c * partial_stride + t] / K + eps).
SHISO_API int shiso_gemm_tcgen05_pair_scaled(const void* x, const float* partials, int partial_count, int partial_stride,
                                             float eps, const void* w, void* y, int y_dtype, int T, int N, int K,
                                             int inter, int sm_count, cudaStream_t stream) {
    if (!partials || partial_count <= 0 || partial_stride < T) return SHISO_ERR_UNSUPPORTED;
    return run_pair(x, w, nullptr, y, y_dtype, T, N, K, inter, partials, partial_count, partial_stride, eps, sm_count, stream);
}
