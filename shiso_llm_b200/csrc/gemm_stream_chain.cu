// A chain of weight-streaming products in ONE persistent kernel: the decode step's products for up
// to 8 rows, from one kernel that is not a product (embedding, attention) to the next.
//
// A product of a decode step reads 8 to 46 MB of weights and is over in a few microseconds; as a
// kernel of its own it pays a start and a tail that the next kernel's start only partly covers
// (measured: about 2.5 us each, half of a step's time at batch 8).  Weights depend on no activation,
// so here the producer warp of every CTA walks the whole list of products and never stops: while
// the consumers of all CTAs meet between two products, the rings (six stages of 33 KB on each of
// 148 SMs) go on filling with the next product's weights, and the memory system sees one stream
// from the first product's first row to the last product's last.
//
// One CTA per SM.  The consumers of product p + 1 may read what the epilogues of product p wrote
// anywhere on the device, so between two products all CTAs meet at a counter in global memory: a
// CTA's epilogue warp adds one after its last store (behind a fence), one thread per CTA polls
// until all have, and the last CTA past the barrier sets the counter back to zero for the next
// launch.  All CTAs are resident at once (the grid is at most the number of SMs and a CTA fits an
// SM), so the wait ends; it is bounded by the clock limit all the same and reports through the
// status word.  What a predecessor product wrote is read with loads that go to L2 (ld.global.cg):
// a line that this SM read earlier in the kernel may sit in its L1, since buffers of one step
// reuse addresses.
//
// Tiles of a product go round the CTAs starting where the product before it stopped, so the CTAs
// that a short product leaves without a tile are not the same ones every time.
//
// The product itself (tiles of 16 weight rows, mma.sync with the weights as the M operand, the
// partial sums of four consumer warps meeting in shared memory) and its epilogues (bias, SwiGLU,
// residual add + next norm's weight + partial squares, row scale, short convolution) are those of
// gemm_stream.cu, with the mode read at run time: one CTA per SM has registers to spare.
#include "gemm_stream.cuh"

#include <vector>

namespace {

using namespace stream;

constexpr int CHAIN_MAX = 16;    // products per launch (the argument block must stay under 4 KB)
constexpr int CHAIN_STAGES = 6;  // ring stages of 33 KB

struct ChainArgs {
    StreamArgs p[CHAIN_MAX];
    int first_owner[CHAIN_MAX];  // the CTA that takes tile 0 of product i
    int count;
    unsigned* arrived;  // [CHAIN_MAX] CTAs whose stores of product i are done
    unsigned* passed;   // [CHAIN_MAX] CTAs that have gone past the barrier behind product i
};
static_assert(sizeof(ChainArgs) <= 4000, "kernel arguments are limited to 4 KB");

__device__ __forceinline__ uint4 load_cg16(const __nv_bfloat16* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) {
        asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    }
    return v;
}

__device__ __forceinline__ float load_cg1(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ int row_of(const StreamArgs& a, int tile, int r) {
    return a.mode == MODE_CONV ? tile_row<true>(a, tile, r) : tile_row<false>(a, tile, r);
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_chain_kernel(const __grid_constant__ ChainArgs c) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    uint64_t* full = (uint64_t*)(ring + CHAIN_STAGES * STAGE_BYTES);
    uint64_t* empty = full + CHAIN_STAGES;
    float* partial = (float*)(empty + CHAIN_STAGES);       // [2][CONSUMERS][32][4]
    float* square_parts = partial + 2 * CONSUMERS * 128;   // [16][PARTIAL_STRIDE]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int grid = (int)gridDim.x;
    bool timed_out = false;
    int* const status = c.p[0].status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < CHAIN_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // ---- producer: through every product without a stop; lane r copies row r of each stage
        int unit = 0;
        for (int p = 0; p < c.count; ++p) {
            const StreamArgs& a = c.p[p];
            const int K = a.K, tiles = a.tiles;
            const int chunks = (K + KC - 1) / KC;
            for (int tile = (blockIdx.x + grid - c.first_owner[p]) % grid; tile < tiles; tile += grid) {
                const int row = lane < ROWS ? row_of(a, tile, lane) : -1;
                const int present = __popc(__ballot_sync(0xffffffffu, row >= 0));
                const __nv_bfloat16* src = a.w + (size_t)(row >= 0 ? row : 0) * K;
                for (int ch = 0; ch < chunks; ++ch, ++unit) {
                    const int s = unit % CHAIN_STAGES;
                    if (unit >= CHAIN_STAGES && !mbar_wait(&empty[s], ((unit / CHAIN_STAGES) - 1) & 1)) timed_out = true;
                    const int cols = min(KC, K - ch * KC);
                    if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)(present * cols * 2));
                    __syncwarp();
                    if (row >= 0)
                        bulk_load(smem_u32(ring + s * STAGE_BYTES) + lane * ROW_BYTES, src + (size_t)ch * KC, (uint32_t)(cols * 2), &full[s]);
                }
            }
        }
        if (timed_out && lane == 0 && status) atomicExch(status, 1);
        pdl_trigger();
        return;
    }

    // ---- consumers
    const int g = lane >> 2, t4 = lane & 3;
    pdl_wait();
    int unit = 0, local = 0;

    for (int p = 0; p < c.count; ++p) {
        const StreamArgs& a = c.p[p];
        if (p > 0) {
            // every CTA's stores of product p - 1 are done before anything of product p is read
            if (threadIdx.x == 0) {
                const unsigned long long start = clock64();
                while (true) {
                    unsigned seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(c.arrived + (p - 1)) : "memory");
                    if (seen >= (unsigned)grid) break;
                    if (clock64() - start > tc::WAIT_LIMIT_CYCLES) {
                        timed_out = true;
                        break;
                    }
                }
                if (atomicAdd(c.passed + (p - 1), 1u) == (unsigned)grid - 1) {  // the last one past it clears it
                    c.passed[p - 1] = 0u;
                    c.arrived[p - 1] = 0u;
                }
            }
            consumer_barrier();
        }
        const int T = a.T, N = a.N, K = a.K, tiles = a.tiles, mode = a.mode;
        const bool conv = mode == MODE_CONV;
        const int chunks = (K + KC - 1) / KC;
        const bool held = chunks <= 2;
        const __nv_bfloat16* const x = a.x;
        const float* const partials_in = a.partials_in;
        const float* const res_in = a.res_in;

        auto load_x = [&](int ch, uint4 (&xv)[KB][2]) {
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const int k = ch * KC + warp * (KC / CONSUMERS) + kb * 64 + t4 * 16;
#pragma unroll
                for (int h = 0; h < 2; ++h) xv[kb][h] = load_cg16(x + (size_t)g * K + k + h * 8, g < T && k + h * 8 < K);
            }
        };

        // SCALED: the partial squares, asked for now and summed at the first epilogue
        constexpr int SLOTS = 16 * PARTIAL_STRIDE / (CONSUMERS * 32);
        float early_part[SLOTS][EARLY_PARTIALS];
        if (partials_in) {
#pragma unroll
            for (int q = 0; q < SLOTS; ++q) {
                const int i = threadIdx.x + q * CONSUMERS * 32;
                const int group = i / PARTIAL_STRIDE, token = i % PARTIAL_STRIDE;
#pragma unroll
                for (int j = 0; j < EARLY_PARTIALS; ++j) {
                    const int row = group + 16 * j;
                    early_part[q][j] = row < a.partial_count ? load_cg1(partials_in + (size_t)row * PARTIAL_STRIDE + token) : 0.0f;
                }
            }
        }

        const int conv_token = lane & 7;
        long long conv_slot = -1;
        if (conv && warp == 0 && conv_token < T) conv_slot = a.conv_slots[a.conv_seq_of_token[conv_token]];

        uint4 xs[2][KB][2];
        load_x(0, xs[0]);
        if (held && chunks == 2) load_x(1, xs[1]);
        bool scale_ready = false;

        for (int tile = (blockIdx.x + grid - c.first_owner[p]) % grid; tile < tiles; tile += grid, ++local) {
            float early_res[2][2], early_nw[2] = {0.0f, 0.0f}, early_bias[2] = {0.0f, 0.0f};
            int rows[2];
            rows[0] = row_of(a, tile, g);
            rows[1] = row_of(a, tile, g + 8);
            if (warp == 0) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (rows[h] >= 0 && mode == MODE_PLAIN) {
                        if (a.bias) early_bias[h] = a.bias[rows[h]];
                        if (res_in) early_nw[h] = a.next_norm_w[rows[h]];
                    }
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int token = t4 * 2 + e;
                        early_res[e][h] = 0.0f;
                        if (res_in && rows[h] >= 0 && token < T) early_res[e][h] = load_cg1(res_in + (size_t)token * N + rows[h]);
                    }
                }
            }

            float conv_window[2][CONV_MAX_TAPS - 1], conv_tap[2][CONV_MAX_TAPS], conv_b[2] = {0.0f, 0.0f};
            if (conv && warp == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int ch = tile * CONV_CHANNELS + (i == 0 ? lane >> 3 : 4);
                    const bool on = conv_slot >= 0 && ch < a.hidden && (i == 0 || lane < 8);
#pragma unroll
                    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
                        conv_tap[i][j] = (on && j < a.conv_taps) ? a.conv_w[(size_t)ch * a.conv_taps + j] : 0.0f;
                        if (j < CONV_MAX_TAPS - 1)
                            conv_window[i][j] = (on && j < a.conv_taps - 1)
                                ? load_cg1(a.conv_state + conv_slot * a.conv_slot_stride + (size_t)j * a.hidden + ch) : 0.0f;
                    }
                    if (on && a.conv_bias) conv_b[i] = a.conv_bias[ch];
                }
            }

            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            auto work = [&](int ch, uint4 (&xv)[KB][2]) {
                const int s = unit % CHAIN_STAGES;
                if (!mbar_wait(&full[s], (unit / CHAIN_STAGES) & 1)) timed_out = true;
                const uint32_t base = smem_u32(ring + s * STAGE_BYTES);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const int col = warp * (KC / CONSUMERS) + kb * 64 + t4 * 16;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint4 wl = make_uint4(0u, 0u, 0u, 0u), wh = wl;
                        if (ch * KC + col + h * 8 < K) {
                            wl = lds16(base + g * ROW_BYTES + (col + h * 8) * 2);
                            wh = lds16(base + (g + 8) * ROW_BYTES + (col + h * 8) * 2);
                        }
                        mma_bf16(acc, wl.x, wh.x, wl.y, wh.y, xv[kb][h].x, xv[kb][h].y);
                        mma_bf16(acc, wl.z, wh.z, wl.w, wh.w, xv[kb][h].z, xv[kb][h].w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
                ++unit;
            };
            if (held) {
                work(0, xs[0]);
                if (chunks == 2) work(1, xs[1]);
            } else {
                for (int ch = 0; ch < chunks; ++ch) {
                    const int next_ch = ch + 1 < chunks ? ch + 1 : 0;
                    const bool more = ch + 1 < chunks || tile + grid < tiles;
                    if (more) load_x(next_ch, xs[1]);
                    work(ch, xs[0]);
                    if (more) {
#pragma unroll
                        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                            for (int h = 0; h < 2; ++h) xs[0][kb][h] = xs[1][kb][h];
                    }
                }
            }

            // ---- the tile's partial sums meet in shared memory, in warp order
            float* mine = partial + (size_t)(local & 1) * CONSUMERS * 128;
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[(warp * 32 + lane) * 4 + e] = acc[e];
            if (!scale_ready && partials_in) {
#pragma unroll
                for (int q = 0; q < SLOTS; ++q) {
                    const int i = threadIdx.x + q * CONSUMERS * 32;
                    const int group = i / PARTIAL_STRIDE, token = i % PARTIAL_STRIDE;
                    float sum = 0.0f;
#pragma unroll
                    for (int j = 0; j < EARLY_PARTIALS; ++j) sum += early_part[q][j];
                    for (int row = group + 16 * EARLY_PARTIALS; row < a.partial_count; row += 16)
                        sum += load_cg1(partials_in + (size_t)row * PARTIAL_STRIDE + token);
                    square_parts[group * PARTIAL_STRIDE + token] = sum;
                }
                scale_ready = true;
            }
            consumer_barrier();
            {
                const int i = threadIdx.x;  // 128 threads, 128 sums
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < CONSUMERS; ++w) sum += mine[w * 128 + i];
                mine[i] = sum;  // only this thread touches this element
            }
            consumer_barrier();
            if (warp != 0) continue;

            // ---- epilogue (warp 0).  In a lane: c0: (row g, token 2t), c1: (row g, token 2t+1), c2/c3: row g + 8.
            if (conv) {
                float inv = 1.0f;
                if (partials_in) {
                    float total = 0.0f;
#pragma unroll
                    for (int q = 0; q < 16; ++q) total += square_parts[q * PARTIAL_STRIDE + conv_token];
                    inv = rsqrtf(total / (float)a.norm_k + a.eps);
                }
                auto value = [&](int r) {
                    const float v = mine[(((r & 7) * 4 + (conv_token >> 1)) * 4) + (r >> 3) * 2 + (conv_token & 1)] * inv;
                    return __bfloat162float(__float2bfloat16_rn(v));
                };
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int j = i == 0 ? lane >> 3 : 4;
                    const int ch = tile * CONV_CHANNELS + j;
                    if (conv_slot < 0 || ch >= a.hidden || (i == 1 && lane >= 8)) continue;
                    const float u = value(j) * value(2 * CONV_CHANNELS + j);
                    float sum = 0.0f;
#pragma unroll
                    for (int k = 0; k < CONV_MAX_TAPS; ++k) {
                        if (k < a.conv_taps) sum = fmaf(conv_tap[i][k], k == a.conv_taps - 1 ? u : conv_window[i][k < CONV_MAX_TAPS - 1 ? k : 0], sum);
                    }
                    const float out = value(CONV_CHANNELS + j) * (sum + conv_b[i]);
                    const size_t at = (size_t)conv_token * a.hidden + ch;
                    if (a.out_f32) ((float*)a.y)[at] = out;
                    else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(out);
                    float* state_row = a.conv_state + conv_slot * a.conv_slot_stride + ch;
#pragma unroll
                    for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
                        if (k < a.conv_taps - 1)
                            state_row[(size_t)k * a.hidden] = k == a.conv_taps - 2 ? u : conv_window[i][k + 1 < CONV_MAX_TAPS - 1 ? k + 1 : 0];
                    }
                }
                continue;
            }
            if (res_in) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int token = t4 * 2 + e;
                    float squares = 0.0f;
                    if (token < T) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (rows[h] < 0) continue;
                            const size_t at = (size_t)token * N + rows[h];
                            const float v = early_res[e][h] + mine[lane * 4 + 2 * h + e] + early_bias[h];
                            a.res_out[at] = v;
                            a.x_out[at] = __float2bfloat16_rn(v * early_nw[h]);
                            squares += v * v;
                        }
                    }
                    squares += __shfl_xor_sync(0xffffffffu, squares, 4);
                    squares += __shfl_xor_sync(0xffffffffu, squares, 8);
                    squares += __shfl_xor_sync(0xffffffffu, squares, 16);
                    if (g == 0) a.partials_out[(size_t)tile * PARTIAL_STRIDE + token] = squares;
                }
                continue;
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int token = t4 * 2 + e;
                if (token >= T) continue;
                float lo = mine[lane * 4 + e], hi = mine[lane * 4 + 2 + e];
                if (partials_in) {
                    float total = 0.0f;
#pragma unroll
                    for (int q = 0; q < 16; ++q) total += square_parts[q * PARTIAL_STRIDE + token];
                    const float inv = rsqrtf(total / (float)a.norm_k + a.eps);
                    lo *= inv;
                    hi *= inv;
                }
                if (mode == MODE_GLU) {
                    if (rows[0] >= 0) {
                        const float v = lo / (1.0f + expf(-lo)) * hi;
                        const size_t at = (size_t)token * a.inter + rows[0];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                } else {
                    if (rows[0] >= 0) {
                        const float v = lo + early_bias[0];
                        const size_t at = (size_t)token * N + rows[0];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                    if (rows[1] >= 0) {
                        const float v = hi + early_bias[1];
                        const size_t at = (size_t)token * N + rows[1];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                }
            }
        }

        // this CTA's stores of product p are done (warp 0 made them all)
        if (warp == 0 && p + 1 < c.count) {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(c.arrived + p, 1u);
        }
    }
    pdl_trigger();
    if (timed_out && lane == 0 && status) atomicExch(status, 1);
}

constexpr int CHAIN_SMEM = CHAIN_STAGES * STAGE_BYTES + 2 * CHAIN_STAGES * 8 + (2 * CONSUMERS * 128 + 16 * PARTIAL_STRIDE) * 4 + 128;

// ---- the chain being collected (one per process: launches come from one thread, in order)
std::vector<StreamArgs> chain;
bool chain_open = false;
int chain_sm_count = 0;
unsigned* chain_counters = nullptr;  // arrived[CHAIN_MAX], passed[CHAIN_MAX]
long long chain_launches = 0, chain_products = 0;

int launch_chain(cudaStream_t stream) {
    if (chain.empty()) return SHISO_OK;
    if (chain.size() == 1) {
        const StreamArgs a = chain[0];
        chain.clear();
        chain_launches += 1;
        chain_products += 1;
        return shiso_stream_launch_one(a, chain_sm_count, stream);
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CHAIN_SMEM);
        if (e != cudaSuccess) return (int)e;
        int resident = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, gemm_stream_chain_kernel, THREADS, CHAIN_SMEM);
        if (e != cudaSuccess) return (int)e;
        if (resident < 1) return SHISO_ERR_UNSUPPORTED;
        if (cudaMalloc(&chain_counters, 2 * CHAIN_MAX * sizeof(unsigned)) != cudaSuccess) return SHISO_ERR_UNSUPPORTED;
        if (cudaMemset(chain_counters, 0, 2 * CHAIN_MAX * sizeof(unsigned)) != cudaSuccess) return SHISO_ERR_UNSUPPORTED;
        configured = true;
    }
    ChainArgs c = {};
    c.count = (int)chain.size();
    int most_tiles = 0;
    long long before = 0;
    // every CTA must be resident for the barriers between products: at most one per SM
    int grid = chain_sm_count;
    for (int i = 0; i < c.count; ++i) most_tiles = chain[i].tiles > most_tiles ? chain[i].tiles : most_tiles;
    if (most_tiles < grid) grid = most_tiles;
    for (int i = 0; i < c.count; ++i) {
        c.p[i] = chain[i];
        c.first_owner[i] = (int)(before % grid);
        before += chain[i].tiles;
    }
    c.arrived = chain_counters;
    c.passed = chain_counters + CHAIN_MAX;
    chain_launches += 1;
    chain_products += c.count;
    chain.clear();
    launch_kernel(gemm_stream_chain_kernel, grid, THREADS, CHAIN_SMEM, stream, c);
    return launch_status();
}

}  // namespace

bool shiso_chain_collect(const StreamArgs& a, cudaStream_t stream) {
    if (!chain_open) return false;
    if ((int)chain.size() == CHAIN_MAX) launch_chain(stream);  // a status other than 0 shows at the next flush
    chain.push_back(a);
    return true;
}

// From now on the weight-streaming products (shiso_gemm_stream*) are collected instead of
// launched; shiso_chain_flush launches what was collected as one kernel (one product: as the
// kernel of its own).  The caller flushes before it launches anything that reads a product's
// output, and closes the chain at the end of the step.
SHISO_API int shiso_chain_begin(int sm_count) {
    if (sm_count <= 0) return SHISO_ERR_SHAPE;
    chain.clear();
    chain_open = true;
    chain_sm_count = sm_count;
    return SHISO_OK;
}

SHISO_API int shiso_chain_flush(cudaStream_t stream) { return launch_chain(stream); }

SHISO_API int shiso_chain_end(cudaStream_t stream) {
    const int status = launch_chain(stream);
    chain_open = false;
    return status;
}

// Drops what was collected and closes the chain (a step that failed on the host).
SHISO_API int shiso_chain_abort() {
    chain.clear();
    chain_open = false;
    return SHISO_OK;
}

// Kernels launched for collected products since the library was loaded.
SHISO_API int shiso_chain_launches() { return (int)(chain_launches & 0x7fffffff); }

// How many products are waiting to be launched (0 when no chain is open).
SHISO_API int shiso_chain_pending() { return chain_open ? (int)chain.size() : 0; }

// After a wait ran out the counters of the barriers between products may be left standing: they
// are set back here (the host calls this when it has read a status word that is not zero).
SHISO_API int shiso_chain_reset() {
    if (chain_counters && cudaMemset(chain_counters, 0, 2 * CHAIN_MAX * sizeof(unsigned)) != cudaSuccess) return SHISO_ERR_UNSUPPORTED;
    return SHISO_OK;
}
