// Y[T, N] = X[T, K] * W[N, K]^T for up to 8 rows, bfloat16: the decode step's matrix products as
// a persistent weight-streaming kernel.
//
// At these sizes a product is over in a few microseconds and is bound by reading W once, so what
// counts is that the weight bytes are in flight from the kernel's first cycle to its last.  (The
// first version gave a CTA 16 weight rows and let it ask for all of them at once; a matrix of
// more than two such CTAs per SM then runs in waves, and every wave pays the memory latency
// again.)  One CTA per SM walks its share of the 16-row tiles.  A producer warp - lane r copies
// weight row r - keeps a ring of four shared-memory stages full with bulk copies
// (cp.async.bulk, 1,024 columns of a row each, completion counted on an mbarrier), up to 129 KB
// ahead of the consumers and independent of them; it starts before the predecessor in the
// dependent-launch chain has finished, as soon as that kernel's CTA has left the SM.  (Three
// stages let the successor's CTA move in beside this one and start its own stream under this
// one's tail; the deeper ring is worth more: 26.4 against 28.4 us for the four products of a
// layer, and five or six stages are no better than four, 27.0 and 26.9 us.  Memory answers a
// request in about 2 us when it is this busy, so 6.5 TB/s want some 13 MB on their way, and
// three stages on 148 SMs are 14.6 MB only while every stage is being filled.  Three stages
// of 2,048 columns - whole rows of a 2048-wide matrix in one copy - took 29.0 us.)
// Four consumer warps split a chunk's columns (256 each), read their 16-byte
// pieces of the two weight rows a lane owns from shared memory (rows are padded by 16 bytes,
// which spreads them over the banks) and feed mma.sync m16n8k16: weights are the M operand, tokens
// the N operand; a lane's 8 consecutive k values feed two MMAs as (k0..k3 | k4..k7) and the
// activation fragment, kept in registers, is loaded with the same permutation, so the sum over k
// is the same set of products.  A tile's partial sums meet in shared memory in warp order; warp 0
// writes the result while the others go on.
//
// What follows the product is folded into the epilogue, because at these sizes every extra kernel
// costs more than its arithmetic:
//   GLU     the weight is a [2 * inter, K] gate-over-up pair; a tile is 8 gate rows and their 8 up
//           rows, and the epilogue writes silu(gate) * up (kernels/cuda/generic/glu.cuh:35-57);
//   STREAM  (a block's output projection) the tile's 16 features are added to the float32 residual
//           stream (into a second buffer), written once more times the next RMS norm's weight as
//           bfloat16 rows - the next product's input but for the row scale - and the sum of their
//           squares per token goes to a table of partials, one row per tile;
//   SCALED  (the product after it) sums the partials of each token in a fixed order and scales
//           its accumulators by rsqrt(mean square + eps) before the activation or the store:
//           x W^T is linear in the row scale, so the norm needs no pass of its own.  The rows are
//           rounded to bfloat16 before the scale instead of after it, which is the same relative
//           rounding.
// What the STREAM and SCALED epilogues read from global memory is asked for at the start of a
// tile, not when it is needed: the epilogue is the tail of a chain of dependent kernels.
// (Measured and left out: filling a stage with four TMA boxes of 256 columns x 16 rows instead of
// sixteen row copies.  The boxes are asked for faster - a copy costs its issuing lane some 35 ns
// whatever its size - but their 512-byte row pieces use memory less well than 2 KB pieces of a
// row: 30.0 against 26.7 us for the four products of a layer in a captured chain.)
// (Asking, from inside this kernel, for the matrix the step reads next to be brought into L2 was
// measured too - cp.async.bulk.prefetch.L2 over a slice per CTA - and made the whole step slower:
// the stream already keeps memory busy, and the extra requests only delay its own rows.  Asked
// for only by the producer warp after its own last copy, and only for the first 4 to 48 MB of the
// matrix that comes next, it is no better: 29.3 us for the four products of a layer without,
// 29.3 / 29.4 / 30.1 / 30.9 / 36.6 us with 4 / 8 / 16 / 24 / 48 MB.)
// (Where a product's time goes, from %globaltimer stamps in a captured chain at 8 rows: a
// successor's producer starts about 1 us before its predecessor's last CTA ends; its consumers
// leave the dependency wait 0.5 to 0.8 us after that end; the activations they then ask for
// arrive 1.0 to 1.3 us later, behind the 14 MB of weights the rings keep in flight; from the
// first product to the last the stream runs at 4.9 to 5.4 TB/s; the epilogue of the last tile
// takes 0.5 us.  Launching the successor at the predecessor's first cycle instead of after its
// last copy moves none of these: 29.9 us a layer either way.)
// (Built, measured and left out: all products between two attention kernels as ONE persistent
// kernel - the producer warps walk the whole list of products without a stop, the consumers of
// all CTAs meet at a counter in global memory between two products, six stages of 33 KB or
// three of 66 KB a CTA.  Results were those of the separate kernels, the time was not: 35.7 us
// for the four products of a layer against 29.4 us as four dependent launches.  A barrier
// between two products is three round trips to L2 in a row (count, flag, the new activations),
// and behind a ring that keeps 190 KB a CTA on their way every one of them waits in the same
// queues as the stream: 3 us a product with all arithmetic taken out.  At a kernel boundary
// the predecessor's stream has drained and the same trips are short.  On the way a kernel that
// only streams showed what the copies themselves can reach on this part: sixteen 2 KB half
// rows a stage, as here, 5.0 TB/s; sixteen whole 4 KB rows 6.7 TB/s; thirty-two 1 KB pieces
// 4.0 TB/s; one lane issuing all sixteen copies 1.1 TB/s.)
//
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the kernel
// carries on (its result is then wrong, and the host raises when it reads the word).
#include "tcgen05.cuh"

namespace {

using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;

constexpr int KC = 1024;                       // columns per stage
constexpr int ROWS = 16;                       // weight rows per tile
constexpr int ROW_BYTES = KC * 2 + 16;         // padded row of a stage
constexpr int STAGE_BYTES = ROWS * ROW_BYTES;  // 33,024
constexpr int STAGES = 4;                      // measured: 3 (two CTAs fit an SM), 5 and 6 are slower
constexpr int CONSUMERS = 4;                   // warps; each takes 256 columns of a chunk
constexpr int KB = KC / CONSUMERS / 64;        // 64-wide k blocks per warp and chunk
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int PARTIAL_STRIDE = 16;             // tokens per row of the partials table
constexpr int EARLY_PARTIALS = 8;

enum { MODE_PLAIN = 0, MODE_GLU = 1, MODE_CONV = 2 };
constexpr int CONV_CHANNELS = 5;  // channels of a CONV tile: their B, C and x rows are 15 of its 16 rows
constexpr int CONV_MAX_TAPS = 4;

struct StreamArgs {
    const __nv_bfloat16* x;  // [T, K]
    const __nv_bfloat16* w;  // [N, K]
    const float* bias;       // [N] or null (plain products only)
    void* y;                 // plain [T, N]; GLU [T, inter]
    int T, N, K, inter, out_f32, mode;
    int tiles;               // 16-row tiles (GLU: 8 gate + 8 up rows)
    int* status;
    // STREAM epilogue
    const float* res_in;
    float* res_out;
    const float* next_norm_w;
    __nv_bfloat16* x_out;
    float* partials_out;     // [tiles, PARTIAL_STRIDE]
    // SCALED epilogue
    const float* partials_in;
    int partial_count, norm_k;
    float eps;
    // CONV epilogue: w is a short convolution's input projection [3 * hidden, K] (rows B, C, x) and
    // every sequence brings one row; y[t, ch] = C * (sum_j conv_w[ch][j] * window_j + conv_bias[ch])
    // where the window is the sequence's last taps - 1 gated inputs B * x followed by this row's,
    // and the state moves on by one row.  B, C and x are rounded to bfloat16 first, as a product
    // that stores them would.
    const float* conv_w;        // [hidden, conv_taps]
    const float* conv_bias;     // [hidden] or null
    float* conv_state;          // [slots][conv_taps - 1][hidden], conv_slot_stride floats between slots
    long long conv_slot_stride;
    const int* conv_seq_of_token;  // [T]
    const int* conv_slots;         // [sequences]
    int conv_taps, hidden;
};

__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Activations were written by a predecessor grid: coherent loads, after the dependency wait.
__device__ __forceinline__ uint4 load_activation16(const __nv_bfloat16* p, bool valid) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) {
        asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    }
    return v;
}

__device__ __forceinline__ float load_stream1(const float* p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void consumer_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
}

// Row of W behind row r (0..15) of a tile, or -1.
template <bool CONV>
__device__ __forceinline__ int tile_row(const StreamArgs& a, int tile, int r) {
    if constexpr (CONV) {
        const int ch = tile * CONV_CHANNELS + r % CONV_CHANNELS;
        return (r < 3 * CONV_CHANNELS && ch < a.hidden) ? (r / CONV_CHANNELS) * a.hidden + ch : -1;
    }
    if (a.mode == MODE_GLU) {
        const int f = tile * 8 + (r & 7);
        return f < a.inter ? (r < 8 ? f : a.inter + f) : -1;
    }
    const int row = tile * ROWS + r;
    return row < a.N ? row : -1;
}

// HELD: the chunks of K whose activations a lane keeps in registers for the whole kernel (K <= HELD *
// KC); they are the same for every tile, and a reload per chunk would put an L2 round trip into
// every stage.  HELD = 0: K is longer than that and the activations of the next chunk are fetched
// while the current one is worked on.
constexpr int MAX_ROWS = 8;  // rows of x the built variants take (NT = 1)

// CONV: the kernel with the short convolution's epilogue; a variant of its own, because what that
// epilogue holds across a tile's products (state, taps, bias) would cost the other modes their
// registers (measured when it was a run-time mode: 0.667 -> 0.735 ms per decode step).
template <int NT, int HELD, bool CONV>
__global__ void __launch_bounds__(THREADS, NT * HELD > 2 ? 1 : 2)
gemm_stream_kernel(StreamArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    uint64_t* full = (uint64_t*)(ring + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    float* partial = (float*)(empty + STAGES);                      // [2][CONSUMERS][NT][32][4]
    float* square_parts = partial + 2 * CONSUMERS * NT * 128;       // [16][PARTIAL_STRIDE]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = (a.K + KC - 1) / KC;
    bool timed_out = false;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CONSUMERS) {
        // ---- producer: weights depend on no predecessor, so nothing here waits for one.  Lane r
        // copies row r of each stage: one thread issuing all sixteen copies took longer per stage
        // than the memory system needs to deliver it.
        int unit = 0;
        for (int tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
            const int row = lane < ROWS ? tile_row<CONV>(a, tile, lane) : -1;
            const int present = __popc(__ballot_sync(0xffffffffu, row >= 0));
            const __nv_bfloat16* src = a.w + (size_t)(row >= 0 ? row : 0) * a.K;
            for (int c = 0; c < chunks; ++c, ++unit) {
                const int s = unit % STAGES;
                if (unit >= STAGES && !mbar_wait(&empty[s], ((unit / STAGES) - 1) & 1)) timed_out = true;
                const int cols = min(KC, a.K - c * KC);
                if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)(present * cols * 2));
                __syncwarp();
                if (row >= 0)
                    bulk_load(smem_u32(ring + s * STAGE_BYTES) + lane * ROW_BYTES, src + (size_t)c * KC, (uint32_t)(cols * 2), &full[s]);
            }
        }
        if (timed_out && lane == 0 && a.status) atomicExch(a.status, 1);
        pdl_trigger();
        return;
    }

    // ---- consumers
    const int g = lane >> 2, t4 = lane & 3;
    pdl_wait();

    // the activations of chunk c this warp needs: KB k blocks of 64, a lane 16 consecutive k of each
    auto load_x = [&](int c, uint4 (&xv)[KB][NT][2]) {
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            const int k = c * KC + warp * (KC / CONSUMERS) + kb * 64 + t4 * 16;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int token = n * 8 + g;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    xv[kb][n][h] = load_activation16(a.x + (size_t)token * a.K + k + h * 8, token < a.T && k + h * 8 < a.K);
            }
        }
    };

    // SCALED: the partial squares, asked for now and summed at the first epilogue.  Slot i of
    // 256 is (group i / 16, token i % 16); a group sums every 16th row of the table.
    constexpr int SLOTS = 16 * PARTIAL_STRIDE / (CONSUMERS * 32);
    float early_part[SLOTS][EARLY_PARTIALS];
    if (a.partials_in) {
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int i = threadIdx.x + q * CONSUMERS * 32;
            const int group = i / PARTIAL_STRIDE, token = i % PARTIAL_STRIDE;
#pragma unroll
            for (int j = 0; j < EARLY_PARTIALS; ++j) {
                const int c = group + 16 * j;
                early_part[q][j] = c < a.partial_count ? load_stream1(a.partials_in + (size_t)c * PARTIAL_STRIDE + token) : 0.0f;
            }
        }
    }

    // CONV: lane l of warp 0 finishes channel l / 8 of a tile for token l % 8, lanes 0..7 also the
    // fifth channel; the token's state slot is looked up once
    const int conv_token = lane & 7;
    long long conv_slot = -1;
    if (CONV && warp == 0 && conv_token < a.T)
        conv_slot = a.conv_slots[a.conv_seq_of_token[conv_token]];

    constexpr int SLOTS_X = HELD > 0 ? HELD : 2;  // rolling: the current chunk and the next
    uint4 xs[SLOTS_X][KB][NT][2];
    if (HELD > 0) {
#pragma unroll
        for (int c = 0; c < HELD; ++c) load_x(c, xs[c]);
    } else {
        load_x(0, xs[0]);
    }
    bool scale_ready = false;
    int unit = 0, local = 0;
    for (int tile = blockIdx.x; tile < a.tiles; tile += gridDim.x, ++local) {
        // STREAM: what the epilogue reads, asked for before the tile's products
        float early_res[NT][2][2], early_nw[2] = {0.0f, 0.0f}, early_bias[2] = {0.0f, 0.0f};
        int rows[2];
        rows[0] = tile_row<CONV>(a, tile, g);
        rows[1] = tile_row<CONV>(a, tile, g + 8);
        if (warp == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (rows[h] >= 0 && a.mode == MODE_PLAIN) {
                    if (a.bias) early_bias[h] = a.bias[rows[h]];
                    if (a.res_in) early_nw[h] = a.next_norm_w[rows[h]];
                }
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int token = n * 8 + t4 * 2 + e;
                        early_res[n][e][h] = 0.0f;
                        if (a.res_in && rows[h] >= 0 && token < a.T) early_res[n][e][h] = load_stream1(a.res_in + (size_t)token * a.N + rows[h]);
                    }
            }
        }

        // CONV: the state, the taps and the bias of this lane's one or two (channel, token) pairs
        float conv_window[2][CONV_MAX_TAPS - 1], conv_tap[2][CONV_MAX_TAPS], conv_b[2] = {0.0f, 0.0f};
        if (CONV && warp == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int ch = tile * CONV_CHANNELS + (i == 0 ? lane >> 3 : 4);
                const bool on = conv_slot >= 0 && ch < a.hidden && (i == 0 || lane < 8);
#pragma unroll
                for (int j = 0; j < CONV_MAX_TAPS; ++j) {
                    conv_tap[i][j] = (on && j < a.conv_taps) ? a.conv_w[(size_t)ch * a.conv_taps + j] : 0.0f;
                    if (j < CONV_MAX_TAPS - 1)
                        conv_window[i][j] = (on && j < a.conv_taps - 1)
                            ? load_stream1(a.conv_state + conv_slot * a.conv_slot_stride + (size_t)j * a.hidden + ch) : 0.0f;
                }
                if (on && a.conv_bias) conv_b[i] = a.conv_bias[ch];
            }
        }

        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;

        // one stage: wait for it, multiply this warp's columns, give it back
        auto work = [&](int c, uint4 (&xv)[KB][NT][2]) {
            const int s = unit % STAGES;
            if (!mbar_wait(&full[s], (unit / STAGES) & 1)) timed_out = true;
            const uint32_t base = smem_u32(ring + s * STAGE_BYTES);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const int col = warp * (KC / CONSUMERS) + kb * 64 + t4 * 16;  // within the chunk
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint4 wl = make_uint4(0u, 0u, 0u, 0u), wh = wl;
                    if (c * KC + col + h * 8 < a.K) {  // past K the stage holds what an earlier chunk left
                        wl = lds16(base + g * ROW_BYTES + (col + h * 8) * 2);
                        wh = lds16(base + (g + 8) * ROW_BYTES + (col + h * 8) * 2);
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        mma_bf16(acc[n], wl.x, wh.x, wl.y, wh.y, xv[kb][n][h].x, xv[kb][n][h].y);
                        mma_bf16(acc[n], wl.z, wh.z, wl.w, wh.w, xv[kb][n][h].z, xv[kb][n][h].w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            ++unit;
        };
        if constexpr (HELD > 0) {
#pragma unroll
            for (int c = 0; c < HELD; ++c) work(c, xs[c]);
        } else {
            for (int c = 0; c < chunks; ++c) {
                // the next unit's activations travel while this one is worked on
                const int next_c = c + 1 < chunks ? c + 1 : 0;
                const bool more = c + 1 < chunks || tile + (int)gridDim.x < a.tiles;
                if (more) load_x(next_c, xs[1]);
                work(c, xs[0]);
                if (more) {
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int h = 0; h < 2; ++h) xs[0][kb][n][h] = xs[1][kb][n][h];
                }
            }
        }

        // ---- the tile's partial sums meet in shared memory, in warp order
        float* mine = partial + (size_t)(local & 1) * CONSUMERS * NT * 128;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) mine[((warp * NT + n) * 32 + lane) * 4 + e] = acc[n][e];
        if (!scale_ready && a.partials_in) {
#pragma unroll
            for (int q = 0; q < SLOTS; ++q) {
                const int i = threadIdx.x + q * CONSUMERS * 32;
                const int group = i / PARTIAL_STRIDE, token = i % PARTIAL_STRIDE;
                float sum = 0.0f;
#pragma unroll
                for (int j = 0; j < EARLY_PARTIALS; ++j) sum += early_part[q][j];
                for (int c = group + 16 * EARLY_PARTIALS; c < a.partial_count; c += 16)
                    sum += load_stream1(a.partials_in + (size_t)c * PARTIAL_STRIDE + token);
                square_parts[group * PARTIAL_STRIDE + token] = sum;
            }
            scale_ready = true;
        }
        consumer_barrier();
        for (int i = threadIdx.x; i < NT * 128; i += CONSUMERS * 32) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < CONSUMERS; ++w) sum += mine[w * NT * 128 + i];
            mine[i] = sum;  // only this thread touches this element
        }
        consumer_barrier();
        if (warp != 0) continue;

        // ---- epilogue (warp 0).  In a lane: c0: (row g, token 2t), c1: (row g, token 2t+1), c2/c3: row g + 8.
        if constexpr (CONV) {
            if constexpr (NT == 1) {
                float inv = 1.0f;
                if (a.partials_in) {
                    float total = 0.0f;
#pragma unroll
                    for (int c = 0; c < 16; ++c) total += square_parts[c * PARTIAL_STRIDE + conv_token];
                    inv = rsqrtf(total / (float)a.norm_k + a.eps);
                }
                // the tile's value of (row r, this lane's token), rounded as a stored product would be
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
            }
            continue;
        }
        if (a.res_in) {
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int token = n * 8 + t4 * 2 + e;
                    float squares = 0.0f;
                    if (token < a.T) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (rows[h] < 0) continue;
                            const size_t at = (size_t)token * a.N + rows[h];
                            const float v = early_res[n][e][h] + mine[(n * 32 + lane) * 4 + 2 * h + e] + early_bias[h];
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
            }
            continue;
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int token = n * 8 + t4 * 2 + e;
                if (token >= a.T) continue;
                float lo = mine[(n * 32 + lane) * 4 + e], hi = mine[(n * 32 + lane) * 4 + 2 + e];
                if (a.partials_in) {
                    float total = 0.0f;
#pragma unroll
                    for (int c = 0; c < 16; ++c) total += square_parts[c * PARTIAL_STRIDE + token];
                    const float inv = rsqrtf(total / (float)a.norm_k + a.eps);
                    lo *= inv;
                    hi *= inv;
                }
                if (a.mode == MODE_GLU) {
                    if (rows[0] >= 0) {
                        const float v = silu_times(lo, hi);
                        const size_t at = (size_t)token * a.inter + rows[0];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                } else {
                    if (rows[0] >= 0) {
                        const float v = lo + early_bias[0];
                        const size_t at = (size_t)token * a.N + rows[0];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                    if (rows[1] >= 0) {
                        const float v = hi + early_bias[1];
                        const size_t at = (size_t)token * a.N + rows[1];
                        if (a.out_f32) ((float*)a.y)[at] = v;
                        else ((__nv_bfloat16*)a.y)[at] = __float2bfloat16_rn(v);
                    }
                }
            }
        }
    }
    pdl_trigger();
    if (timed_out && lane == 0 && a.status) atomicExch(a.status, 1);
}

template <int NT, int HELD, bool CONV>
int launch_as(const StreamArgs& a, int sm_count, cudaStream_t stream) {
    constexpr int SMEM = STAGES * STAGE_BYTES + 2 * STAGES * 8 + (2 * CONSUMERS * NT * 128 + 16 * PARTIAL_STRIDE) * 4 + 128;
    auto kernel = gemm_stream_kernel<NT, HELD, CONV>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int grid = a.tiles < sm_count ? a.tiles : sm_count;
    launch_kernel(kernel, grid, THREADS, SMEM, stream, a);
    return launch_status();
}

int launch_stream(StreamArgs& a, int sm_count, cudaStream_t stream) {
    a.tiles = a.mode == MODE_GLU ? (a.inter + 7) / 8 : a.mode == MODE_CONV ? (a.hidden + CONV_CHANNELS - 1) / CONV_CHANNELS : (a.N + ROWS - 1) / ROWS;
    a.status = shiso_tc_status_word();
    const int chunks = (a.K + KC - 1) / KC;
    // NT = 1: one 8-token tile per weight fragment.  With two (9..16 rows) the held activations
    // took the registers of a second CTA per SM, and a decode step at batch 16 ran at 17.9k
    // tokens/s against 19.8k with the tensor-memory kernel and separate norm kernels; reading
    // the activations from L2 every stage instead fell to 11.5k.  Those rows are not built.
    if (a.mode == MODE_CONV) {
        if (chunks == 1) return launch_as<1, 1, true>(a, sm_count, stream);
        if (chunks == 2) return launch_as<1, 2, true>(a, sm_count, stream);
        return launch_as<1, 0, true>(a, sm_count, stream);
    }
    if (chunks == 1) return launch_as<1, 1, false>(a, sm_count, stream);
    if (chunks == 2) return launch_as<1, 2, false>(a, sm_count, stream);
    return launch_as<1, 0, false>(a, sm_count, stream);
}

}  // namespace

// x [T, K] bf16 (T <= 8), w [N, K] bf16, K a multiple of 8, pointers 16-byte aligned.
// inter == 0: y[T, N] = x w^T (+ bias).  inter > 0: N == 2 * inter, y[T, inter] = silu(x gate^T) * (x up^T).
// In the GLU layout a tile's row r < 8 is gate row 8 * tile + r and row r >= 8 its up row.
SHISO_API int shiso_gemm_stream(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T, int N,
                                int K, int inter, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (T > MAX_ROWS || K % 8 != 0 || K <= 0 || sm_count <= 0) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return SHISO_ERR_ALIGN;
    if (inter > 0 && (N != 2 * inter || bias)) return SHISO_ERR_SHAPE;
    StreamArgs a = {};
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
    return launch_stream(a, sm_count, stream);
}

// A block's output projection into the residual stream: res_out = res_in + x w^T (+ bias),
// x_out = bf16(res_out * next_norm_w), partials_out[tile][token] = sum over the tile's 16 features
// of res_out^2 (ceil(N / 16) rows of 16 floats).
SHISO_API int shiso_gemm_stream_into(const void* x, const void* w, const float* bias, const float* res_in,
                                     float* res_out, const float* next_norm_w, void* x_out, float* partials_out,
                                     int T, int N, int K, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (T > MAX_ROWS || K % 8 != 0 || K <= 0 || sm_count <= 0) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return SHISO_ERR_ALIGN;
    if (!res_in || !res_out || res_in == res_out || !next_norm_w || !x_out || !partials_out) return SHISO_ERR_SHAPE;
    StreamArgs a = {};
    a.x = (const __nv_bfloat16*)x;
    a.w = (const __nv_bfloat16*)w;
    a.bias = bias;
    a.T = T;
    a.N = N;
    a.K = K;
    a.mode = MODE_PLAIN;
    a.res_in = res_in;
    a.res_out = res_out;
    a.next_norm_w = next_norm_w;
    a.x_out = (__nv_bfloat16*)x_out;
    a.partials_out = partials_out;
    return launch_stream(a, sm_count, stream);
}

// The product after it: y = (x w^T) * rsqrt(sum_c partials[c][token] / K + eps) per token (then
// SwiGLU when inter > 0).
SHISO_API int shiso_gemm_stream_scaled(const void* x, const float* partials, int partial_count, float eps,
                                       const void* w, void* y, int y_dtype, int T, int N, int K, int inter,
                                       int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (T > MAX_ROWS || K % 8 != 0 || K <= 0 || !partials || partial_count <= 0 || sm_count <= 0) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return SHISO_ERR_ALIGN;
    if (inter > 0 && N != 2 * inter) return SHISO_ERR_SHAPE;
    StreamArgs a = {};
    a.x = (const __nv_bfloat16*)x;
    a.w = (const __nv_bfloat16*)w;
    a.y = y;
    a.T = T;
    a.N = N;
    a.K = K;
    a.inter = inter;
    a.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    a.mode = inter > 0 ? MODE_GLU : MODE_PLAIN;
    a.partials_in = partials;
    a.partial_count = partial_count;
    a.norm_k = K;
    a.eps = eps;
    return launch_stream(a, sm_count, stream);
}

// A short convolution's input projection and the gated convolution behind it in one launch, for
// steps in which every sequence brings one row (T <= 8 rows): w [3 * hidden, K] bf16 (rows B, C,
// x), conv_w [hidden, taps] (2..4 taps), state [slots][taps - 1][hidden] float with slot_stride
// floats between slots, slots[seq_of_token[t]] the slot of row t; y [T, hidden].  With `partials`
// the rows of x lack their RMS scale, as in shiso_gemm_stream_scaled; null: x is taken as it is.
SHISO_API int shiso_gemm_stream_conv(const void* x, const float* partials, int partial_count, float eps, const void* w,
                                     const float* conv_w, const float* conv_bias, float* state, long long slot_stride,
                                     const int* seq_of_token, const int* slots, void* y, int y_dtype, int T, int hidden,
                                     int K, int taps, int sm_count, cudaStream_t stream) {
    if (T <= 0 || hidden <= 0) return SHISO_OK;
    if (T > MAX_ROWS || K % 8 != 0 || K <= 0 || sm_count <= 0 || taps < 2 || taps > CONV_MAX_TAPS) return SHISO_ERR_UNSUPPORTED;
    if (partials && partial_count <= 0) return SHISO_ERR_SHAPE;
    if (!conv_w || !state || !seq_of_token || !slots) return SHISO_ERR_SHAPE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return SHISO_ERR_ALIGN;
    StreamArgs a = {};
    a.x = (const __nv_bfloat16*)x;
    a.w = (const __nv_bfloat16*)w;
    a.y = y;
    a.T = T;
    a.N = 3 * hidden;
    a.K = K;
    a.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    a.mode = MODE_CONV;
    a.partials_in = partials;
    a.partial_count = partial_count;
    a.norm_k = K;
    a.eps = eps;
    a.conv_w = conv_w;
    a.conv_bias = conv_bias;
    a.conv_state = state;
    a.conv_slot_stride = slot_stride;
    a.conv_seq_of_token = seq_of_token;
    a.conv_slots = slots;
    a.conv_taps = taps;
    a.hidden = hidden;
    return launch_stream(a, sm_count, stream);
}
