// What the weight-streaming products share: sizes of a stage, the argument block of one product,
// loads that are safe behind a predecessor's stores, and the mapping from a tile's rows to rows of
// the matrix.  gemm_stream.cu launches one product per kernel; gemm_stream_chain.cu runs a list of
// them in one persistent kernel.
#pragma once

#include "tcgen05.cuh"

namespace stream {


using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;

constexpr int KC = 1024;                       // columns per stage
constexpr int ROWS = 16;                       // weight rows per tile
constexpr int ROW_BYTES = KC * 2 + 16;         // padded row of a stage
constexpr int STAGE_BYTES = ROWS * ROW_BYTES;  // 33,024
constexpr int STAGES = 3;                      // two CTAs (this kernel's and its successor's) must fit an SM
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


}  // namespace stream

// A list of products that is being collected instead of launched (gemm_stream_chain.cu).
// `shiso_chain_collect` takes a product whose arguments are complete and returns true when a chain
// is open: the caller then launches nothing.
bool shiso_chain_collect(const stream::StreamArgs& a, cudaStream_t stream);
// One product as a kernel of its own (gemm_stream.cu).
int shiso_stream_launch_one(const stream::StreamArgs& a, int sm_count, cudaStream_t stream);
