// Paged GQA attention for steps that hold prompt portions (bfloat16): a tiled, online-softmax
// kernel on the tensor cores.
//
// One CTA owns 64 consecutive query rows of one sequence and up to four query heads of one KV
// group (HG of them): four warps per head, 16 rows per warp.  The heads of a group read the
// same keys and values, so a tile brought to shared memory serves all of them.  Key and value tiles of 64 positions are gathered from the paged cache
// through the block table into shared memory with cp.async (two stages), scores are
// Q K^T with mma.sync m16n8k16 (bfloat16 in, float out), the softmax statistics are kept in
// float per row, and P V accumulates in float registers.  A row at position p sees keys
// max(0, p + 1 - window) .. p; rows of a portion see the portion's own keys because the
// store kernel runs first (crates/shiso-engine/src/dense/attn.rs:28-33).  The reference's
// CUDA prefill kernel is scalar (16 x 16 tiles, kernels/cuda/dense/dense_attn.cuh:208-355);
// its tensor-core twin exists for Metal only (kernels/metal/dense/dense_attn.metal:356-536).
//
// Query tiles never cross a sequence: CTA x is mapped to (sequence, tile) by walking the
// step's q_start array.  Positions outside a row's range are masked to -inf; key and value
// rows outside the tile's range are zero-filled, never read (a window group's table has
// holes there).
//
// Long portions of head size 64 take the tensor-memory kernel of attention_prefill_tc.cu; this
// one, with the softmax between its two products in registers, takes every other head size
// (multiples of 16 up to 128), short portions, and steps that mix a few prompt rows with decode rows.
#include "common.cuh"

namespace {

constexpr int BM = 64;   // query rows per CTA
constexpr int BN = 64;   // keys per tile

struct PrefillArgs {
    const __nv_bfloat16* q;        // [T, heads * D]
    const __nv_bfloat16* k_cache;  // [pages, page, kv_heads, D]
    const __nv_bfloat16* v_cache;
    const int* block_table;        // [S, width]
    const int* q_start;            // [S + 1]
    const int* start_pos;          // [S]
    __nv_bfloat16* out;            // [T, heads * D]
    int width, num_seqs, heads, kv_heads, page_size, window;
    float scale_log2;              // scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int HG>
__global__ void __launch_bounds__(HG * 128)
flash_prefill_kernel(PrefillArgs a) {
    constexpr int THREADS = HG * 128;
    pdl_wait();
    constexpr int ROW_BYTES = D * 2 + 16;  // 16 bytes of padding: ldmatrix rows fall on distinct banks
    constexpr int CHUNKS = D / 8;          // 16-byte pieces per row
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;

    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* q_s = smem;                               // [HG][BM][ROW_BYTES]
    uint8_t* k_s = q_s + HG * BM * ROW_BYTES;          // [2][BN][ROW_BYTES]
    uint8_t* v_s = k_s + 2 * BN * ROW_BYTES;           // [2][BN][ROW_BYTES]
    __shared__ int tile_seq, tile_row0;

    // ---- which (sequence, tile) is this CTA?
    if (threadIdx.x == 0) {
        // the last tiles of a portion have the most keys: they take the first CTAs of every head
        // chunk (the grid's fast index), so that the grid's tail is made of short ones
        int left = gridDim.y - 1 - blockIdx.y, found = -1, row0 = 0;
        for (int s = 0; s < a.num_seqs; ++s) {
            const int tiles = (a.q_start[s + 1] - a.q_start[s] + BM - 1) / BM;
            if (left < tiles) {
                found = s;
                row0 = left * BM;
                break;
            }
            left -= tiles;
        }
        tile_seq = found;
        tile_row0 = row0;
    }
    __syncthreads();
    const int seq = tile_seq;
    if (seq < 0) return;
    const int row0 = tile_row0;
    const int first_token = a.q_start[seq] + row0;
    const int rows = min(BM, a.q_start[seq + 1] - first_token);
    const int first_pos = a.start_pos[seq] + row0;
    const int last_pos = first_pos + rows - 1;
    const int group = a.heads / a.kv_heads;
    const int chunks = (group + HG - 1) / HG;          // head chunks per KV head
    const int kv_head = blockIdx.x / chunks;
    const int head0 = kv_head * group + (blockIdx.x % chunks) * HG;
    const int heads_here = min(HG, kv_head * group + group - head0);
    const int* table = a.block_table + (size_t)seq * a.width;
    const int key_lo = a.window > 0 ? max(0, first_pos + 1 - a.window) : 0;  // the smallest key any row sees
    const int tile_first = key_lo / BN, tile_last = last_pos / BN;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int head_sel = warp >> 2;            // which of the CTA's heads this warp serves
    const int row_block = (warp & 3) * 16;     // its 16 query rows inside the tile
    const int head = head0 + head_sel;
    const bool active = head_sel < heads_here;  // warp-uniform

    // ---- Q tiles -> shared (rows past the portion, and heads past the group, are zero)
    for (int c = tid; c < HG * BM * CHUNKS; c += THREADS) {
        const int hr = c / CHUNKS, ch = c % CHUNKS;
        const int hs = hr / BM, r = hr % BM;
        const bool valid = r < rows && hs < heads_here;
        const __nv_bfloat16* src = a.q + ((size_t)(first_token + min(r, rows - 1)) * a.heads + head0 + min(hs, heads_here - 1)) * D + ch * 8;
        cp_async16(q_s + hr * ROW_BYTES + ch * 16, src, valid);
    }
    auto load_kv = [&](int tile, int stage) {
        uint8_t* kd = k_s + stage * BN * ROW_BYTES;
        uint8_t* vd = v_s + stage * BN * ROW_BYTES;
        for (int c = tid; c < BN * CHUNKS; c += THREADS) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const int key = tile * BN + r;
            const bool valid = key >= key_lo && key <= last_pos;
            size_t row = 0;
            if (valid) row = (size_t)table[key / a.page_size] * a.page_size + key % a.page_size;
            const size_t at = (row * a.kv_heads + kv_head) * D + ch * 8;
            cp_async16(kd + r * ROW_BYTES + ch * 16, a.k_cache + at, valid);
            cp_async16(vd + r * ROW_BYTES + ch * 16, a.v_cache + at, valid);
        }
    };
    load_kv(tile_first, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    float o_acc[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[KSTEPS][4];
    const int my_pos[2] = {first_pos + row_block + g, first_pos + row_block + g + 8};

    for (int tile = tile_first; tile <= tile_last; ++tile) {
        const int stage = (tile - tile_first) & 1;
        if (tile < tile_last) load_kv(tile + 1, stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        if (tile == tile_first) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                const int r = head_sel * BM + row_block + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = kk * 16 + (lane >> 4) * 8;
                ldmatrix_x4(smem_addr(q_s + r * ROW_BYTES + col * 2), q_frag[kk][0], q_frag[kk][1], q_frag[kk][2], q_frag[kk][3]);
            }
        }
        const uint8_t* kt = k_s + stage * BN * ROW_BYTES;
        const uint8_t* vt = v_s + stage * BN * ROW_BYTES;

        // a warp whose rows all lie before this tile's first key, or whose windows all start after
        // its last, has nothing to add: every score would be masked
        const bool warp_has_keys = active && tile * BN <= first_pos + row_block + 15 &&
                                   (a.window <= 0 || tile * BN + BN - 1 > first_pos + row_block - a.window);
        if (warp_has_keys) {
        // ---- S = Q K^T for this warp's 16 rows x 64 keys
        float s_acc[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
            for (int j = 0; j < BN / 8; j += 2) {
                const int r = j * 8 + (lane & 7) + (lane >> 4) * 8;
                const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_addr(kt + r * ROW_BYTES + col * 2), b0, b1, b2, b3);
                mma_bf16(s_acc[j], q_frag[kk], b0, b1);
                mma_bf16(s_acc[j + 1], q_frag[kk], b2, b3);
            }
        }

        // ---- mask, online softmax (base 2)
        const int key0 = tile * BN;
        float tile_max[2] = {-INFINITY, -INFINITY};
        // every key of the tile is seen by every row of this warp: no mask to evaluate
        const bool all_seen = key0 + BN - 1 <= first_pos + row_block &&
                              (a.window <= 0 || key0 > first_pos + row_block + 15 - a.window);
        if (all_seen) {
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = s_acc[j][e] * a.scale_log2;
                    s_acc[j][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                    const int pos = my_pos[e >> 1];
                    const bool seen = key <= pos && (a.window <= 0 || key > pos - a.window);
                    const float v = seen ? s_acc[j][e] * a.scale_log2 : -INFINITY;
                    s_acc[j][e] = v;
                    tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                }
            }
        }
        float correction[2], use_max[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float m = tile_max[r];
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
            const float new_max = fmaxf(row_max[r], m);
            use_max[r] = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen no key yet
            correction[r] = exp2f(row_max[r] - use_max[r]);
            row_max[r] = new_max;
        }
        float tile_sum[2] = {0.0f, 0.0f};
        uint32_t p_frag[BN / 16][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = exp2f(s_acc[j][e] - use_max[e >> 1]);
                tile_sum[e >> 1] += p[e];
            }
            p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
            p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * correction[r] + tile_sum[r];
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            o_acc[i][0] *= correction[0];
            o_acc[i][1] *= correction[0];
            o_acc[i][2] *= correction[1];
            o_acc[i][3] *= correction[1];
        }

        // ---- O += P V
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
            for (int dn = 0; dn < DTILES; dn += 2) {
                const int r = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = (dn + (lane >> 4)) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(smem_addr(vt + r * ROW_BYTES + col * 2), b0, b1, b2, b3);
                mma_bf16(o_acc[dn], p_frag[ks], b0, b1);
                mma_bf16(o_acc[dn + 1], p_frag[ks], b2, b3);
            }
        }
        }  // warp_has_keys
        __syncthreads();  // the stage is refilled by the next iteration's prefetch
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    pdl_trigger();

    // ---- normalise and store
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float s = row_sum[r];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        row_sum[r] = s > 0.0f ? 1.0f / s : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row_block + g + r * 8;
        if (active && row < rows) {
            __nv_bfloat16* dst = a.out + ((size_t)(first_token + row) * a.heads + head) * D;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
                const uint32_t packed = pack_bf16(o_acc[i][r * 2] * row_sum[r], o_acc[i][r * 2 + 1] * row_sum[r]);
                *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = packed;
            }
        }
    }
}

template <int D, int HG>
int launch_heads(const PrefillArgs& a, int tiles, cudaStream_t stream) {
    constexpr int SMEM = (HG * BM + 4 * BN) * (D * 2 + 16);
    auto kernel = flash_prefill_kernel<D, HG>;
    if (SMEM > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
    }
    const int group = a.heads / a.kv_heads;
    dim3 grid(a.kv_heads * ((group + HG - 1) / HG), tiles);
    launch_kernel(kernel, grid, HG * 128, SMEM, stream, a);
    return launch_status();
}

// heads of a KV group served by one CTA: as many as the group has, up to 4 (2 for wide heads,
// whose output accumulators need the registers)
template <int D>
int launch(const PrefillArgs& a, int tiles, cudaStream_t stream) {
    const int group = a.heads / a.kv_heads;
    constexpr int MAX_HG = D <= 64 ? 4 : 2;
    if constexpr (MAX_HG >= 4) {
        if (group >= 3) return launch_heads<D, 4>(a, tiles, stream);
    }
    if (group >= 2) return launch_heads<D, 2>(a, tiles, stream);
    return launch_heads<D, 1>(a, tiles, stream);
}

}  // namespace

// `max_tiles` >= sum over sequences of ceil(q_len / 64); surplus CTAs exit at once.
SHISO_API int shiso_prefill_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                      int table_width, const int* q_start, const int* start_pos, void* out,
                                      int num_seqs, int max_tiles, int heads, int kv_heads, int head_dim, int page_size,
                                      float scale, int window, cudaStream_t stream) {
    if (num_seqs <= 0 || max_tiles <= 0) return SHISO_OK;
    if (kv_heads <= 0 || heads % kv_heads) return SHISO_ERR_SHAPE;
    if (head_dim % 16 || head_dim < 16 || head_dim > 128 || max_tiles > 65535) return SHISO_ERR_UNSUPPORTED;
    PrefillArgs a;
    a.q = (const __nv_bfloat16*)q;
    a.k_cache = (const __nv_bfloat16*)k_cache;
    a.v_cache = (const __nv_bfloat16*)v_cache;
    a.block_table = block_table;
    a.q_start = q_start;
    a.start_pos = start_pos;
    a.out = (__nv_bfloat16*)out;
    a.width = table_width;
    a.num_seqs = num_seqs;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.page_size = page_size;
    a.window = window;
    a.scale_log2 = scale * 1.4426950408889634f;
    switch (head_dim) {
        case 16: return launch<16>(a, max_tiles, stream);
        case 32: return launch<32>(a, max_tiles, stream);
        case 48: return launch<48>(a, max_tiles, stream);
        case 64: return launch<64>(a, max_tiles, stream);
        case 80: return launch<80>(a, max_tiles, stream);
        case 96: return launch<96>(a, max_tiles, stream);
        case 112: return launch<112>(a, max_tiles, stream);
        case 128: return launch<128>(a, max_tiles, stream);
        default: return SHISO_ERR_UNSUPPORTED;
    }
}
