// Paged attention for long prompt portions on the tensor-memory path (tcgen05), bfloat16,
// head size 64.
//
// One CTA owns 128 consecutive query rows of one sequence and one query head and walks the key
// tiles of 128 positions its rows can see.  Per tile:
//   S = Q K^T      tcgen05.mma (M 128, N 128, K 64), Q and the key tile in shared memory (K-major,
//                  128-byte swizzle), S in tensor memory: 128 lanes x 128 float columns;
//   softmax        four warps, a thread per row (= TMEM lane): the row's scores are read from
//                  tensor memory twice (maximum; then exponentials, their sum, and P as bfloat16
//                  into shared memory in the swizzled K-major layout the next product reads);
//   P V            tcgen05.mma (M 128, N 64, K 128), V as it lies in the cache (positions x 64, the
//                  "MN-major" B operand), into 64 more TMEM columns;
//   O += P V       accumulates in tensor memory; before it, when a row's maximum has grown, the warp
//                  that owns the row rescales its 32 lanes of O there (load, multiply, store) - most
//                  tiles after the first few need nothing.
// A producer warp brings key and value tiles from the paged cache with TMA - one box per page,
// through the block table - two stages ahead; an MMA warp issues the products.  Within a CTA a
// tile's steps follow one another; two CTAs share an SM (192 TMEM columns and 97 KB each), so one
// CTA's products run under the other's softmax.
//
// Pages wholly outside the rows' range (before every window, after the last row, holes of a
// window group's table) are never read: their box is fetched at a row coordinate past the end
// of the cache, which TMA fills with zeros.  Rows of a fetched page that lie outside the range
// are masked in the scores and zeroed in the value tile before the second product, so nothing
// stored there can reach the result.
//
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the kernel carries
// on to its end (TMEM is freed), its result then being wrong.
#include <type_traits>

#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKEY = 128; // keys per tile
constexpr int HEAD = 64;  // head size
constexpr int ROW = 128;  // bytes per row of a tile (64 bf16)
constexpr int Q_BYTES = BQ * ROW;
constexpr int KV_BYTES = BKEY * ROW;
constexpr int THREADS = 192;           // warps 0-3 softmax, 4 producer, 5 MMA
constexpr int SMEM_BYTES = Q_BYTES + 3 * KV_BYTES + 1024 + 256;  // two CTAs per SM
constexpr int TMEM_COLS = 256;         // 128 for S, 64 for O, 64 for P (two bfloat16 a column)

struct TcArgs {
    const int* block_table;  // [S, width]
    const int* q_start;      // [S + 1]
    const int* start_pos;    // [S]
    __nv_bfloat16* out;      // [T, heads * 64]
    int* status;
    int width, num_seqs, heads, kv_heads, page_size, window;
    int cache_rows;          // pages * page size: a row coordinate from here on reads zeros
    float scale_log2;        // scale * log2(e)
    long long* stamps;
};
long long* g_stamps = nullptr;
#define CK(i) do { if (a.stamps && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && it == 8) a.stamps[i] = clock64(); } while (0)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_ld_pin32(uint32_t* r) {
    tmem_ld_pin(r);
    tmem_ld_pin(r + 16);
}

// The softmax is bound by the instructions it issues, so it is written with the widest ones the
// SM has: a maximum of three, and multiply-add / add on pairs of floats held in a 64-bit register.
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// (the bound of 256 threads caps the registers at 128: registers are handed out for groups of four
// warps, so a CTA of six warps takes as many as one of eight, and two CTAs must fit an SM)
__global__ void __launch_bounds__(256, 2)
flash_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;
    uint8_t* k_s = q_s + Q_BYTES;        // [2][KV_BYTES]
    uint8_t* v_s = k_s + 2 * KV_BYTES;   // one stage: the value tile is wanted only after the softmax
    uint64_t* bars = (uint64_t*)(v_s + KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;   // [2]
    uint64_t* k_empty = bars + 3;  // [2]
    uint64_t* v_full = bars + 5;   // [1] (+ 1 unused)
    uint64_t* v_empty = bars + 7;  // [1] (+ 1 unused)
    uint64_t* s_full = bars + 9;
    uint64_t* p_full = bars + 10;
    uint64_t* o_full = bars + 11;
    uint32_t* tmem_slot = (uint32_t*)(bars + 12);
    int* shared_ints = (int*)(tmem_slot + 1);  // [0] failed, [1] sequence, [2] first row of the tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        mbar_init(s_full, 1);
        mbar_init(p_full, 4);  // one arrival per softmax warp
        mbar_init(o_full, 1);
        shared_ints[0] = 0;
        // which (sequence, tile) is this CTA?  The last tiles of a portion have the most keys:
        // they take the first CTAs - of every head, the head being the grid's fast index - so
        // that the grid's tail is made of short ones.  (With the tile as the fast index each
        // head's long tiles came after the short ones of the head before, the last heads began
        // their longest tiles in the second wave, and a 2,048-row portion took 85 us, not 52.)
        int left = gridDim.y - 1 - blockIdx.y, found = -1, row0 = 0;
        for (int s = 0; s < a.num_seqs; ++s) {
            const int tiles = (a.q_start[s + 1] - a.q_start[s] + BQ - 1) / BQ;
            if (left < tiles) {
                found = s;
                row0 = left * BQ;
                break;
            }
            left -= tiles;
        }
        shared_ints[1] = found;
        shared_ints[2] = row0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const int seq = shared_ints[1];
    if (seq < 0) return;  // uniform: before any TMEM allocation
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int row0 = shared_ints[2];
    const int first_token = a.q_start[seq] + row0;
    const int rows = min(BQ, a.q_start[seq + 1] - first_token);
    const int first_pos = a.start_pos[seq] + row0;
    const int last_pos = first_pos + rows - 1;
    const int head = blockIdx.x;
    const int kv_head = head / (a.heads / a.kv_heads);
    const int key_lo = a.window > 0 ? max(0, first_pos + 1 - a.window) : 0;  // the smallest key any row sees
    const int tile_first = key_lo / BKEY, tile_last = last_pos / BKEY;
    const int num_tiles = tile_last - tile_first + 1;
    bool failed = false;

    pdl_wait();  // queries, keys and values were written by the kernels before this one

    if (warp == 4) {
        // ---- producer: lane p brings page p of every tile (its key box and its value box), and
        // looks the page up in the block table a tile ahead, so that no copy waits for a lookup
        if (lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(q_s, &map_q, head * HEAD, first_token, q_full);
        }
        const int* table = a.block_table + (size_t)seq * a.width;
        const int pages_per_tile = BKEY / a.page_size;
        auto lookup = [&](int it) {
            const int key = (tile_first + it) * BKEY + lane * a.page_size;
            int page = -1;
            if (lane < pages_per_tile && key <= last_pos && key + a.page_size > key_lo) page = table[key / a.page_size];
            return page >= 0 ? page * a.page_size : a.cache_rows;  // a row past the end of the cache: zeros
        };
        int row_next = lookup(0);
        for (int it = 0; it < num_tiles; ++it) {
            const int s = it & 1;
            const int row = row_next;
            if (it + 1 < num_tiles) row_next = lookup(it + 1);
            for (int kv = 0; kv < 2; ++kv) {
                uint64_t* full = kv ? &v_full[0] : &k_full[s];
                uint64_t* empty = kv ? &v_empty[0] : &k_empty[s];
                uint8_t* dst = kv ? v_s : k_s + s * KV_BYTES;
                const bool reused = kv ? it >= 1 : it >= 2;
                const int uses_before = kv ? it : it >> 1;
                if (reused && !mbar_wait(empty, (uses_before - 1) & 1)) failed = true;
                if (lane == 0) mbar_expect_tx(full, KV_BYTES);
                __syncwarp();
                if (lane < pages_per_tile) tma_load_3d(dst + lane * a.page_size * ROW, kv ? &map_v : &map_k, 0, kv_head, row, full);
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(BQ, BKEY);
            const uint32_t idesc_o = umma_idesc(BQ, HEAD) | (1u << 16);  // B (the value tile) is MN-major
            const uint32_t s_tmem = tmem_base, o_tmem = tmem_base + BKEY, p_tmem = tmem_base + BKEY + HEAD;
            const uint32_t q_addr = smem_u32(q_s);
            auto scores = [&](int it) {
                const int s = it & 1;
                if (!mbar_wait(&k_full[s], (it >> 1) & 1)) failed = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = smem_u32(k_s + s * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HEAD / UMMA_K; ++ks)
                    umma_bf16(s_tmem, umma_desc(q_addr + ks * 32), umma_desc(k_addr + ks * 32), idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(s_full);
                umma_commit(&k_empty[s]);
            };
            if (!mbar_wait(q_full, 0)) failed = true;
            scores(0);
            for (int it = 0; it < num_tiles; ++it) {
                const int s = it & 1;
                if (!mbar_wait(p_full, it & 1)) failed = true;   // P is written, S and O_tile are read
                // the next tile's scores first: its softmax can begin while P V is still running
                if (it + 1 < num_tiles) scores(it + 1);
                if (!mbar_wait(&v_full[0], it & 1)) failed = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = smem_u32(v_s);
#pragma unroll
                for (int ks = 0; ks < BKEY / UMMA_K; ++ks)
                    umma_bf16_a_tmem(o_tmem, p_tmem + ks * (UMMA_K / 2), umma_desc(v_addr + ks * 16 * ROW), idesc_o, (it > 0 || ks > 0) ? 1u : 0u);
                umma_commit(o_full);
                umma_commit(&v_empty[0]);
            }
        }
    } else {
        // ---- softmax warps: thread = query row = TMEM lane
        const int r = warp * 32 + lane;
        const int my_pos = first_pos + r;
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        float row_max = -INFINITY, row_sum = 0.0f;
        for (int it = 0; it < num_tiles; ++it) {
            const int s = it & 1;
            const int key0 = (tile_first + it) * BKEY;
            // every key of the tile is seen by every row of the CTA: no mask, nothing to zero
            const bool open = key0 + BKEY - 1 <= first_pos && (a.window <= 0 || key0 > first_pos + BQ - 1 - a.window);
            CK(0);
            if (!mbar_wait(s_full, it & 1)) failed = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            CK(1);
            // The two passes over the row's scores, compiled twice: for a tile every row sees whole
            // (OPEN, most of them) without a single comparison, and with the mask.
            float alpha = 1.0f, tile_sum = 0.0f, new_max = row_max;
            auto softmax_tile = [&](auto open_tag) {
                constexpr bool OPEN = decltype(open_tag)::value;
                // Two register blocks of 32 columns take turns: one travels from tensor memory
                // while the other is worked on.
                uint32_t blk_a[32], blk_b[32];
                auto seen = [&](int key) { return key <= my_pos && (a.window <= 0 || key > my_pos - a.window); };
                // pass 1: the row's maximum over the tile
                float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one of 128 links
                auto max_block = [&](const uint32_t* raw, int c) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float v0 = __uint_as_float(raw[i]), v1 = __uint_as_float(raw[i + 1]);
                        if (!OPEN) {
                            if (!seen(key0 + c + i)) v0 = -INFINITY;
                            if (!seen(key0 + c + i + 1)) v1 = -INFINITY;
                        }
                        part_max[(i >> 1) & 3] = max3(part_max[(i >> 1) & 3], v0, v1);
                    }
                };
                tmem_ld32_issue(lane_base, blk_a);
                tmem_ld_wait(); tmem_ld_pin32(blk_a); tmem_ld32_issue(lane_base + 32, blk_b); max_block(blk_a, 0);
                tmem_ld_wait(); tmem_ld_pin32(blk_b); tmem_ld32_issue(lane_base + 64, blk_a); max_block(blk_b, 32);
                tmem_ld_wait(); tmem_ld_pin32(blk_a); tmem_ld32_issue(lane_base + 96, blk_b); max_block(blk_a, 64);
                tmem_ld_wait(); tmem_ld_pin32(blk_b); tmem_ld32_issue(lane_base, blk_a); max_block(blk_b, 96);  // pass 2's first block is on its way
                // the scale is positive: the maximum commutes with it
                const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3])) * a.scale_log2;
                new_max = fmaxf(row_max, tile_max);
                const float base = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen nothing yet
                alpha = ex2(row_max - base);                               // exp2(-inf) = 0 on the first tile
                CK(2);
                if (it > 0) {
                    // the product of the tile before is complete: O may be rescaled, P overwritten
                    if (!mbar_wait(o_full, (it - 1) & 1)) failed = true;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (!__all_sync(0xffffffffu, alpha == 1.0f)) {
                        // some row of this warp has a new maximum: O *= exp2(old - new), in tensor
                        // memory (block a is on its way: its wait comes first, block b is free)
                        tmem_ld_wait();
#pragma unroll 1
                        for (int c = 0; c < HEAD; c += 32) {
                            tmem_ld32_issue(lane_base + BKEY + c, blk_b);
                            tmem_ld_wait();
                            tmem_ld_pin32(blk_b);
#pragma unroll
                            for (int i = 0; i < 32; ++i) blk_b[i] = __float_as_uint(__uint_as_float(blk_b[i]) * alpha);
                            tmem_st32(lane_base + BKEY + c, blk_b);
                        }
                        tmem_st_wait();
                    }
                }
                CK(3);
                // pass 2: exponentials, their sum, and P into shared memory
                const uint64_t scale2 = pack2(a.scale_log2, a.scale_log2), minus_base2 = pack2(-base, -base);
                uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
                auto exp_block = [&](const uint32_t* raw, int c) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0, p1;
                        unpack2(fma2(pack2(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])), scale2, minus_base2), p0, p1);
                        p0 = ex2(p0);
                        p1 = ex2(p1);
                        if (!OPEN) {
                            if (!seen(key0 + c + i)) p0 = 0.0f;
                            if (!seen(key0 + c + i + 1)) p1 = 0.0f;
                        }
                        sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
                        packed[i >> 1] = bf16x2(p0, p1);
                    }
                    // 32 keys = 16 columns of this lane's row of P
                    tmem_st16(lane_base + BKEY + HEAD + (c >> 1), packed);
                };
                tmem_ld_wait(); tmem_ld_pin32(blk_a); tmem_ld32_issue(lane_base + 32, blk_b); exp_block(blk_a, 0);
                tmem_ld_wait(); tmem_ld_pin32(blk_b); tmem_ld32_issue(lane_base + 64, blk_a); exp_block(blk_b, 32);
                tmem_ld_wait(); tmem_ld_pin32(blk_a); tmem_ld32_issue(lane_base + 96, blk_b); exp_block(blk_a, 64);
                tmem_ld_wait(); tmem_ld_pin32(blk_b); exp_block(blk_b, 96);
                CK(4);
                float s0, s1, s2, s3;
                unpack2(sum2[0], s0, s1);
                unpack2(sum2[1], s2, s3);
                tile_sum = (s0 + s1) + (s2 + s3);
            };
            if (open) softmax_tile(std::true_type{});
            else softmax_tile(std::false_type{});
            row_sum = row_sum * alpha + tile_sum;
            row_max = new_max;
            if (!open) {
                // thread r also looks after value row r of the tile: outside the range it becomes zero
                if (!mbar_wait(&v_full[0], it & 1)) failed = true;
                const int key = key0 + r;
                if (key < key_lo || key > last_pos) {
                    uint4* row = reinterpret_cast<uint4*>(v_s + r * ROW);
#pragma unroll
                    for (int i = 0; i < ROW / 16; ++i) row[i] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            tmem_st_wait();  // P is in tensor memory
            if (!open) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // value rows zeroed by threads, read by the MMA
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            CK(5);

        }
        pdl_trigger();
        if (!mbar_wait(o_full, (num_tiles - 1) & 1)) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;  // an empty span yields zeros
        uint4* dst = reinterpret_cast<uint4*>(a.out + ((size_t)(first_token + r) * a.heads + head) * HEAD);
#pragma unroll 1
        for (int c = 0; c < HEAD; c += 32) {
            uint32_t raw[32];
            tmem_ld32_issue(lane_base + BKEY + c, raw);  // all lanes of the warp take part in the load
            tmem_ld_wait();
            tmem_ld_pin32(raw);
            if (r < rows) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 v;
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        h[j] = __floats2bfloat162_rn(__uint_as_float(raw[8 * i + 2 * j]) * inv, __uint_as_float(raw[8 * i + 2 * j + 1]) * inv);
                    dst[c / 8 + i] = v;
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (failed) shared_ints[0] = 1;
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (shared_ints[0] != 0 && threadIdx.x == 0 && a.status) atomicExch(a.status, 1);
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

SHISO_API int shiso_flash_set_stamps(long long* ptr) { g_stamps = ptr; return 0; }

// Whether the tensor-memory kernel takes this case (the caller falls back to the mma.sync kernel).
SHISO_API int shiso_prefill_attention_tc_supported(int head_dim, int page_size) {
    return head_dim == HEAD && page_size >= 8 && page_size <= BKEY && page_size % 8 == 0 && BKEY % page_size == 0 &&
           tc::encode_fn() != nullptr;
}

// q [T, heads * 64] bf16, caches [pages, page_size, kv_heads, 64] bf16, out [T, heads * 64].
// max_tiles: an upper bound on the number of 128-row query tiles over all sequences.
SHISO_API int shiso_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                         int table_width, const int* q_start, const int* start_pos, void* out,
                                         int tokens, int num_seqs, int max_tiles, int heads, int kv_heads,
                                         int page_size, long long num_pages, float scale, int window,
                                         cudaStream_t stream) {
    if (num_seqs <= 0 || max_tiles <= 0 || tokens <= 0) return SHISO_OK;
    if (kv_heads <= 0 || heads % kv_heads) return SHISO_ERR_SHAPE;
    if (!shiso_prefill_attention_tc_supported(HEAD, page_size) || max_tiles > 65535) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return SHISO_ERR_ALIGN;
    const long long cache_rows = num_pages * page_size;
    if (cache_rows + page_size > 0x7fffffffLL) return SHISO_ERR_UNSUPPORTED;
    CUtensorMap mq, mk, mv;
    if (!tc::tensor_map(q, tokens, heads * HEAD, BQ, &mq) || !tc::tensor_map_paged(k_cache, cache_rows, kv_heads, page_size, &mk) ||
        !tc::tensor_map_paged(v_cache, cache_rows, kv_heads, page_size, &mv))
        return SHISO_ERR_UNSUPPORTED;
    TcArgs a;
    a.block_table = block_table;
    a.q_start = q_start;
    a.start_pos = start_pos;
    a.out = (__nv_bfloat16*)out;
    a.status = shiso_tc_status_word();
    a.width = table_width;
    a.num_seqs = num_seqs;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.page_size = page_size;
    a.window = window;
    a.cache_rows = (int)cache_rows;
    a.scale_log2 = scale * 1.4426950408889634f;
    a.stamps = g_stamps;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        // two CTAs per SM need nearly all of the SM's shared memory: ask for the largest carve-out
        cudaFuncSetAttribute(flash_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(heads, max_tiles);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, flash_tc_kernel, mq, mk, mv, a);
}
