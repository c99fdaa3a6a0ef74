// Paged attention for long prompt portions on the tensor-memory path (tcgen05), bfloat16,
// head size 64.
//
// One CTA owns 128 consecutive query rows of one sequence and one query head and walks the key
// tiles of 64 positions its rows can see.  Per tile:
//   S = Q K^T      tcgen05.mma (M 128, N 64, K 64), Q and the key tile in shared memory (K-major,
//                  128-byte swizzle), S in tensor memory: 128 lanes x 64 float columns, in one of
//                  two buffers, so that the scores of the tile after next are computed while
//                  this tile's softmax runs;
//   softmax        four warps, a thread per row (= TMEM lane): the row's 64 scores are read from
//                  tensor memory once and stay in registers for the maximum and the exponentials;
//                  P goes back to tensor memory as bfloat16 (two to a column), in one of two
//                  buffers;
//   O += P V       tcgen05.mma (M 128, N 64, K 64) with P as the A operand from tensor memory and V
//                  as it lies in the cache (positions x 64, the "MN-major" B operand), accumulated
//                  in 64 more columns.
// The exponentials are taken against a maximum that is only raised when a tile's maximum exceeds
// it by more than 2^8 (P stays below 256, sums are float): raising it means waiting for every
// product issued so far and scaling the 32 lanes of O a warp owns in tensor memory (load,
// multiply, store), and with the stale maximum most tiles wait for nothing but their own scores.
// The result divides by the sum taken against the same maximum, so it is the same softmax.
// A producer warp brings key and value tiles from the paged cache with TMA - one box per page,
// through the block table - four stages ahead; an MMA warp issues the products.  Two CTAs share
// an SM (256 TMEM columns and 81 KB each).
//
// Pages wholly outside the rows' range (before every window, after the last row, holes of a
// window group's table) are never read: their box is fetched at a row coordinate past the end
// of the cache, which TMA fills with zeros.  Rows of a fetched page that lie outside the range
// are masked in the scores and zeroed in the value tile before the second product, so nothing
// stored there can reach the result.
//
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the kernel carries
// on to its end (TMEM is freed), its result then being wrong.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BQ = 128;   // query rows per CTA
constexpr int BKEY = 64;  // keys per tile
constexpr int HEAD = 64;  // head size
constexpr int ROW = 128;  // bytes per row of a tile (64 bf16)
constexpr int Q_BYTES = BQ * ROW;
constexpr int KV_BYTES = BKEY * ROW;
constexpr int STAGES = 4;              // key tiles, and value tiles
constexpr int THREADS = 192;           // warps 0-3 softmax, 4 producer, 5 MMA
constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * KV_BYTES + 1024 + 256;  // 81.25 KB: two CTAs per SM
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0;               // two buffers of 64 float columns
constexpr int O_COL = 2 * BKEY;        // 64 float columns
constexpr int P_COL = O_COL + HEAD;    // two buffers of 32 columns (two bfloat16 each)
constexpr float RAISE_STEP = 8.0f;     // log2 units a tile's maximum must exceed the one in use by

struct TcArgs {
    const int* block_table;  // [S, width]
    const int* q_start;      // [S + 1]
    const int* start_pos;    // [S]
    __nv_bfloat16* out;      // [T, heads * 64]
    int* status;
    int width, num_seqs, heads, kv_heads, page_size, window;
    int cache_rows;          // pages * page size: a row coordinate from here on reads zeros
    float scale_log2;        // scale * log2(e)
};

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
    uint8_t* k_s = q_s + Q_BYTES;             // [STAGES][KV_BYTES]
    uint8_t* v_s = k_s + STAGES * KV_BYTES;   // [STAGES][KV_BYTES]
    uint64_t* bars = (uint64_t*)(v_s + STAGES * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;              // [STAGES]
    uint64_t* k_empty = k_full + STAGES;      // [STAGES]
    uint64_t* v_full = k_empty + STAGES;      // [STAGES]
    uint64_t* v_empty = v_full + STAGES;      // [STAGES]
    uint64_t* s_full = v_empty + STAGES;      // [2] the scores of a tile are complete
    uint64_t* p_full = s_full + 2;            // [2] its P is written (and its scores are read)
    uint64_t* pv_done = p_full + 2;           // [2] its product with the values is complete
    uint32_t* tmem_slot = (uint32_t*)(pv_done + 2);
    int* shared_ints = (int*)(tmem_slot + 1);  // [0] failed, [1] sequence, [2] first row of the tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 4);  // one arrival per softmax warp
            mbar_init(&pv_done[i], 1);
        }
        shared_ints[0] = 0;
        // which (sequence, tile) is this CTA?  The last tiles of a portion have the most keys:
        // they take the first CTAs - of every head, the head being the grid's fast index - so
        // that the grid's tail is made of short ones.  (With the tile as the fast index each
        // head's long tiles came after the short ones of the head before, the last heads began
        // their longest tiles in the second wave, and a 2,048-row portion took 85 us, not 67.)
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
            const int s = it % STAGES, uses_before = it / STAGES;
            const int row = row_next;
            if (it + 1 < num_tiles) row_next = lookup(it + 1);
            for (int kv = 0; kv < 2; ++kv) {
                uint64_t* full = kv ? &v_full[s] : &k_full[s];
                uint64_t* empty = kv ? &v_empty[s] : &k_empty[s];
                uint8_t* dst = (kv ? v_s : k_s) + s * KV_BYTES;
                if (uses_before > 0 && !mbar_wait(empty, (uses_before - 1) & 1)) failed = true;
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
            const uint32_t o_tmem = tmem_base + O_COL;
            const uint32_t q_addr = smem_u32(q_s);
            auto scores = [&](int it) {
                const int s = it % STAGES;
                if (!mbar_wait(&k_full[s], (it / STAGES) & 1)) failed = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t k_addr = smem_u32(k_s + s * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HEAD / UMMA_K; ++ks)
                    umma_bf16(tmem_base + S_COL + (it & 1) * BKEY, umma_desc(q_addr + ks * 32), umma_desc(k_addr + ks * 32), idesc_s, ks > 0 ? 1u : 0u);
                umma_commit(&s_full[it & 1]);
                umma_commit(&k_empty[s]);
            };
            if (!mbar_wait(q_full, 0)) failed = true;
            scores(0);
            if (num_tiles > 1) scores(1);
            for (int it = 0; it < num_tiles; ++it) {
                const int b = it & 1, vs = it % STAGES;
                if (!mbar_wait(&p_full[b], (it >> 1) & 1)) failed = true;   // P is written, its scores are read
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (it + 2 < num_tiles) scores(it + 2);  // into the buffer this tile's scores left
                if (!mbar_wait(&v_full[vs], (it / STAGES) & 1)) failed = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t v_addr = smem_u32(v_s + vs * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < BKEY / UMMA_K; ++ks)
                    umma_bf16_a_tmem(o_tmem, tmem_base + P_COL + b * (BKEY / 2) + ks * (UMMA_K / 2), umma_desc(v_addr + ks * 16 * ROW), idesc_o,
                                     (it > 0 || ks > 0) ? 1u : 0u);
                umma_commit(&pv_done[b]);
                umma_commit(&v_empty[vs]);
            }
        }
    } else {
        // ---- softmax warps: thread = query row = TMEM lane
        const int r = warp * 32 + lane;
        const int my_pos = first_pos + r;
        const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
        float row_max = -INFINITY, row_sum = 0.0f;  // the maximum in use (scaled, log2 units) and the sum against it
        for (int it = 0; it < num_tiles; ++it) {
            const int b = it & 1;
            const int key0 = (tile_first + it) * BKEY;
            // every key of the tile is seen by every row of the CTA: no mask, nothing to zero
            const bool open = key0 + BKEY - 1 <= first_pos && (a.window <= 0 || key0 > first_pos + BQ - 1 - a.window);
            if (!mbar_wait(&s_full[b], (it >> 1) & 1)) failed = true;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[BKEY];
            tmem_ld32_issue(lane_base + S_COL + b * BKEY, sv);
            tmem_ld32_issue(lane_base + S_COL + b * BKEY + 32, sv + 32);
            tmem_ld_wait();
            tmem_ld_pin32(sv);
            tmem_ld_pin32(sv + 32);
            if (!open) {
                // a key this row does not see scores minus infinity: its exponential is zero
#pragma unroll
                for (int i = 0; i < BKEY; ++i) {
                    const int key = key0 + i;
                    if (!(key <= my_pos && (a.window <= 0 || key > my_pos - a.window))) sv[i] = __float_as_uint(-INFINITY);
                }
            }
            float part_max[8];  // eight chains of four links, not one of 64
#pragma unroll
            for (int j = 0; j < 8; ++j) part_max[j] = fmaxf(__uint_as_float(sv[2 * j]), __uint_as_float(sv[2 * j + 1]));
#pragma unroll
            for (int i = 16; i < BKEY; i += 2) part_max[(i >> 1) & 7] = max3(part_max[(i >> 1) & 7], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
            // the scale is positive: the maximum commutes with it
            const float tile_max = fmaxf(max3(part_max[0], part_max[1], part_max[2]), max3(max3(part_max[3], part_max[4], part_max[5]), part_max[6], part_max[7])) * a.scale_log2;
            // raised only by a tile that exceeds it clearly (the comparison is false for a row that
            // has seen nothing in this tile either: minus infinity on both sides)
            const float new_max = tile_max - row_max > RAISE_STEP ? tile_max : row_max;
            const float base = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen nothing yet
            const float alpha = ex2(row_max - base);                   // exp2(-inf) = 0 for a first maximum, 1 when unchanged
            // this tile's P buffer was the A operand of the product two tiles back
            if (it >= 2 && !mbar_wait(&pv_done[b], ((it - 2) >> 1) & 1)) failed = true;
            if (it > 0 && __any_sync(0xffffffffu, new_max != row_max)) {
                // some row of this warp raises its maximum: every product issued so far must be
                // complete, then O *= exp2(old - new) in tensor memory
                if (!mbar_wait(&pv_done[b ^ 1], ((it - 1) >> 1) & 1)) failed = true;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t o[32];
#pragma unroll 1
                for (int c = 0; c < HEAD; c += 32) {
                    tmem_ld32_issue(lane_base + O_COL + c, o);
                    tmem_ld_wait();
                    tmem_ld_pin32(o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + O_COL + c, o);
                }
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // exponentials, their sum, and P into tensor memory
            const uint64_t scale2 = pack2(a.scale_log2, a.scale_log2), minus_base2 = pack2(-base, -base);
            uint64_t sum2[2] = {pack2(0.0f, 0.0f), pack2(0.0f, 0.0f)};
#pragma unroll
            for (int c = 0; c < BKEY; c += 32) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    unpack2(fma2(pack2(__uint_as_float(sv[c + i]), __uint_as_float(sv[c + i + 1])), scale2, minus_base2), p0, p1);
                    p0 = ex2(p0);
                    p1 = ex2(p1);
                    sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
                    packed[i >> 1] = bf16x2(p0, p1);
                }
                tmem_st16(lane_base + P_COL + b * (BKEY / 2) + (c >> 1), packed);  // 32 keys = 16 columns of this lane's row
            }
            float s0, s1, s2, s3;
            unpack2(sum2[0], s0, s1);
            unpack2(sum2[1], s2, s3);
            row_sum = row_sum * alpha + ((s0 + s1) + (s2 + s3));
            row_max = new_max;
            if (!open) {
                // thread r also looks after value row r of the tile: outside the range it becomes zero
                const int vs = it % STAGES;
                if (!mbar_wait(&v_full[vs], (it / STAGES) & 1)) failed = true;
                const int key = key0 + r;
                if (r < BKEY && (key < key_lo || key > last_pos)) {
                    uint4* row = reinterpret_cast<uint4*>(v_s + vs * KV_BYTES + r * ROW);
#pragma unroll
                    for (int i = 0; i < ROW / 16; ++i) row[i] = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // value rows zeroed by threads, read by the MMA
            }
            tmem_st_wait();  // P (and a scaled O) are in tensor memory
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
        }
        pdl_trigger();
        if (!mbar_wait(&pv_done[(num_tiles - 1) & 1], ((num_tiles - 1) >> 1) & 1)) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = row_sum > 0.0f ? 1.0f / row_sum : 0.0f;  // an empty span yields zeros
        uint4* dst = reinterpret_cast<uint4*>(a.out + ((size_t)(first_token + r) * a.heads + head) * HEAD);
#pragma unroll 1
        for (int c = 0; c < HEAD; c += 32) {
            uint32_t raw[32];
            tmem_ld32_issue(lane_base + O_COL + c, raw);  // all lanes of the warp take part in the load
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
