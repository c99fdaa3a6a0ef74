// Paged GQA attention for decode steps (one token per sequence), bfloat16, head size 64:
// the keys and values come in by TMA and the parts of a sequence are merged in the same kernel.
//
// The work is cut as in attention_decode.cu: one CTA per (part of the keys, KV head, sequence)
// serves the query heads of the group from one read of the cache (the reference reads it once
// per query head: kernels/cuda/dense/dense_attn.cuh:44-180).  What differs is how the bytes
// move.  A producer warp brings every page of a 64-key tile with one 3-D TMA box (page rows x
// one head x 64 values, 128-byte swizzle), each lane looking its own page up in the block
// table, into a ring of six tiles with full/empty mbarriers: a CTA with six tiles or fewer
// has all of its keys and values in flight at once, and a long part streams without a
// CTA-wide barrier per tile.  Four consumer warps take 16 keys of a tile each (Q K^T and P V
// as m16n8k16 MMAs, float softmax statistics) and are merged at the end.
//
// The parts of one (sequence, KV head) are a thread-block cluster (at most 8): every part sends
// its heads' results to the CTA that merges that head, through the cluster's shared memory; the
// cluster meets once and each CTA adds up what it was sent in part order and writes its heads'
// output, so there is no second launch and no traffic through global memory, and the result does
// not depend on which CTA finished last.
//
// Measured and dropped: one wave of persistent CTAs that walk (part, KV head, sequence) items
// with the ring running on across items.  The hand-over at the end of an item (fence, counter,
// the last part's reads) stalls that CTA's stream for microseconds, which the hardware's own
// scheduling of many short CTAs hides better: batch 64 x 2,190 keys in 4 parts took 81 us
// against 68 us here, in 8 parts 147 against 87.
//
// Where a call's time goes, from %globaltimer stamps of every CTA (batch 8 x 2,158 keys, 4 parts
// of 9 tiles, a call every 16.4 us in a captured chain): the CTAs are resident and their first
// tiles loaded before the predecessor ends; the queries are ready 1.0 us after the dependency
// wait; the tiles take 4.6 to 9.5 us with a ring of four (6.4 us at most with six: batch 8
// 17.0 -> 14.5 us, 8,192 keys 39.8 -> 31.9 us, a decode step at batch 64 58.0k -> 61.9k tokens/s);
// the four warps' merge and the part's store 1.3 us; counter, fence and the last CTA's merge 3.8 us.
//
// Every wait is bounded by a clock limit and reports through the status word.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int HEAD = 64;
constexpr int TILE = 64;           // keys per tile
constexpr int ROW = HEAD * 2;      // bytes per key or value row
constexpr int TILE_BYTES = TILE * ROW;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;  // keys, then values
// Tiles in a CTA's ring.  Six: two CTAs fit an SM (with four tiles and three CTAs an SM a part of nine
// tiles went round the ring twice).  A CTA alone takes about 0.7 us a tile whatever the SM's other
// CTAs do (the chain product - maximum - exponentials - product of one tile), so two CTAs an SM draw
// the HBM rate only while all of them are resident: 256 CTAs (batch 32 x 8 KV heads x 2,158 keys)
// took 25.9 us, 384 took 49.2 and 512 took 50.7 - a second wave of the same length.  Unsplit launches
// of more CTAs than two an SM therefore take rings of three tiles and no inbox: four CTAs fit an SM.
constexpr int RING_DEEP = 6, RING_SHALLOW = 3;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int KSTEPS = HEAD / 16;
constexpr int DTILES = HEAD / 8;
constexpr int MERGE_ROW = HEAD + 2;  // floats: output, running maximum (log2 units), sum
constexpr int MAX_PARTS = 16;       // the parts of a (sequence, KV head) are a thread-block cluster: up to 8 everywhere, 16 where the device schedules such clusters
constexpr int INBOX_ROWS = 32;      // rows a CTA may be sent: parts x the heads it merges, below 16 + 8
constexpr int smem_bytes(int stages, bool inbox) {  // ring, 256 bytes of barriers and flags, inbox; 1 KB to align the ring
    return stages * STAGE_BYTES + 256 + (inbox ? INBOX_ROWS * MERGE_ROW * 4 : 0) + 1024;
}

struct DecodeTmaArgs {
    const __nv_bfloat16* q;   // [T, heads * 64]
    const int* block_table;   // [S, width]
    const int* positions;     // [T]
    const int* seq_of_token;  // [T]
    __nv_bfloat16* out;       // [T, heads * 64]
    int* status;
    int width, heads, kv_heads, page_size, splits, window;
    int cache_rows;           // pages * page size: a row coordinate from here on reads zeros
    float scale_log2;
    // FROM_QKV: the step's rows come straight from the qkv product, [T, (heads + 2 * kv_heads) * 64]
    // (q unused): per-head RMS norm and rotation of q and of the new key happen here, and with
    // `store` the new key and value are written to the caches (else another layer has written them)
    const __nv_bfloat16* qkv;
    const float* q_w;         // [64] norm weights
    const float* k_w;
    const float* inv_freq;    // [32]
    __nv_bfloat16* k_cache;   // [pages, page, kv_heads, 64]
    __nv_bfloat16* v_cache;
    float eps;
    int store;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// All threads of all CTAs of the cluster meet.
__device__ __forceinline__ void cluster_meet() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The shared::cluster address of `local` (an address in this CTA's shared memory) in CTA `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}

__device__ __forceinline__ void store_remote(uint32_t address, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(address), "f"(v) : "memory");
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory"); }

__device__ __forceinline__ void unpack4(uint2 raw, float* v) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

__device__ __forceinline__ uint2 pack4(const float* v) {
    uint2 raw;
    raw.x = pack2(v[0], v[1]);
    raw.y = pack2(v[2], v[3]);
    return raw;
}

// FROM_QKV: a variant of its own (what it holds would cost the plain kernel registers).
// (five warps take the registers of eight: the bound of 256 threads x 2 CTAs caps them at 128 a thread)
// (the shallow ring: 160 threads x 4 CTAs caps them at 102; 96 are used and the FROM_QKV variant spills 8 bytes)
template <bool FROM_QKV, int STAGES>
__global__ void __launch_bounds__(STAGES == RING_SHALLOW ? 160 : 256, STAGES == RING_SHALLOW ? 4 : 2)
decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, DecodeTmaArgs a) {
    static_assert(CONSUMERS * 16 * MERGE_ROW * 4 <= STAGES * STAGE_BYTES, "the merge area lies over the ring");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // [STAGES][keys | values]
    uint64_t* full = (uint64_t*)(ring + STAGES * STAGE_BYTES);  // barriers and flags: 256 bytes
    uint64_t* empty = full + STAGES;
    int* shared_ints = (int*)(empty + STAGES);  // [0] failed
    float* inbox = (float*)(ring + STAGES * STAGE_BYTES + 256);  // [INBOX_ROWS][MERGE_ROW]: what the parts send this CTA (none with the shallow ring: one part)
    float* merge = (float*)ring;                // after the loop: [CONSUMERS][16][MERGE_ROW]

    const int split = blockIdx.x, g_head = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pages_per_tile = TILE / a.page_size;

    // Step data (positions, tables) was uploaded before the chain of kernels began: it may be
    // read before the predecessor has finished.  Tiles are counted on the absolute 64-key grid,
    // so that a tile is whole pages whatever the window's edge.
    const int pos = a.positions[t];
    const int seq = a.seq_of_token[t];  // asked for beside the position, not after it
    const int lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
    const int first_tile = lo / TILE, last_tile = pos / TILE;
    const int n_tiles = last_tile - first_tile + 1;
    const int per_part = (n_tiles + a.splits - 1) / a.splits;
    const int parts = (n_tiles + per_part - 1) / per_part;  // parts that have keys
    const int tile0 = first_tile + split * per_part;
    const int my_tiles = min(per_part, last_tile + 1 - tile0);
    if (my_tiles <= 0) {  // uniform: a part past the sequence's end has nothing to send
        if (parts > 1) cluster_meet();
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 2 * pages_per_tile);  // one arrival (with its bytes) per box
            mbar_init(&empty[s], CONSUMERS);
        }
        shared_ints[0] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    bool failed = false;

    const int group = a.heads / a.kv_heads;
    const int g = lane >> 2, t4 = lane & 3;
    float o_acc[DTILES][4];
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};

    if (warp == CONSUMERS) {
        // ---- producer: a lane owns one box (a page of keys or of values) of one of the tiles
        // of a round; it waits for the stage, announces its bytes and issues the copy
        const int boxes = 2 * pages_per_tile;
        const int tiles_per_round = min(STAGES, 32 / boxes);
        const int sub = lane / boxes, rest = lane % boxes, kv = rest & 1, pg = rest >> 1;
        const int* table = a.block_table + (size_t)seq * a.width;
        const uint32_t box_bytes = a.page_size * ROW;
        for (int base = 0; base < my_tiles && !failed; base += tiles_per_round) {
            const int i = base + sub;
            const bool on = sub < tiles_per_round && i < my_tiles;
            int row = a.cache_rows;  // a page wholly outside the keys this token sees: zeros
            if (on) {
                const int key = (tile0 + i) * TILE + pg * a.page_size;
                if (key <= pos && key + a.page_size > lo) row = table[key / a.page_size] * a.page_size;
            }
            // the cache rows of this step were written by the kernel before - unless this kernel
            // writes them itself: then the caches hold nothing of this step yet, the kernel
            // before only made the qkv rows, and the keys and values may start to move at once
            if (base == 0 && !FROM_QKV) pdl_wait();
            if (on) {
                const int stage = i % STAGES, use = i / STAGES;
                if (use > 0 && !mbar_wait(&empty[stage], (use - 1) & 1)) {
                    failed = true;
                } else {
                    mbar_expect_tx(&full[stage], box_bytes);
                    tma_load_3d(ring + stage * STAGE_BYTES + kv * TILE_BYTES + pg * box_bytes, kv ? &map_v : &map_k, 0, g_head,
                                row, &full[stage]);
                }
            }
            failed = __any_sync(0xffffffffu, failed);
        }
    } else {
        // ---- consumers: warp w scores keys 16w .. 16w+15 of every tile
        // FROM_QKV: what depends on no predecessor comes first - lane p's sine and cosine of pair
        // p's angle (passed round by shuffles later) and this thread's norm weights
        float cs_lane = 1.0f, sn_lane = 0.0f, wq_lo[8], wq_hi[8];
        if constexpr (FROM_QKV) {
            sincosf((float)pos * a.inv_freq[lane], &sn_lane, &cs_lane);
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // i = 4 kk + 2 h + e: column 16 kk + 8 h + 2 t4 + e and its partner 32 on
                const int c = (i >> 2) * 16 + ((i >> 1) & 1) * 8 + t4 * 2 + (i & 1);
                wq_lo[i] = a.q_w[c];
                wq_hi[i] = a.q_w[c + 32];
            }
        }
        pdl_wait();
        uint32_t q_frag[KSTEPS][4];
        {
            // the group's queries as the 16 rows of the MMA's A operand (rows past the group are zero)
            const int units = a.heads + 2 * a.kv_heads;
            const __nv_bfloat16* q_rows = FROM_QKV ? a.qkv + (size_t)t * units * HEAD : a.q + (size_t)t * a.heads * HEAD;
            const uint32_t* q_lo = reinterpret_cast<const uint32_t*>(q_rows + (size_t)(g_head * group + min(g, group - 1)) * HEAD);
            const uint32_t* q_hi = reinterpret_cast<const uint32_t*>(q_rows + (size_t)(g_head * group + min(g + 8, group - 1)) * HEAD);
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                q_frag[kk][0] = g < group ? q_lo[kk * 8 + t4] : 0u;
                q_frag[kk][1] = g + 8 < group ? q_hi[kk * 8 + t4] : 0u;
                q_frag[kk][2] = g < group ? q_lo[kk * 8 + 4 + t4] : 0u;
                q_frag[kk][3] = g + 8 < group ? q_hi[kk * 8 + 4 + t4] : 0u;
            }
            if constexpr (FROM_QKV) {
                // RMS norm over the head and rotation of the pairs (c, c + 32): a thread holds
                // columns 16 kk + 8 h + 2 t4 + e of rows g and g + 8, so a row's 64 values lie in the
                // four threads of a quad and a pair lies in one thread (kk and kk + 2)
                float ss[2] = {0.0f, 0.0f};
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q_frag[kk][r]));
                        ss[r & 1] += v.x * v.x + v.y * v.y;
                    }
                float inv[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 1);
                    ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], 2);
                    inv[r] = rsqrtf(ss[r] / (float)HEAD + a.eps);
                }
#pragma unroll
                for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = kk * 16 + h * 8 + t4 * 2;  // and c + 1; partners c + 32, c + 33
                        float cs[2], sn[2], w_lo[2], w_hi[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            cs[e] = __shfl_sync(0xffffffffu, cs_lane, c + e);
                            sn[e] = __shfl_sync(0xffffffffu, sn_lane, c + e);
                            w_lo[e] = wq_lo[kk * 4 + h * 2 + e];
                            w_hi[e] = wq_hi[kk * 4 + h * 2 + e];
                        }
#pragma unroll
                        for (int r = 0; r < 2; ++r) {  // rows g and g + 8
                            const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q_frag[kk][h * 2 + r]));
                            const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q_frag[kk + 2][h * 2 + r]));
                            const float x0 = lo2.x * inv[r] * w_lo[0], y0 = hi2.x * inv[r] * w_hi[0];
                            const float x1 = lo2.y * inv[r] * w_lo[1], y1 = hi2.y * inv[r] * w_hi[1];
                            q_frag[kk][h * 2 + r] = pack2(x0 * cs[0] - y0 * sn[0], x1 * cs[1] - y1 * sn[1]);
                            q_frag[kk + 2][h * 2 + r] = pack2(x0 * sn[0] + y0 * cs[0], x1 * sn[1] + y1 * cs[1]);
                        }
                    }
            }
        }
#pragma unroll
        for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
        const uint32_t swz = lane & 7;  // a row's 16-byte pieces are stored at piece ^ (row & 7)
        for (int i = 0; i < my_tiles; ++i) {
            const int stage = i % STAGES, use = i / STAGES;
            if (!mbar_wait(&full[stage], use & 1)) {
                failed = true;
                break;
            }
            const uint32_t kt = smem_u32(ring + stage * STAGE_BYTES) + warp * 16 * ROW;
            const uint32_t vt = kt + TILE_BYTES;
            const int key0 = (tile0 + i) * TILE + warp * 16;
            if constexpr (FROM_QKV) {
                if (a.store && pos >= key0 && pos < key0 + 16) {
                    // This token's own key and value are not in the cache yet: this warp owns their
                    // row of the tile, makes them from the qkv row - eight lanes a head, the
                    // arithmetic of the norm + rotate + store kernel, so that the cache holds the
                    // same bits whichever kernel wrote a row - and writes them into the tile and
                    // into the cache.  Lanes 0..7: the key; lanes 8..15: the value.
                    const int l8 = lane & 7, what = lane >> 3;
                    const int units = a.heads + 2 * a.kv_heads;
                    const int unit = a.heads + (what == 0 ? 0 : a.kv_heads) + g_head;
                    uint2 lo_raw = make_uint2(0u, 0u), hi_raw = lo_raw;
                    if (what < 2) {
                        const __nv_bfloat16* src = a.qkv + ((size_t)t * units + unit) * HEAD + 4 * l8;
                        lo_raw = *reinterpret_cast<const uint2*>(src);
                        hi_raw = *reinterpret_cast<const uint2*>(src + 32);
                    }
                    float x[4], y[4];
                    unpack4(lo_raw, x);
                    unpack4(hi_raw, y);
                    float square = 0.0f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) square += x[e] * x[e] + y[e] * y[e];
                    square += __shfl_xor_sync(0xffffffffu, square, 1);
                    square += __shfl_xor_sync(0xffffffffu, square, 2);
                    square += __shfl_xor_sync(0xffffffffu, square, 4);
                    float cs[4], sn[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {  // all lanes take part
                        cs[e] = __shfl_sync(0xffffffffu, cs_lane, 4 * l8 + e);
                        sn[e] = __shfl_sync(0xffffffffu, sn_lane, 4 * l8 + e);
                    }
                    if (what == 0) {
                        const float inv = rsqrtf(square / (float)HEAD + a.eps);
                        float out_lo[4], out_hi[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int p = 4 * l8 + e;
                            const float xv = x[e] * inv * a.k_w[p], yv = y[e] * inv * a.k_w[p + 32];
                            out_lo[e] = xv * cs[e] - yv * sn[e];
                            out_hi[e] = xv * sn[e] + yv * cs[e];
                        }
                        lo_raw = pack4(out_lo);
                        hi_raw = pack4(out_hi);
                    }
                    if (what < 2) {
                        const int page = a.block_table[(size_t)seq * a.width + pos / a.page_size];
                        const size_t cache_row = (size_t)page * a.page_size + pos % a.page_size;
                        __nv_bfloat16* dst = (what == 0 ? a.k_cache : a.v_cache) + (cache_row * a.kv_heads + g_head) * HEAD + 4 * l8;
                        *reinterpret_cast<uint2*>(dst) = lo_raw;
                        *reinterpret_cast<uint2*>(dst + 32) = hi_raw;
                        // the row in the tile: 16-byte piece (l8 >> 1) of the row's low half, piece 4 + .. of its high half
                        const uint32_t r = (uint32_t)(pos - (tile0 + i) * TILE);
                        const uint32_t row_addr = smem_u32(ring + stage * STAGE_BYTES) + what * TILE_BYTES + r * ROW;
                        const uint32_t piece = l8 >> 1, inside = (l8 & 1) * 8;
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(row_addr + (((piece) ^ (r & 7)) << 4) + inside), "r"(lo_raw.x), "r"(lo_raw.y) : "memory");
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(row_addr + (((piece + 4) ^ (r & 7)) << 4) + inside), "r"(hi_raw.x), "r"(hi_raw.y) : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before a later copy refills the stage
                    __syncwarp();
                }
            }
            if (key0 <= pos && key0 + 16 > lo) {  // warp-uniform: some of this warp's keys are seen
                float s_acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    const uint32_t r = (lane & 7) + (lane >> 4) * 8;
                    const uint32_t piece = kk * 2 + ((lane >> 3) & 1);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(kt + r * ROW + ((piece ^ swz) << 4), b0, b1, b2, b3);
                    mma16816(s_acc[0], q_frag[kk], b0, b1);
                    mma16816(s_acc[1], q_frag[kk], b2, b3);
                }
                float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                        const float v = (key >= lo && key <= pos) ? s_acc[j][e] * a.scale_log2 : -INFINITY;
                        s_acc[j][e] = v;
                        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                    }
                }
                float correction[2], use_max[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float m = tile_max[r];
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                    const float new_max = fmaxf(row_max[r], m);  // finite: one of the 16 keys is seen
                    use_max[r] = new_max;
                    correction[r] = exp2f(row_max[r] - new_max);
                    row_max[r] = new_max;
                }
                float tile_sum[2] = {0.0f, 0.0f};
                uint32_t p_frag[4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        p[e] = exp2f(s_acc[j][e] - use_max[e >> 1]);
                        tile_sum[e >> 1] += p[e];
                    }
                    p_frag[j * 2 + 0] = pack2(p[0], p[1]);
                    p_frag[j * 2 + 1] = pack2(p[2], p[3]);
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * correction[r] + tile_sum[r];
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    o_acc[d][0] *= correction[0];
                    o_acc[d][1] *= correction[0];
                    o_acc[d][2] *= correction[1];
                    o_acc[d][3] *= correction[1];
                }
#pragma unroll
                for (int dn = 0; dn < DTILES; dn += 2) {
                    const uint32_t r = (lane & 7) + ((lane >> 3) & 1) * 8;
                    const uint32_t piece = dn + (lane >> 4);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(vt + r * ROW + ((piece ^ swz) << 4), b0, b1, b2, b3);
                    mma16816(o_acc[dn], p_frag, b0, b1);
                    mma16816(o_acc[dn + 1], p_frag, b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);  // the producer may refill the stage
        }
    }
    pdl_trigger();
    if (failed) shared_ints[0] = 1;
    if (warp == CONSUMERS) {
        if (parts > 1) cluster_meet();
        return;
    }

    // ---- the four warps' results side by side (over the ring: every tile has been consumed)
    consumer_sync();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        float* dst = merge + ((size_t)warp * 16 + g + r * 8) * MERGE_ROW;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            dst[d * 8 + t4 * 2] = o_acc[d][r * 2];
            dst[d * 8 + t4 * 2 + 1] = o_acc[d][r * 2 + 1];
        }
        if (t4 == 0) {
            dst[HEAD] = row_max[r];
            dst[HEAD + 1] = sum;
        }
    }
    consumer_sync();
    const bool alone = parts == 1;  // nothing to merge with: the output is written here
    // Head h of the group is merged by part h % parts, which keeps the rows the parts send it at
    // inbox[(h / parts) * parts + part]: every part's result leaves for its head's CTA through
    // the cluster's shared memory, the cluster meets once, and each CTA adds up the rows of its
    // heads in part order.  (The parts used to leave their rows in global memory and count
    // themselves off on a counter there, the last one adding them up: fence, counter and its
    // reads took 3.8 us after the last part was written.)
    const uint32_t inbox_local = smem_u32(inbox);
    for (int i = tid; i < group * HEAD; i += CONSUMERS * 32) {
        const int h = i / HEAD, col = i % HEAD;
        float m = -INFINITY;
        for (int w = 0; w < CONSUMERS; ++w) m = fmaxf(m, merge[((size_t)w * 16 + h) * MERGE_ROW + HEAD]);
        float sum = 0.0f, o = 0.0f;
        for (int w = 0; w < CONSUMERS; ++w) {
            const float* src = merge + ((size_t)w * 16 + h) * MERGE_ROW;
            const float f = src[HEAD] == -INFINITY ? 0.0f : exp2f(src[HEAD] - m);
            sum += f * src[HEAD + 1];
            o += f * src[col];
        }
        if (alone) {
            const size_t head = (size_t)t * a.heads + g_head * group + h;
            a.out[head * HEAD + col] = __float2bfloat16_rn(sum > 0.0f ? o / sum : 0.0f);
        } else {
            const uint32_t row = in_cta(inbox_local, (uint32_t)(h % parts)) + (uint32_t)(((h / parts) * parts + split) * MERGE_ROW) * 4u;
            store_remote(row + col * 4u, o);
            if (col == 0) {
                store_remote(row + HEAD * 4u, m);
                store_remote(row + (HEAD + 1) * 4u, sum);
            }
        }
    }
    if (!alone) {
        cluster_meet();
        for (int i = tid; i < group * HEAD; i += CONSUMERS * 32) {
            const int h = i / HEAD, col = i % HEAD;
            if (h % parts != split) continue;
            const float* base = inbox + (size_t)(h / parts) * parts * MERGE_ROW;
            float m = -INFINITY;
            for (int s = 0; s < parts; ++s) m = fmaxf(m, base[s * MERGE_ROW + HEAD]);
            float sum = 0.0f, acc = 0.0f;
            for (int s = 0; s < parts; ++s) {  // part order
                const float sm = base[s * MERGE_ROW + HEAD];
                const float f = sm == -INFINITY ? 0.0f : exp2f(sm - m);
                sum += f * base[s * MERGE_ROW + HEAD + 1];
                acc += f * base[s * MERGE_ROW + col];
            }
            const size_t head = (size_t)t * a.heads + g_head * group + h;
            a.out[head * HEAD + col] = __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
        }
    }
    if (tid == 0 && shared_ints[0] != 0 && a.status) atomicExch(a.status, 1);
}

}  // namespace

// Whether the TMA decode kernel takes this shape (others take shiso_decode_attention).
SHISO_API int shiso_decode_attention_fused_supported(int heads, int kv_heads, int head_dim, int page_size) {
    return head_dim == HEAD && kv_heads > 0 && heads % kv_heads == 0 && heads / kv_heads <= 16 && page_size >= 8 &&
           page_size <= TILE && page_size % 8 == 0 && TILE % page_size == 0 && tc::encode_fn() != nullptr;
}

namespace {

template <bool FROM_QKV, int STAGES>
int launch_decode_tma_ring(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTmaArgs& a, int tokens, cudaStream_t stream) {
    constexpr int SMEM_BYTES = smem_bytes(STAGES, STAGES != RING_SHALLOW);
    auto kernel = decode_tma_kernel<FROM_QKV, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        configured = true;
    }
    static bool wide = false;  // clusters of more than 8 CTAs are not portable: the kernel has to allow them
    if (a.splits > 8 && !wide) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        wide = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.splits, a.kv_heads, tokens);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;  // the parts of a (sequence, KV head)
    attr[1].val.clusterDim.x = a.splits;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kernel, mk, mv, a);
}

template <bool FROM_QKV>
int launch_decode_tma(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeTmaArgs& a, int tokens, cudaStream_t stream) {
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    }
    // Waves of four CTAs an SM take a little over twice as long as waves of two, so the shallow ring
    // pays where it saves a partly empty wave: above two and up to four CTAs an SM (batch 48 x 8 KV
    // heads x 2,158 keys: 49.2 -> 40.2 us), above six and up to eight (batch 128: 105.9 -> 96.4 us);
    // between four and six three waves of two are shorter (batch 96: 85.8 us with the shallow ring,
    // the step 2 % slower), and beyond eight the two differ little.
    const long long ctas = (long long)a.kv_heads * tokens, pair = 2LL * sm_count;
    if (a.splits == 1 && ((ctas > pair && ctas <= 2 * pair) || (ctas > 3 * pair && ctas <= 4 * pair)))
        return launch_decode_tma_ring<FROM_QKV, RING_SHALLOW>(mk, mv, a, tokens, stream);
    return launch_decode_tma_ring<FROM_QKV, RING_DEEP>(mk, mv, a, tokens, stream);
}

// What both entry points check and fill in.
int prepare_decode_tma(const void* k_cache, const void* v_cache, const int* block_table, int table_width,
                       const int* positions, const int* seq_of_token, void* out, int tokens,
                       int heads, int kv_heads, int head_dim, int page_size, long long num_pages, float scale, int window,
                       int splits, DecodeTmaArgs* a, CUtensorMap* mk, CUtensorMap* mv) {
    if (kv_heads <= 0 || heads % kv_heads || splits < 1) return SHISO_ERR_SHAPE;
    if (splits > MAX_PARTS) return SHISO_ERR_UNSUPPORTED;
    if (!shiso_decode_attention_fused_supported(heads, kv_heads, head_dim, page_size)) return SHISO_ERR_UNSUPPORTED;
    if (((uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return SHISO_ERR_ALIGN;
    if (tokens > 65535 || kv_heads > 65535) return SHISO_ERR_UNSUPPORTED;  // grid limits
    const long long cache_rows = num_pages * page_size;
    if (cache_rows + page_size > 0x7fffffffLL) return SHISO_ERR_UNSUPPORTED;
    if (!tc::tensor_map_paged(k_cache, cache_rows, kv_heads, page_size, mk) ||
        !tc::tensor_map_paged(v_cache, cache_rows, kv_heads, page_size, mv))
        return SHISO_ERR_UNSUPPORTED;
    *a = DecodeTmaArgs{};
    a->block_table = block_table;
    a->positions = positions;
    a->seq_of_token = seq_of_token;
    a->out = (__nv_bfloat16*)out;
    a->status = shiso_tc_status_word();
    a->width = table_width;
    a->heads = heads;
    a->kv_heads = kv_heads;
    a->page_size = page_size;
    a->splits = splits;
    a->window = window;
    a->cache_rows = (int)cache_rows;
    a->scale_log2 = scale * 1.4426950408889634f;
    return SHISO_OK;
}

}  // namespace

// The most parts a launch may have: 16 where the device can place a cluster of 16 CTAs of the
// deep ring (asked of the occupancy calculator once), else the portable 8.
SHISO_API int shiso_decode_attention_fused_max_parts() {
    static int most = 0;
    if (most == 0) {
        most = 8;
        bool fits = true;
        for (int variant = 0; variant < 2 && fits; ++variant) {
            const void* kernel = variant == 0 ? (const void*)decode_tma_kernel<false, RING_DEEP> : (const void*)decode_tma_kernel<true, RING_DEEP>;
            constexpr int SMEM = smem_bytes(RING_DEEP, true);
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
                cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
                fits = false;
                break;
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(16, 1, 1);
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = SMEM;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 16;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) fits = false;
        }
        cudaGetLastError();
        if (fits) most = 16;
    }
    return most;
}

// As shiso_decode_attention, with the number of pages of the caches; at most shiso_decode_attention_fused_max_parts() parts, which merge
// through their cluster's shared memory (no scratch in global memory).
SHISO_API int shiso_decode_attention_fused(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                           int table_width, const int* positions, const int* seq_of_token,
                                           void* out, int tokens, int heads, int kv_heads, int head_dim,
                                           int page_size, long long num_pages, float scale, int window, int splits,
                                           cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if ((uintptr_t)q & 15) return SHISO_ERR_ALIGN;
    DecodeTmaArgs a;
    CUtensorMap mk, mv;
    const int status = prepare_decode_tma(k_cache, v_cache, block_table, table_width, positions, seq_of_token,
                                          out, tokens, heads, kv_heads, head_dim, page_size, num_pages, scale, window, splits, &a,
                                          &mk, &mv);
    if (status != SHISO_OK) return status;
    a.q = (const __nv_bfloat16*)q;
    return launch_decode_tma<false>(mk, mv, a, tokens, stream);
}

// The same from the rows of the qkv product, [T, (heads + 2 * kv_heads) * 64] bf16: the per-head RMS
// norm (weights q_w, k_w [64], eps) and the rotation of all 64 values by position * inv_freq[32]
// of the queries and of each token's new key happen in the kernel, and with `store` the new key
// and value are written into the caches (with the bits the norm + rotate + store kernel writes).
// One row per sequence.
SHISO_API int shiso_decode_attention_from_qkv(const void* qkv, const float* q_w, const float* k_w, const float* inv_freq,
                                              float eps, void* k_cache, void* v_cache, const int* block_table,
                                              int table_width, const int* positions, const int* seq_of_token,
                                              void* out, int tokens, int heads, int kv_heads,
                                              int head_dim, int page_size, long long num_pages, float scale, int window,
                                              int splits, int store, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (!qkv || !q_w || !k_w || !inv_freq) return SHISO_ERR_SHAPE;
    if ((uintptr_t)qkv & 15) return SHISO_ERR_ALIGN;
    DecodeTmaArgs a;
    CUtensorMap mk, mv;
    const int status = prepare_decode_tma(k_cache, v_cache, block_table, table_width, positions, seq_of_token,
                                          out, tokens, heads, kv_heads, head_dim, page_size, num_pages, scale, window, splits, &a,
                                          &mk, &mv);
    if (status != SHISO_OK) return status;
    a.qkv = (const __nv_bfloat16*)qkv;
    a.q_w = q_w;
    a.k_w = k_w;
    a.inv_freq = inv_freq;
    a.k_cache = (__nv_bfloat16*)k_cache;
    a.v_cache = (__nv_bfloat16*)v_cache;
    a.eps = eps;
    a.store = store;
    return launch_decode_tma<true>(mk, mv, a, tokens, stream);
}
