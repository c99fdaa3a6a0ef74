// Paged GQA attention for steps in which every sequence brings one token (decode), bfloat16.
//
// A decode step reads every live request's keys and values once; at batch 64 that is half
// of the step's bytes, so the kernel is organised around reading the cache once and wide:
// one CTA per (key range, KV head, sequence) serves all query heads of the group from the
// same keys and values, as rows of one tensor-core tile (the reference reads them once per
// query head with scalar code: kernels/cuda/dense/dense_attn.cuh:44-180), and the key range of a sequence is cut into
// `splits` parts so that a few long sequences still fill 148 SMs.  Each part leaves an
// unnormalised output with its running maximum and sum in scratch memory; a second kernel
// merges the parts in index order.  The number of parts is fixed by the launch (capacity),
// the cut points are computed on the device from the sequence's own length, so a captured
// step serves any lengths.
//
// Scores, softmax statistics and P*V are float; keys, values and the query are bfloat16.
#include <stdio.h>

#include "common.cuh"
#include "no_alloc.h"

namespace {

constexpr int WARPS = 4;

struct DecodeArgs {
    const __nv_bfloat16* q;        // [T, heads * d]
    const __nv_bfloat16* k_cache;  // [pages, page, kv_heads, d]
    const __nv_bfloat16* v_cache;
    const int* block_table;        // [S, width]
    const int* positions;          // [T]
    const int* seq_of_token;       // [T]
    float* partial;                // [T, heads, splits, d + 2]
    int width, heads, kv_heads, head_dim, page_size, splits, window;
    float scale;
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

constexpr int TILE_KEYS = 64;  // keys per shared-memory tile; each of the four warps takes 16 of them
constexpr int KV_STAGES = 2;   // tiles in flight; more stages cost occupancy and measured slower (4 stages: 20 us against 17 us at batch 8)

// D = head size (a multiple of 16 up to 128).  The query heads of one KV group (at most 16)
// are the rows of a 16-row MMA tile, so one pass over the keys serves the whole group and the
// arithmetic per key is a handful of tensor-core instructions instead of hundreds of FMAs -
// what is left is moving the cache.  Keys and values of 64 positions are gathered through
// the block table into shared memory with cp.async (16-byte pieces, whole rows, two stages);
// warp w scores keys 16w .. 16w+15 of a tile (Q K^T, m16n8k16), keeps its own running
// maximum, sum and output (P V), and the four warps are merged at the end.
template <int D>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(DecodeArgs a) {
    pdl_wait();
    constexpr int ROW_BYTES = D * 2 + 16;  // padded rows: ldmatrix without bank conflicts
    constexpr int CHUNKS = D / 8;
    constexpr int KSTEPS = D / 16;
    constexpr int DTILES = D / 8;

    extern __shared__ __align__(16) uint8_t smem_bytes[];
    uint8_t* q_s = smem_bytes;                           // [16][ROW_BYTES]
    uint8_t* k_s = q_s + 16 * ROW_BYTES;                       // [KV_STAGES][TILE_KEYS][ROW_BYTES]
    uint8_t* v_s = k_s + KV_STAGES * TILE_KEYS * ROW_BYTES;    // [KV_STAGES][TILE_KEYS][ROW_BYTES]
    float* merge = reinterpret_cast<float*>(k_s);        // after the loop: [WARPS][16][D + 2]

    const int group = a.heads / a.kv_heads;
    const int split = blockIdx.x, g_head = blockIdx.y, t = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int pos = a.positions[t];
    const int lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
    const int n_keys = pos + 1 - lo;
    // A part is at least one tile; longer ranges are divided evenly in whole tiles.  Parts past
    // the sequence's end have nothing to do.
    int chunk = (n_keys + a.splits - 1) / a.splits;
    chunk = max(TILE_KEYS, (chunk + TILE_KEYS - 1) / TILE_KEYS * TILE_KEYS);
    const int begin = lo + split * chunk;
    const int end = min(begin + chunk, pos + 1);
    const int* table = a.block_table + (size_t)a.seq_of_token[t] * a.width;
    const int tiles = end > begin ? (end - begin + TILE_KEYS - 1) / TILE_KEYS : 0;

    // the group's queries as 16 rows (rows past the group are zero)
    for (int c = tid; c < 16 * CHUNKS; c += WARPS * 32) {
        const int r = c / CHUNKS, ch = c % CHUNKS;
        const __nv_bfloat16* src = a.q + ((size_t)t * a.heads + g_head * group + min(r, group - 1)) * D + ch * 8;
        cp_async16(q_s + r * ROW_BYTES + ch * 16, src, r < group);
    }
    auto load_tile = [&](int tile, int stage) {
        uint8_t* kd = k_s + stage * TILE_KEYS * ROW_BYTES;
        uint8_t* vd = v_s + stage * TILE_KEYS * ROW_BYTES;
        for (int c = tid; c < TILE_KEYS * CHUNKS; c += WARPS * 32) {
            const int r = c / CHUNKS, ch = c % CHUNKS;
            const int key = begin + tile * TILE_KEYS + r;
            const bool valid = key < end;
            size_t row = 0;
            if (valid) row = (size_t)table[key / a.page_size] * a.page_size + key % a.page_size;
            const size_t at = (row * a.kv_heads + g_head) * D + ch * 8;
            cp_async16(kd + r * ROW_BYTES + ch * 16, a.k_cache + at, valid);
            cp_async16(vd + r * ROW_BYTES + ch * 16, a.v_cache + at, valid);
        }
    };
#pragma unroll
    for (int s = 0; s < KV_STAGES - 1; ++s) {
        if (s < tiles) load_tile(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    float o_acc[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[KSTEPS][4];
    const float scale_log2 = a.scale * 1.4426950408889634f;

    for (int tile = 0; tile < tiles; ++tile) {
        const int stage = tile % KV_STAGES;
        if (tile + KV_STAGES - 1 < tiles) load_tile(tile + KV_STAGES - 1, (tile + KV_STAGES - 1) % KV_STAGES);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(KV_STAGES - 1) : "memory");  // this tile's group has landed
        __syncthreads();
        if (tile == 0) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = kk * 16 + (lane >> 4) * 8;
                ldmatrix_x4(smem_addr(q_s + r * ROW_BYTES + col * 2), q_frag[kk][0], q_frag[kk][1], q_frag[kk][2], q_frag[kk][3]);
            }
        }
        const uint8_t* kt = k_s + stage * TILE_KEYS * ROW_BYTES + warp * 16 * ROW_BYTES;  // this warp's 16 keys
        const uint8_t* vt = v_s + stage * TILE_KEYS * ROW_BYTES + warp * 16 * ROW_BYTES;
        const int key0 = begin + tile * TILE_KEYS + warp * 16;
        if (key0 < end) {  // warp-uniform: this warp has keys in the tile
            float s_acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                const int r = (lane & 7) + (lane >> 4) * 8;
                const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_addr(kt + r * ROW_BYTES + col * 2), b0, b1, b2, b3);
                mma_bf16(s_acc[0], q_frag[kk], b0, b1);
                mma_bf16(s_acc[1], q_frag[kk], b2, b3);
            }
            float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                    const float v = key < end ? s_acc[j][e] * scale_log2 : -INFINITY;
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
                const float new_max = fmaxf(row_max[r], m);  // finite: key0 < end
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
                p_frag[j * 2 + 0] = pack_bf16(p[0], p[1]);
                p_frag[j * 2 + 1] = pack_bf16(p[2], p[3]);
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
#pragma unroll
            for (int dn = 0; dn < DTILES; dn += 2) {
                const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = (dn + (lane >> 4)) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(smem_addr(vt + r * ROW_BYTES + col * 2), b0, b1, b2, b3);
                mma_bf16(o_acc[dn], p_frag, b0, b1);
                mma_bf16(o_acc[dn + 1], p_frag, b2, b3);
            }
        }
        __syncthreads();  // the stage is refilled by the next iteration's prefetch
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    pdl_trigger();
    __syncthreads();

    // ---- merge the four warps (warp order), in log2 units, and write the part's result
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float sum = row_sum[r];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int row = g + r * 8;
        float* dst = merge + ((size_t)warp * 16 + row) * (D + 2);
#pragma unroll
        for (int i = 0; i < DTILES; ++i) {
            dst[i * 8 + t4 * 2] = o_acc[i][r * 2];
            dst[i * 8 + t4 * 2 + 1] = o_acc[i][r * 2 + 1];
        }
        if (t4 == 0) {
            dst[D] = row_max[r];
            dst[D + 1] = sum;
        }
    }
    __syncthreads();
    for (int i = tid; i < group * D; i += WARPS * 32) {
        const int h = i / D, col = i % D;
        float m = -INFINITY;
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge[((size_t)w * 16 + h) * (D + 2) + D]);
        float sum = 0.0f, out = 0.0f;
        for (int w = 0; w < WARPS; ++w) {
            const float* src = merge + ((size_t)w * 16 + h) * (D + 2);
            const float f = src[D] == -INFINITY ? 0.0f : exp2f(src[D] - m);
            sum += f * src[D + 1];
            out += f * src[col];
        }
        float* dst = a.partial + (((size_t)t * a.heads + g_head * group + h) * a.splits + split) * (D + 2);
        dst[col] = out;
        if (col == 0) {
            dst[D] = m;      // running maximum in log2 units
            dst[D + 1] = sum;
        }
    }
}

__global__ void decode_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int heads,
                                    int head_dim, int splits) {
    pdl_begin();
    const int h = blockIdx.x, t = blockIdx.y;
    const int d = head_dim;
    const float* base = partial + ((size_t)t * heads + h) * splits * (d + 2);
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, base[s * (d + 2) + d]);
    for (int col = threadIdx.x; col < d; col += blockDim.x) {
        float sum = 0.0f, acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const float sm = base[s * (d + 2) + d];
            const float f = sm == -INFINITY ? 0.0f : exp2f(sm - m);  // maxima are kept in log2 units
            sum += f * base[s * (d + 2) + d + 1];
            acc += f * base[s * (d + 2) + col];
        }
        out[((size_t)t * heads + h) * d + col] = __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
    }
}

template <int D>
int launch_split(const DecodeArgs& a, int tokens, cudaStream_t stream) {
    constexpr int ROW_BYTES = D * 2 + 16;
    constexpr int TILE_BYTES = (16 + 2 * KV_STAGES * TILE_KEYS) * ROW_BYTES;
    constexpr int MERGE_BYTES = 16 * ROW_BYTES + WARPS * 16 * (D + 2) * 4;
    constexpr int SMEM = TILE_BYTES > MERGE_BYTES ? TILE_BYTES : MERGE_BYTES;
    auto kernel = decode_split_kernel<D>;
    if (SMEM > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
    }
    dim3 grid(a.splits, a.kv_heads, tokens);
    launch_kernel(kernel, grid, WARPS * 32, SMEM, stream, a);
    return launch_status();
}

}  // namespace

// Floats of scratch the caller must provide for `tokens` rows and `splits` parts.
SHISO_API long long shiso_decode_attention_scratch_floats(int tokens, int heads, int head_dim, int splits) {
    return (long long)tokens * heads * splits * (head_dim + 2);
}

SHISO_API int shiso_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                     int table_width, const int* positions, const int* seq_of_token, float* scratch,
                                     void* out, int tokens, int heads, int kv_heads, int head_dim, int page_size,
                                     float scale, int window, int splits, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (kv_heads <= 0 || heads % kv_heads || splits < 1) return SHISO_ERR_SHAPE;
    if (head_dim % 16 || head_dim < 16 || head_dim > 128) return SHISO_ERR_UNSUPPORTED;  // these take the general kernel
    const int group = heads / kv_heads;
    if (group > 16) return SHISO_ERR_UNSUPPORTED;
    DecodeArgs a;
    a.q = (const __nv_bfloat16*)q;
    a.k_cache = (const __nv_bfloat16*)k_cache;
    a.v_cache = (const __nv_bfloat16*)v_cache;
    a.block_table = block_table;
    a.positions = positions;
    a.seq_of_token = seq_of_token;
    a.partial = scratch;
    a.width = table_width;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.head_dim = head_dim;
    a.page_size = page_size;
    a.splits = splits;
    a.window = window;
    a.scale = scale;
    int status = SHISO_ERR_UNSUPPORTED;
    switch (head_dim) {
        case 16: status = launch_split<16>(a, tokens, stream); break;
        case 32: status = launch_split<32>(a, tokens, stream); break;
        case 48: status = launch_split<48>(a, tokens, stream); break;
        case 64: status = launch_split<64>(a, tokens, stream); break;
        case 80: status = launch_split<80>(a, tokens, stream); break;
        case 96: status = launch_split<96>(a, tokens, stream); break;
        case 112: status = launch_split<112>(a, tokens, stream); break;
        case 128: status = launch_split<128>(a, tokens, stream); break;
        default: break;
    }
    if (status != 0) return status;
    dim3 grid(heads, tokens);
    launch_kernel(decode_merge_kernel, grid, head_dim >= 128 ? 128 : 64, 0, stream, scratch, (__nv_bfloat16*)out, heads, head_dim, splits);
    return launch_status();
}

// ---------------------------------------------------------------------------- no allocation
//
// The variant for callers that must not allocate (see no_alloc.h): the same two kernels, with
// the partial results in a fixed array of the device image.  In host code `no_alloc_scratch`
// is only a handle for the symbol, not a device address; the address is asked for once per
// device below and that pointer is what the kernels get.

static __device__ __align__(256) float no_alloc_scratch[SHISO_NO_ALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* no_alloc_address[MAX_DEVICES];  // per device, filled by the first call on that device
thread_local char no_alloc_error[256] = "";
}  // namespace

SHISO_API const char* shiso_no_alloc_last_error(void) { return no_alloc_error; }

SHISO_API int shiso_decode_attention_no_alloc(const void* q, const void* k_cache, const void* v_cache,
                                              const int* block_table, int table_width, const int* positions,
                                              const int* seq_of_token, void* out, int tokens, int heads, int kv_heads,
                                              int head_dim, int page_size, float scale, int window, int splits,
                                              cudaStream_t stream) {
    no_alloc_error[0] = 0;
    if (tokens <= 0) return SHISO_OK;
    if (heads <= 0 || head_dim <= 0 || splits < 1) {
        snprintf(no_alloc_error, sizeof(no_alloc_error), "heads, head_dim and splits must be positive");
        return SHISO_ERR_SHAPE;
    }
    const long long need = shiso_decode_attention_scratch_floats(tokens, heads, head_dim, splits);
    if (need > (long long)SHISO_NO_ALLOC_SCRATCH_FLOATS) {
        snprintf(no_alloc_error, sizeof(no_alloc_error),
                 "decode attention without allocation: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of "
                 "scratch, the built-in array holds %d; use fewer splits or tokens, or the entry point that takes a scratch buffer",
                 tokens, heads, splits, head_dim, need, (int)SHISO_NO_ALLOC_SCRATCH_FLOATS);
        return SHISO_ERR_TOO_LARGE;
    }
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) {
        snprintf(no_alloc_error, sizeof(no_alloc_error), "device index %d is outside the table of %d", device, MAX_DEVICES);
        return SHISO_ERR_UNSUPPORTED;
    }
    if (no_alloc_address[device] == nullptr) {
        // Set-up, once per device, with that device current: the symbol's address on THIS device.
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, no_alloc_scratch);
        if (e != cudaSuccess) {
            snprintf(no_alloc_error, sizeof(no_alloc_error), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
        no_alloc_address[device] = address;
    }
    return shiso_decode_attention(q, k_cache, v_cache, block_table, table_width, positions, seq_of_token,
                                  no_alloc_address[device], out, tokens, heads, kv_heads, head_dim, page_size, scale,
                                  window, splits, stream);
}
