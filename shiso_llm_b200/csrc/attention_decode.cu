// Paged GQA attention for steps in which every sequence brings one token (decode), bfloat16.
//
// A decode step reads every live request's keys and values once; at batch 64 that is half
// of the step's bytes, so the kernel is organised around reading the cache once and wide:
// one CTA per (key range, KV head, sequence) serves all query heads of the group from the
// same keys and values (the reference reads them once per query head:
// kernels/cuda/dense/dense_attn.cuh:44-180), and the key range of a sequence is cut into
// `splits` parts so that a few long sequences still fill 148 SMs.  Each part leaves an
// unnormalised output with its running maximum and sum in scratch memory; a second kernel
// merges the parts in index order.  The number of parts is fixed by the launch (capacity),
// the cut points are computed on the device from the sequence's own length, so a captured
// step serves any lengths.
//
// Scores: lane-per-key dot products against the float query in shared memory;
// softmax statistics in float; P*V with one key per iteration, lanes across head columns.
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

// D = head size (16, 32, 64, 128 or 256), GMAX = query heads per KV head, rounded up.
//
// Memory-level parallelism is what this kernel lives on, so both phases issue all their
// loads before they use any.  Scores: lane-per-key, the key row read in 16-byte pieces, 8
// of them in flight per lane.  P*V: the value rows of a 32-key group are read 16 bytes per
// lane with D/8 lanes across a row, so 8 load instructions fetch the whole group; a lane
// accumulates 8 columns of the rows it sees and the lanes that share columns are summed
// once at the end.
template <int D, int GMAX>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(DecodeArgs a) {
    pdl_begin();
    constexpr int LANES_PER_ROW = D / 8;                                   // 2 .. 32
    constexpr int ROWS_PER_LOAD = 32 / LANES_PER_ROW;                      // 16 .. 1
    constexpr int V_LOADS = 32 / ROWS_PER_LOAD;                            // loads per 32-key group
    constexpr int K_CHUNK = D < 64 ? D : 64;                               // elements of a key row per batch of loads

    extern __shared__ float smem[];
    const int group = a.heads / a.kv_heads;
    float* q_s = smem;                               // [GMAX][D]
    float* p_s = q_s + GMAX * D;                     // [WARPS][GMAX][32]
    int* row_s = (int*)(p_s + WARPS * GMAX * 32);    // [WARPS][32]
    float* merge_ml = (float*)(row_s + WARPS * 32);  // [WARPS][GMAX][2]
    float* merge_acc = merge_ml + WARPS * GMAX * 2;  // [WARPS][GMAX][D]

    const int split = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pos = a.positions[t];
    const int lo = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
    const int n_keys = pos + 1 - lo;
    int chunk = (n_keys + a.splits - 1) / a.splits;
    chunk = (chunk + 31) & ~31;
    const int begin = lo + split * chunk;
    const int end = min(begin + chunk, pos + 1);
    const int* table = a.block_table + (size_t)a.seq_of_token[t] * a.width;

    for (int i = threadIdx.x; i < group * D; i += blockDim.x) {
        const int h = i / D, c = i % D;
        q_s[h * D + c] = __bfloat162float(a.q[((size_t)t * a.heads + g * group + h) * D + c]);
    }
    __syncthreads();

    const int my_col = (lane % LANES_PER_ROW) * 8;   // the 8 value columns this lane accumulates
    const int my_sub = lane / LANES_PER_ROW;         // which row of each load this lane sees
    float acc[GMAX][8];
    float run_max[GMAX], run_sum[GMAX];
#pragma unroll
    for (int h = 0; h < GMAX; ++h) {
        run_max[h] = -INFINITY;
        run_sum[h] = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[h][c] = 0.0f;
    }

    for (int p0 = begin + warp * 32; p0 < end; p0 += WARPS * 32) {
        const int p = p0 + lane;
        const bool valid = p < end;
        float score[GMAX];
#pragma unroll
        for (int h = 0; h < GMAX; ++h) score[h] = 0.0f;
        int row = 0;
        if (valid) {
            row = table[p / a.page_size] * a.page_size + p % a.page_size;
            const __nv_bfloat16* k_row = a.k_cache + ((size_t)row * a.kv_heads + g) * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += K_CHUNK) {
                uint4 raw[K_CHUNK / 8];
#pragma unroll
                for (int i = 0; i < K_CHUNK / 8; ++i) raw[i] = *reinterpret_cast<const uint4*>(k_row + c0 + i * 8);
#pragma unroll
                for (int i = 0; i < K_CHUNK / 8; ++i) {
                    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
                    float kf[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __bfloat1622float2(pairs[e]);
                        kf[2 * e] = f.x;
                        kf[2 * e + 1] = f.y;
                    }
#pragma unroll
                    for (int h = 0; h < GMAX; ++h) {
                        if (h < group) {
                            const float4 q0 = *reinterpret_cast<const float4*>(q_s + h * D + c0 + i * 8);
                            const float4 q1 = *reinterpret_cast<const float4*>(q_s + h * D + c0 + i * 8 + 4);
                            score[h] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3] +
                                        q1.x * kf[4] + q1.y * kf[5] + q1.z * kf[6] + q1.w * kf[7];
                        }
                    }
                }
            }
        }
        row_s[warp * 32 + lane] = row;
#pragma unroll
        for (int h = 0; h < GMAX; ++h) {
            if (h < group) {
                const float s = valid ? score[h] * a.scale : -INFINITY;  // the scale meets the reduced dot
                const float new_max = fmaxf(run_max[h], warp_max(s));
                const float weight = valid ? expf(s - new_max) : 0.0f;
                const float correction = expf(run_max[h] - new_max);
                run_sum[h] = run_sum[h] * correction + warp_sum(weight);
                run_max[h] = new_max;
#pragma unroll
                for (int c = 0; c < 8; ++c) acc[h][c] *= correction;
                p_s[(warp * GMAX + h) * 32 + lane] = weight;
            }
        }
        __syncwarp();
        const int count = min(32, end - p0);
        uint4 vraw[V_LOADS];
#pragma unroll
        for (int i = 0; i < V_LOADS; ++i) {
            const int j = i * ROWS_PER_LOAD + my_sub;
            vraw[i] = make_uint4(0u, 0u, 0u, 0u);
            if (j < count) {
                const __nv_bfloat16* v_row = a.v_cache + ((size_t)row_s[warp * 32 + j] * a.kv_heads + g) * D;
                vraw[i] = *reinterpret_cast<const uint4*>(v_row + my_col);
            }
        }
#pragma unroll
        for (int i = 0; i < V_LOADS; ++i) {
            const int j = i * ROWS_PER_LOAD + my_sub;  // weights of keys past `count` are zero
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&vraw[i]);
            float vf[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(pairs[e]);
                vf[2 * e] = f.x;
                vf[2 * e + 1] = f.y;
            }
#pragma unroll
            for (int h = 0; h < GMAX; ++h) {
                if (h < group) {
                    const float w = p_s[(warp * GMAX + h) * 32 + j];
#pragma unroll
                    for (int c = 0; c < 8; ++c) acc[h][c] = fmaf(w, vf[c], acc[h][c]);
                }
            }
        }
        __syncwarp();
    }

    // lanes that hold the same columns (different rows) are summed, then the four warps merge
#pragma unroll
    for (int h = 0; h < GMAX; ++h) {
        if (h < group) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float v = acc[h][c];
#pragma unroll
                for (int o = LANES_PER_ROW; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[h][c] = v;
            }
            if (lane == 0) {
                merge_ml[(warp * GMAX + h) * 2] = run_max[h];
                merge_ml[(warp * GMAX + h) * 2 + 1] = run_sum[h];
            }
            if (lane < LANES_PER_ROW) {
#pragma unroll
                for (int c = 0; c < 8; ++c) merge_acc[(warp * GMAX + h) * D + my_col + c] = acc[h][c];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * D; i += blockDim.x) {
        const int h = i / D, col = i % D;
        float m = -INFINITY;
        for (int w = 0; w < WARPS; ++w) m = fmaxf(m, merge_ml[(w * GMAX + h) * 2]);
        float sum = 0.0f, out = 0.0f;
        for (int w = 0; w < WARPS; ++w) {
            const float wm = merge_ml[(w * GMAX + h) * 2];
            const float f = wm == -INFINITY ? 0.0f : expf(wm - m);
            sum += f * merge_ml[(w * GMAX + h) * 2 + 1];
            out += f * merge_acc[(w * GMAX + h) * D + col];
        }
        float* dst = a.partial + (((size_t)t * a.heads + g * group + h) * a.splits + split) * (D + 2);
        dst[col] = out;
        if (col == 0) {
            dst[D] = m;
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
            const float f = sm == -INFINITY ? 0.0f : expf(sm - m);
            sum += f * base[s * (d + 2) + d + 1];
            acc += f * base[s * (d + 2) + col];
        }
        out[((size_t)t * heads + h) * d + col] = __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
    }
}

template <int D, int GMAX>
int launch_split(const DecodeArgs& a, int tokens, cudaStream_t stream) {
    const size_t smem = sizeof(float) * ((size_t)GMAX * D + WARPS * GMAX * 32 + WARPS * 32 + WARPS * GMAX * 2 +
                                         (size_t)WARPS * GMAX * D);
    auto kernel = decode_split_kernel<D, GMAX>;
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
    }
    dim3 grid(a.splits, a.kv_heads, tokens);
    launch_kernel(kernel, grid, WARPS * 32, smem, stream, a);
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
    if (head_dim != 16 && head_dim != 32 && head_dim != 64 && head_dim != 128 && head_dim != 256)
        return SHISO_ERR_UNSUPPORTED;  // other head sizes take the general kernel
    const int group = heads / kv_heads;
    if (group > 8) return SHISO_ERR_UNSUPPORTED;
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
    const int gmax = group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8;
    int status = SHISO_ERR_UNSUPPORTED;
#define SHISO_CASE(D_, G_) if (head_dim == D_ && gmax == G_) status = launch_split<D_, G_>(a, tokens, stream);
#define SHISO_CASES(D_) SHISO_CASE(D_, 1) SHISO_CASE(D_, 2) SHISO_CASE(D_, 4) SHISO_CASE(D_, 8)
    SHISO_CASES(16) SHISO_CASES(32) SHISO_CASES(64) SHISO_CASES(128) SHISO_CASES(256)
#undef SHISO_CASES
#undef SHISO_CASE
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
