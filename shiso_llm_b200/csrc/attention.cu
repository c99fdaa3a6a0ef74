// Per-head QK norm + rotation + paged KV store, and paged GQA attention (general kernel).
//
// Norm/rotate/store follows kernels/cuda/dense/dense_norm_rope.cuh:25-141: each query
// and key head is RMS-normalised over head_dim with a [head_dim] weight, then rotated in
// half-split pairs (i, i + rotary_dim/2) by the angle pos * inv_freq[i]
// (dense_common.cuh:166-180; the frequency ladder arrives as a table computed once on
// the host); the key is cached normalised and rotated, the value raw, at row
// table[pos / page] * page + pos % page (dense_common.cuh:120-126).
//
// Attention follows kernels/cuda/dense/dense_attn.cuh:44-180: per (row, head) an online
// softmax over positions lo..pos (inclusive; lo = max(0, pos + 1 - window)), score =
// (q . k) * scale applied to the reduced dot, KV head = head / (heads / kv_heads).  One
// warp owns a (row, head) pair and walks the keys in order in groups of 32, so the
// result depends only on the row's own position and cache, not on the batch.  This is the
// kernel of the 32-bit path and of any head size; faster kernels for bfloat16 live in
// their own files.
#include "common.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS = 4;

template <typename AT>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(const AT* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                          const float* __restrict__ inv_freq, const int* __restrict__ positions,
                          const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                          int table_width, AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                          AT* __restrict__ q_out, int tokens, int heads, int kv_heads, int head_dim,
                          int rotary_dim, int page_size, float eps, int store) {
    pdl_begin();
    __shared__ float staged[WARPS][MAX_HEAD_DIM];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units = heads + 2 * kv_heads;
    const long long unit_index = (long long)blockIdx.x * WARPS + warp;
    if (unit_index >= (long long)tokens * units) return;
    const int t = (int)(unit_index / units);
    const int u = (int)(unit_index % units);
    const int row_width = units * head_dim;
    const AT* src = qkv + (size_t)t * row_width + (size_t)u * head_dim;
    const bool is_q = u < heads;
    const bool is_k = !is_q && u < heads + kv_heads;
    if (!is_q && !store) return;

    float* v = staged[warp];
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    float ss = 0.0f;
    if (sizeof(AT) == 2 && (head_dim & 1) == 0) {
        // two values per access (rows start on 4-byte boundaries when head_dim is even)
        const __nv_bfloat162* src2 = reinterpret_cast<const __nv_bfloat162*>(src);
        for (int i = lane; i < head_dim / 2; i += 32) {
            const float2 x = __bfloat1622float2(src2[i]);
            v[2 * i] = x.x;
            v[2 * i + 1] = x.y;
            ss += x.x * x.x + x.y * x.y;
        }
    } else {
        for (int i = lane; i < head_dim; i += 32) {
            const float x = to_f32(src[i]);
            v[i] = x;
            ss += x * x;
        }
    }
    __syncwarp();
    if (w) {
        const float inv = rsqrtf(warp_sum(ss) / (float)head_dim + eps);
        for (int i = lane; i < head_dim; i += 32) v[i] = v[i] * inv * w[i];
    }
    __syncwarp();
    if ((is_q || is_k) && rotary_dim > 0) {
        const int half = rotary_dim / 2;
        const float pos = (float)positions[t];
        for (int i = lane; i < half; i += 32) {
            const float angle = pos * inv_freq[i];
            float s, c;
            sincosf(angle, &s, &c);
            const float a = v[i], b = v[i + half];
            v[i] = a * c - b * s;
            v[i + half] = a * s + b * c;
        }
        __syncwarp();
    }
    AT* dst;
    if (is_q) {
        dst = q_out + (size_t)t * heads * head_dim + (size_t)u * head_dim;
    } else {
        const int pos = positions[t];
        const int page = block_table[(size_t)seq_of_token[t] * table_width + pos / page_size];
        const size_t row = (size_t)page * page_size + pos % page_size;
        const int h = is_k ? u - heads : u - heads - kv_heads;
        dst = (is_k ? k_cache : v_cache) + (row * kv_heads + h) * head_dim;
    }
    if (sizeof(AT) == 2 && (head_dim & 1) == 0) {
        __nv_bfloat162* dst2 = reinterpret_cast<__nv_bfloat162*>(dst);
        for (int i = lane; i < head_dim / 2; i += 32) dst2[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    } else {
        for (int i = lane; i < head_dim; i += 32) dst[i] = from_f32<AT>(v[i]);
    }
}

template <typename AT>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_kernel(const AT* __restrict__ q, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache,
                       const int* __restrict__ block_table, int table_width, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, AT* __restrict__ out, int tokens, int heads,
                       int kv_heads, int head_dim, int page_size, float scale, int window) {
    pdl_wait();
    __shared__ float q_s[WARPS][MAX_HEAD_DIM];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long index = (long long)blockIdx.x * WARPS + warp;
    if (index >= (long long)tokens * heads) return;
    const int t = (int)(index / heads), h = (int)(index % heads);
    const int g = h / (heads / kv_heads);
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos + 1 - window) : 0;
    const int* table = block_table + (size_t)seq_of_token[t] * table_width;

    const AT* q_row = q + ((size_t)t * heads + h) * head_dim;
    for (int i = lane; i < head_dim; i += 32) q_s[warp][i] = to_f32(q_row[i]);
    __syncwarp();

    constexpr int PER_LANE = MAX_HEAD_DIM / 32;
    float acc[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
    float run_max = -INFINITY, run_sum = 0.0f;

    for (int p0 = lo; p0 <= pos; p0 += 32) {
        const int p = p0 + lane;
        float s = -INFINITY;
        size_t my_row = 0;
        if (p <= pos) {
            my_row = ((size_t)table[p / page_size] * page_size + p % page_size) * kv_heads + g;
            const AT* k_row = k_cache + my_row * head_dim;
            float dot = 0.0f;
            for (int i = 0; i < head_dim; ++i) dot = fmaf(q_s[warp][i], to_f32(k_row[i]), dot);
            s = dot * scale;
        }
        const float new_max = fmaxf(run_max, warp_max(s));
        const float weight = (p <= pos) ? expf(s - new_max) : 0.0f;
        const float correction = expf(run_max - new_max);  // exp(-inf) = 0 on the first group
        run_sum = run_sum * correction + warp_sum(weight);
        run_max = new_max;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) acc[i] *= correction;
        const int count = min(32, pos - p0 + 1);
        for (int j = 0; j < count; ++j) {
            const float wj = __shfl_sync(0xffffffffu, weight, j);
            const size_t row_j = __shfl_sync(0xffffffffu, my_row, j);
            const AT* v_row = v_cache + row_j * head_dim;
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const int e = lane + 32 * i;
                if (e < head_dim) acc[i] = fmaf(wj, to_f32(v_row[e]), acc[i]);
            }
        }
    }
    pdl_trigger();
    AT* o = out + ((size_t)t * heads + h) * head_dim;
    const float inv = run_sum > 0.0f ? 1.0f / run_sum : 0.0f;  // an empty span yields zeros
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < head_dim) o[e] = from_f32<AT>(acc[i] * inv);
    }
}

}  // namespace

SHISO_API int shiso_qk_norm_rope_store(const void* qkv, int act_dtype, const float* q_w, const float* k_w,
                                       const float* inv_freq, const int* positions, const int* seq_of_token,
                                       const int* block_table, int table_width, void* k_cache, void* v_cache,
                                       void* q_out, int tokens, int heads, int kv_heads, int head_dim,
                                       int rotary_dim, int page_size, float eps, int store, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (head_dim <= 0 || head_dim > MAX_HEAD_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        return SHISO_ERR_SHAPE;
    if (rotary_dim > 0 && !inv_freq) return SHISO_ERR_SHAPE;
    const long long units = (long long)tokens * (heads + 2 * kv_heads);
    const unsigned blocks = ceil_div_u(units, WARPS);
    if (act_dtype == SHISO_F32)
        launch_kernel(qk_norm_rope_store_kernel<float>, blocks, WARPS * 32, 0, stream, 
            (const float*)qkv, q_w, k_w, inv_freq, positions, seq_of_token, block_table, table_width,
            (float*)k_cache, (float*)v_cache, (float*)q_out, tokens, heads, kv_heads, head_dim, rotary_dim,
            page_size, eps, store);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, 
            (const __nv_bfloat16*)qkv, q_w, k_w, inv_freq, positions, seq_of_token, block_table, table_width,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (__nv_bfloat16*)q_out, tokens, heads, kv_heads,
            head_dim, rotary_dim, page_size, eps, store);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

SHISO_API int shiso_paged_attention(const void* q, int act_dtype, const void* k_cache, const void* v_cache,
                                    const int* block_table, int table_width, const int* positions,
                                    const int* seq_of_token, void* out, int tokens, int heads, int kv_heads,
                                    int head_dim, int page_size, float scale, int window, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (head_dim <= 0 || head_dim > MAX_HEAD_DIM || kv_heads <= 0 || heads % kv_heads) return SHISO_ERR_SHAPE;
    const unsigned blocks = ceil_div_u((long long)tokens * heads, WARPS);
    if (act_dtype == SHISO_F32)
        launch_kernel(paged_attention_kernel<float>, blocks, WARPS * 32, 0, stream, 
            (const float*)q, (const float*)k_cache, (const float*)v_cache, block_table, table_width, positions,
            seq_of_token, (float*)out, tokens, heads, kv_heads, head_dim, page_size, scale, window);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(paged_attention_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, block_table,
            table_width, positions, seq_of_token, (__nv_bfloat16*)out, tokens, heads, kv_heads, head_dim,
            page_size, scale, window);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
