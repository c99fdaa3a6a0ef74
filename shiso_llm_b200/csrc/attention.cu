// Per-head QK norm + rotation + paged KV store, and paged GQA attention (general kernel).
//
// Norm/rotate/store follows kernels/cuda/dense/dense_norm_rope.cuh:25-141: each query
// and key head is RMS-normalised over head_dim with a [head_dim] weight, then rotated in
// half-split pairs (i, i + rotary_dim/2) by the angle pos * inv_freq[i]
// (dense_common.cuh:166-180; the frequency ladder arrives as a table computed once on
// the host) - or, when the caller says `interleaved`, in adjacent pairs (2i, 2i + 1), which
// is how some checkpoints are exported; the key is cached normalised and rotated, the value raw, at row
// table[pos / page] * page + pos % page (dense_common.cuh:120-126).
//
// Attention follows kernels/cuda/dense/dense_attn.cuh:44-180: per (row, head) an online
// softmax over positions lo..pos (inclusive; lo = max(0, pos + 1 - window)), score =
// (q . k) * scale applied to the reduced dot, KV head = head / (heads / kv_heads).  One
// warp owns a (row, head) pair and walks the keys in order in groups of 32, so the
// result depends only on the row's own position and cache, not on the batch.  This is the
// kernel of the 32-bit path and of any head size; faster kernels for bfloat16 live in
// their own files.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int MAX_HEAD_DIM = 256;
constexpr int WARPS = 4;

// A unit is one head of one token: a query head, a key head or a value head.  A warp owns
// `per_warp` consecutive units of one token and keeps a unit in registers: lane l holds the
// rotation pairs (p, p + rotary_dim/2) for p = l, l + 32, .. and the elements past rotary_dim
// in the same stride.  The angle's sine and cosine are computed once per warp and serve all its
// units (the angle depends on the token and the pair, not on the head).  A unit is a few hundred
// bytes, so its time is the latency of its loads: the next unit's values are asked for before
// the current one is worked on, and HD_MAX (the head size rounded up to 64, 128 or 256) sizes the
// registers so that small heads leave room for many warps.  The lane layout, and with it every
// sum's order, is the same whatever per_warp and HD_MAX are.
template <int HD_MAX>
struct UnitRegs {
    float a[HD_MAX / 64], b[HD_MAX / 64], tl[HD_MAX / 32];
};

template <typename AT, int HD_MAX>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store_kernel(const AT* __restrict__ qkv, const float* __restrict__ q_w, const float* __restrict__ k_w,
                          const float* __restrict__ inv_freq, const int* __restrict__ positions,
                          const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                          int table_width, AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                          AT* __restrict__ q_out, int tokens, int heads, int kv_heads, int head_dim,
                          int rotary_dim, int page_size, float eps, int store, int per_warp, int interleaved) {
    pdl_begin();
    constexpr int PAIRS = HD_MAX / 64;  // rotation pairs a lane can hold
    constexpr int TAIL = HD_MAX / 32;   // unrotated elements a lane can hold
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units = heads + 2 * kv_heads;
    const int warps_per_token = (units + per_warp - 1) / per_warp;
    const long long warp_index = (long long)blockIdx.x * WARPS + warp;
    if (warp_index >= (long long)tokens * warps_per_token) return;
    const int t = (int)(warp_index / warps_per_token);
    const int u_first = (int)(warp_index % warps_per_token) * per_warp;
    const int u_last = min(store ? units : heads, u_first + per_warp);
    if (u_first >= u_last) return;
    const int half = rotary_dim / 2;
    const AT* token_row = qkv + (size_t)t * units * head_dim;
    // the two elements of rotation pair p: (p, p + half), or neighbours (2p, 2p + 1)
    auto first_of = [&](int p) { return interleaved ? 2 * p : p; };
    auto second_of = [&](int p) { return interleaved ? 2 * p + 1 : p + half; };

    auto load_unit = [&](int u, UnitRegs<HD_MAX>& r) {
        const AT* src = token_row + (size_t)u * head_dim;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            const int p = lane + 32 * j;
            r.a[j] = p < half ? to_f32(src[first_of(p)]) : 0.0f;
            r.b[j] = p < half ? to_f32(src[second_of(p)]) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < TAIL; ++j) {
            const int e = rotary_dim + lane + 32 * j;
            r.tl[j] = e < head_dim ? to_f32(src[e]) : 0.0f;
        }
    };

    UnitRegs<HD_MAX> cur, nxt;
    load_unit(u_first, cur);
    const int pos_i = positions[t];
    size_t cache_row = 0;
    if (u_last > heads) {
        const int page = block_table[(size_t)seq_of_token[t] * table_width + pos_i / page_size];
        cache_row = (size_t)page * page_size + pos_i % page_size;
    }
    float cs[PAIRS], sn[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; ++j) {
        const int p = lane + 32 * j;
        cs[j] = 1.0f;
        sn[j] = 0.0f;
        if (p < half && u_first < heads + kv_heads) sincosf((float)pos_i * inv_freq[p], &sn[j], &cs[j]);
    }

    for (int u = u_first; u < u_last; ++u) {
        if (u + 1 < u_last) load_unit(u + 1, nxt);
        const bool is_q = u < heads;
        const bool is_k = !is_q && u < heads + kv_heads;
        AT* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * heads + u) * head_dim;
        } else {
            const int h = is_k ? u - heads : u - heads - kv_heads;
            dst = (is_k ? k_cache : v_cache) + (cache_row * kv_heads + h) * head_dim;
        }
        if (is_q || is_k) {
            const float* w = is_q ? q_w : k_w;
            float ss = 0.0f;  // summed in the order pairs, then tail, whatever HD_MAX is
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) ss += cur.a[j] * cur.a[j] + cur.b[j] * cur.b[j];
#pragma unroll
            for (int j = 0; j < TAIL; ++j) ss += cur.tl[j] * cur.tl[j];
            const float inv = rsqrtf(warp_sum(ss) / (float)head_dim + eps);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int p = lane + 32 * j;
                if (p < half) {
                    const float x = cur.a[j] * inv * w[first_of(p)], y = cur.b[j] * inv * w[second_of(p)];
                    dst[first_of(p)] = from_f32<AT>(x * cs[j] - y * sn[j]);
                    dst[second_of(p)] = from_f32<AT>(x * sn[j] + y * cs[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < TAIL; ++j) {
                const int e = rotary_dim + lane + 32 * j;
                if (e < head_dim) dst[e] = from_f32<AT>(cur.tl[j] * inv * w[e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const int p = lane + 32 * j;
                if (p < half) {
                    dst[first_of(p)] = from_f32<AT>(cur.a[j]);
                    dst[second_of(p)] = from_f32<AT>(cur.b[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < TAIL; ++j) {
                const int e = rotary_dim + lane + 32 * j;
                if (e < head_dim) dst[e] = from_f32<AT>(cur.tl[j]);
            }
        }
        cur = nxt;
    }
}

// The same for bfloat16 heads of 64 values that are rotated whole (rotary_dim == 64): eight
// lanes share a head - a lane holds values 4l..4l+3 and their rotation partners 32+4l..32+4l+3,
// two 8-byte loads and stores instead of four 2-byte ones - so a warp works on four heads at a
// time, `groups_per_warp` such groups one after the other with the next group's loads in flight,
// and the angle's sine and cosine serve all of them.  At 2,048 rows the kernel above moved its
// 25 MB at 1.1 TB/s, most of its time being instructions per byte.
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_store64_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_w,
                            const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                            const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                            const int* __restrict__ block_table, int table_width, __nv_bfloat16* __restrict__ k_cache,
                            __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ q_out, int tokens, int heads,
                            int kv_heads, int page_size, float eps, int store, int groups_per_warp) {
    pdl_begin();
    constexpr int D = 64, HALF = 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane >> 3, l8 = lane & 7;
    const int units = heads + 2 * kv_heads;
    const int live_units = store ? units : heads;
    const int groups = (live_units + 3) / 4;
    const int warps_per_token = (groups + groups_per_warp - 1) / groups_per_warp;
    const long long warp_index = (long long)blockIdx.x * WARPS + warp;
    if (warp_index >= (long long)tokens * warps_per_token) return;
    const int t = (int)(warp_index / warps_per_token);
    const int g_first = (int)(warp_index % warps_per_token) * groups_per_warp;
    const int g_last = min(groups, g_first + groups_per_warp);
    const __nv_bfloat16* token_row = qkv + (size_t)t * units * D;

    auto load_unit = [&](int g, uint2& lo, uint2& hi) {
        const int u = g * 4 + sub;
        lo = hi = make_uint2(0u, 0u);
        if (g < g_last && u < live_units) {
            const __nv_bfloat16* src = token_row + (size_t)u * D + 4 * l8;
            lo = *reinterpret_cast<const uint2*>(src);
            hi = *reinterpret_cast<const uint2*>(src + HALF);
        }
    };
    uint2 lo, hi, next_lo, next_hi;
    load_unit(g_first, lo, hi);

    const int pos_i = positions[t];
    size_t cache_row = 0;
    if (g_last * 4 > heads) {
        const int page = block_table[(size_t)seq_of_token[t] * table_width + pos_i / page_size];
        cache_row = (size_t)page * page_size + pos_i % page_size;
    }
    float cs[4], sn[4], wq[8], wk[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int p = 4 * l8 + e;
        cs[e] = 1.0f;
        sn[e] = 0.0f;
        if (g_first * 4 < heads + kv_heads) sincosf((float)pos_i * inv_freq[p], &sn[e], &cs[e]);
        wq[e] = q_w[p];
        wq[4 + e] = q_w[p + HALF];
        wk[e] = k_w[p];
        wk[4 + e] = k_w[p + HALF];
    }

    auto unpack = [](uint2 raw, float* v) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    };
    auto pack = [](const float* v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        return raw;
    };

    for (int g = g_first; g < g_last; ++g) {
        load_unit(g + 1, next_lo, next_hi);
        const int u = g * 4 + sub;
        const bool is_q = u < heads;
        const bool is_k = !is_q && u < heads + kv_heads;
        float a[4], b[4];
        unpack(lo, a);
        unpack(hi, b);
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += a[e] * a[e] + b[e] * b[e];
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (u < live_units) {
            __nv_bfloat16* dst;
            if (is_q) {
                dst = q_out + ((size_t)t * heads + u) * D;
            } else {
                const int h = is_k ? u - heads : u - heads - kv_heads;
                dst = (is_k ? k_cache : v_cache) + (cache_row * kv_heads + h) * D;
            }
            if (is_q || is_k) {
                const float inv = rsqrtf(ss / (float)D + eps);
                const float* w = is_q ? wq : wk;
                float out_lo[4], out_hi[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x = a[e] * inv * w[e], y = b[e] * inv * w[4 + e];
                    out_lo[e] = x * cs[e] - y * sn[e];
                    out_hi[e] = x * sn[e] + y * cs[e];
                }
                *reinterpret_cast<uint2*>(dst + 4 * l8) = pack(out_lo);
                *reinterpret_cast<uint2*>(dst + HALF + 4 * l8) = pack(out_hi);
            } else {
                *reinterpret_cast<uint2*>(dst + 4 * l8) = lo;
                *reinterpret_cast<uint2*>(dst + HALF + 4 * l8) = hi;
            }
        }
        lo = next_lo;
        hi = next_hi;
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
                                       int rotary_dim, int page_size, float eps, int store, int interleaved,
                                       cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (head_dim <= 0 || head_dim > MAX_HEAD_DIM || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        return SHISO_ERR_SHAPE;
    if (rotary_dim > 0 && !inv_freq) return SHISO_ERR_SHAPE;
    const int units = heads + 2 * kv_heads;
    if (act_dtype == SHISO_BF16 && head_dim == 64 && rotary_dim == 64 && !interleaved &&
        (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q_out) & 7) == 0) {
        // groups of four heads: one per warp when there are few, up to eight in a row when there are many
        const int groups = ((store ? units : heads) + 3) / 4;
        int per_warp = (int)(((long long)tokens * groups + 8191) / 8192);
        per_warp = per_warp < 1 ? 1 : (per_warp > 8 ? 8 : per_warp);
        const unsigned blocks = ceil_div_u((long long)tokens * ((groups + per_warp - 1) / per_warp), WARPS);
        launch_kernel(qk_norm_rope_store64_kernel, blocks, WARPS * 32, 0, stream, (const __nv_bfloat16*)qkv, q_w, k_w, inv_freq,
                      positions, seq_of_token, block_table, table_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                      (__nv_bfloat16*)q_out, tokens, heads, kv_heads, page_size, eps, store, per_warp);
        return launch_status();
    }
    // Few units: one per warp, for the shortest chain.  Many: up to eight per warp, which share
    // the angle's sine and cosine.
    const long long all_units = (long long)tokens * units;
    int per_warp = (int)((all_units + 16383) / 16384);
    per_warp = per_warp < 1 ? 1 : (per_warp > 8 ? 8 : per_warp);
    const unsigned blocks = ceil_div_u((long long)tokens * ((units + per_warp - 1) / per_warp), WARPS);
    auto go = [&](auto kernel, auto* typed) {
        using T = std::remove_pointer_t<decltype(typed)>;
        launch_kernel(kernel, blocks, WARPS * 32, 0, stream, (const T*)qkv, q_w, k_w, inv_freq, positions, seq_of_token,
                      block_table, table_width, (T*)k_cache, (T*)v_cache, (T*)q_out, tokens, heads, kv_heads, head_dim,
                      rotary_dim, page_size, eps, store, per_warp, interleaved ? 1 : 0);
    };
    if (act_dtype == SHISO_F32) {
        float* tag = nullptr;
        if (head_dim <= 64) go(qk_norm_rope_store_kernel<float, 64>, tag);
        else if (head_dim <= 128) go(qk_norm_rope_store_kernel<float, 128>, tag);
        else go(qk_norm_rope_store_kernel<float, 256>, tag);
    } else if (act_dtype == SHISO_BF16) {
        __nv_bfloat16* tag = nullptr;
        if (head_dim <= 64) go(qk_norm_rope_store_kernel<__nv_bfloat16, 64>, tag);
        else if (head_dim <= 128) go(qk_norm_rope_store_kernel<__nv_bfloat16, 128>, tag);
        else go(qk_norm_rope_store_kernel<__nv_bfloat16, 256>, tag);
    } else {
        return SHISO_ERR_DTYPE;
    }
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
