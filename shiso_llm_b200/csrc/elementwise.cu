// Row kernels: embedding gather, RMS norm, fused residual-add + RMS norm, SwiGLU.
//
// Formulas follow the reference's kernels: y = x * rsqrt(mean(x^2) + eps) * w with
// the weight multiplying directly (kernels/cuda/generic/norm.cuh:39-95); the fused
// close stores the sum and normalises the stored sum (norm.cuh:105-165);
// silu(g) * u with silu(z) = z / (1 + exp(-z)) and no clamp
// (kernels/cuda/generic/glu.cuh:35-57).  The residual stream is float in both
// compute types, so the sum a + b is formed and kept in 32-bit.
#include "common.cuh"

bool shiso_pdl_enabled() {
    static const bool enabled = [] {
        const char* v = getenv("SHISO_PDL");
        return !(v && v[0] == '0');
    }();
    return enabled;
}

// --------------------------------------------------------------------------- embedding

// A row's token id comes from `ids`, or - where feed_index[t] >= 0 - from fed_tokens at that
// index: the token a sampling kernel picked on the device a step earlier, which the host has
// not seen yet.
template <typename WT>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ feed_index,
                             const int* fed_tokens, const WT* __restrict__ table,
                             float* __restrict__ out, int hidden, int vocab) {
    pdl_begin();
    const int t = blockIdx.x;
    int id = ids[t];
    if (feed_index) {
        const int from = feed_index[t];
        if (from >= 0) id = fed_tokens[from];
    }
    const bool valid = id >= 0 && id < vocab;  // the host refuses such ids; never read outside
    const WT* row = table + (size_t)(valid ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = valid ? to_f32(row[i]) : 0.0f;
}

SHISO_API int shiso_embed(const int* ids, const int* feed_index, const int* fed_tokens, const void* table,
                          int table_dtype, float* out, int tokens, int hidden, int vocab, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if ((feed_index == nullptr) != (fed_tokens == nullptr)) return SHISO_ERR_SHAPE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == SHISO_F32)
        launch_kernel(embed_kernel<float>, tokens, threads, 0, stream, ids, feed_index, fed_tokens, (const float*)table, out, hidden, vocab);
    else if (table_dtype == SHISO_BF16)
        launch_kernel(embed_kernel<__nv_bfloat16>, tokens, threads, 0, stream, ids, feed_index, fed_tokens, (const __nv_bfloat16*)table, out, hidden, vocab);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ rows,
                                   float* __restrict__ out, int hidden) {
    pdl_begin();
    const float* s = src + (size_t)rows[blockIdx.x] * hidden;
    float* d = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) d[i] = s[i];
}

SHISO_API int shiso_gather_rows(const float* src, const int* rows, float* out, int count, int hidden,
                                cudaStream_t stream) {
    if (count <= 0) return SHISO_OK;
    launch_kernel(gather_rows_kernel, count, 256, 0, stream, src, rows, out, hidden);
    return launch_status();
}

// --------------------------------------------------------------------------- RMS norm

// One block per row.  With `delta`: sum = residual + delta is formed in float; when
// `rows` is null the sum is written back to `residual` (the stream moves on), else
// row blockIdx.x of the output is the norm of source row rows[blockIdx.x] and the
// residual is left alone (used for the final norm of the wanted rows only).
template <typename AT>
__global__ void rmsnorm_kernel(float* __restrict__ residual, const AT* __restrict__ delta,
                               const int* __restrict__ rows, const float* __restrict__ w,
                               AT* __restrict__ out, int hidden, float eps) {
    pdl_begin();
    __shared__ float scratch[33];
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = residual + (size_t)src_row * hidden;
    const AT* d = delta ? delta + (size_t)src_row * hidden : nullptr;
    AT* o = out + (size_t)blockIdx.x * hidden;
    extern __shared__ float row_cache[];  // hidden floats: the summed row

    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = r[i];
        if (d) {
            v += to_f32(d[i]);
            if (!rows) r[i] = v;
        }
        row_cache[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<AT>(row_cache[i] * inv * w[i]);
}

// Four elements per thread and pass (hidden a multiple of 4): 16-byte accesses of the float
// residual, 8-byte accesses of bfloat16 rows.  Same arithmetic and the same order of the
// per-thread sums as the scalar kernel's would be for this thread-to-element map.
template <typename AT> struct Pack4;
template <> struct Pack4<float> {
    using type = float4;
    __device__ static float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    __device__ static void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Pack4<__nv_bfloat16> {
    using type = uint2;
    __device__ static float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    __device__ static void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename AT>
__global__ void rmsnorm_vec_kernel(float* residual, const AT* delta, const int* rows, const float* w, AT* out,
                                   int hidden, float eps) {
    pdl_begin();
    __shared__ float scratch[33];
    extern __shared__ float4 row_cache4[];
    const int src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = residual + (size_t)src_row * hidden;
    const AT* d = delta ? delta + (size_t)src_row * hidden : nullptr;
    AT* o = out + (size_t)blockIdx.x * hidden;
    const int quads = hidden / 4;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        float4 v = *reinterpret_cast<const float4*>(r + 4 * i);
        if (d) {
            const float4 dv = Pack4<AT>::load(d + 4 * i);
            v.x += dv.x;
            v.y += dv.y;
            v.z += dv.z;
            v.w += dv.w;
            if (!rows) *reinterpret_cast<float4*>(r + 4 * i) = v;
        }
        row_cache4[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        const float4 v = row_cache4[i];
        const float4 wv = *reinterpret_cast<const float4*>(w + 4 * i);
        Pack4<AT>::store(o + 4 * i, make_float4(v.x * inv * wv.x, v.y * inv * wv.y, v.z * inv * wv.z, v.w * inv * wv.w));
    }
}

// Rows of up to 4,096 values kept in registers: 128 threads with Q groups of four values each,
// all of a thread's loads in flight at once, no copy of the row in shared memory.  One wave of
// CTAs walks the rows, the next row's loads in flight while this one is summed and written
// (2,048 rows of 2,048 in a captured chain: 9.7 us = 5.2 TB/s of its 50 MB; one row per CTA 10.1 us;
// the shared-memory kernel above 11.5 us).
template <typename AT, int Q>
__global__ void __launch_bounds__(128)
rmsnorm_reg_kernel(float* residual, const AT* delta, const int* rows, const float* w, AT* out, int out_rows, int hidden,
                   float eps) {
    pdl_begin();
    __shared__ float scratch[33];
    const int quads = hidden / 4;
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    // A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ..: the next row's loads are in flight
    // while this row is summed and written, so that reads and writes overlap over the whole launch.
    auto load_row = [&](int index, float4 (&v)[Q], float4 (&dv)[Q]) {
        const int src_row = rows ? rows[index] : index;
        const float* r = residual + (size_t)src_row * hidden;
        const AT* d = delta ? delta + (size_t)src_row * hidden : nullptr;
#pragma unroll
        for (int q = 0; q < Q; ++q) {
            const int i = threadIdx.x + q * 128;
            v[q] = i < quads ? *reinterpret_cast<const float4*>(r + 4 * i) : zero;
            dv[q] = (d && i < quads) ? Pack4<AT>::load(d + 4 * i) : zero;
        }
    };
    float4 v[Q], dv[Q], next_v[Q], next_dv[Q], wv[Q];
    int index = blockIdx.x;
    if (index >= out_rows) return;
    load_row(index, v, dv);
#pragma unroll
    for (int q = 0; q < Q; ++q) {
        const int i = threadIdx.x + q * 128;
        wv[q] = i < quads ? *reinterpret_cast<const float4*>(w + 4 * i) : zero;
    }
    for (; index < out_rows; index += gridDim.x) {
        const bool more = index + (int)gridDim.x < out_rows;
        if (more) load_row(index + gridDim.x, next_v, next_dv);
        float* r = residual + (size_t)(rows ? rows[index] : index) * hidden;
        AT* o = out + (size_t)index * hidden;
        float ss = 0.0f;
#pragma unroll
        for (int q = 0; q < Q; ++q) {
            const int i = threadIdx.x + q * 128;
            if (delta) {
                v[q].x += dv[q].x;
                v[q].y += dv[q].y;
                v[q].z += dv[q].z;
                v[q].w += dv[q].w;
                if (!rows && i < quads) *reinterpret_cast<float4*>(r + 4 * i) = v[q];
            }
            ss += v[q].x * v[q].x + v[q].y * v[q].y + v[q].z * v[q].z + v[q].w * v[q].w;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
#pragma unroll
        for (int q = 0; q < Q; ++q) {
            const int i = threadIdx.x + q * 128;
            if (i < quads)
                Pack4<AT>::store(o + 4 * i, make_float4(v[q].x * inv * wv[q].x, v[q].y * inv * wv[q].y, v[q].z * inv * wv[q].z,
                                                        v[q].w * inv * wv[q].w));
        }
        if (more) {
#pragma unroll
            for (int q = 0; q < Q; ++q) {
                v[q] = next_v[q];
                dv[q] = next_dv[q];
            }
        }
    }
}

template <typename AT>
static void launch_rmsnorm_reg(int groups, float* residual, const AT* delta, const int* rows, const float* w, AT* out,
                               int out_rows, int hidden, float eps, cudaStream_t stream) {
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count < 1) sm_count = 1;
    }
    const int per_sm = groups <= 1 ? 16 : (groups <= 2 ? 8 : (groups <= 4 ? 5 : 2));  // CTAs that fit an SM with the variant's registers (38 / 56 / 96 / 182)
    const int grid = out_rows < sm_count * per_sm ? out_rows : sm_count * per_sm;
    if (groups <= 1) launch_kernel(rmsnorm_reg_kernel<AT, 1>, grid, 128, 0, stream, residual, delta, rows, w, out, out_rows, hidden, eps);
    else if (groups <= 2) launch_kernel(rmsnorm_reg_kernel<AT, 2>, grid, 128, 0, stream, residual, delta, rows, w, out, out_rows, hidden, eps);
    else if (groups <= 4) launch_kernel(rmsnorm_reg_kernel<AT, 4>, grid, 128, 0, stream, residual, delta, rows, w, out, out_rows, hidden, eps);
    else launch_kernel(rmsnorm_reg_kernel<AT, 8>, grid, 128, 0, stream, residual, delta, rows, w, out, out_rows, hidden, eps);
}

SHISO_API int shiso_rmsnorm(float* residual, const void* delta, const int* rows, const float* w, void* out,
                            int act_dtype, int out_rows, int hidden, float eps, cudaStream_t stream) {
    if (out_rows <= 0) return SHISO_OK;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return SHISO_ERR_SHAPE;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const bool aligned = (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (hidden % 4 == 0 && aligned && hidden <= 4096) {
        const int groups = (hidden / 4 + 127) / 128;
        if (act_dtype == SHISO_F32)
            launch_rmsnorm_reg<float>(groups, residual, (const float*)delta, rows, w, (float*)out, out_rows, hidden, eps, stream);
        else if (act_dtype == SHISO_BF16)
            launch_rmsnorm_reg<__nv_bfloat16>(groups, residual, (const __nv_bfloat16*)delta, rows, w, (__nv_bfloat16*)out, out_rows, hidden, eps, stream);
        else
            return SHISO_ERR_DTYPE;
        return launch_status();
    }
    if (hidden % 4 == 0 && aligned && smem <= 48 * 1024) {
        const int vec_threads = hidden >= 2048 ? 256 : 128;
        if (act_dtype == SHISO_F32)
            launch_kernel(rmsnorm_vec_kernel<float>, out_rows, vec_threads, smem, stream, residual, (const float*)delta, rows, w, (float*)out, hidden, eps);
        else if (act_dtype == SHISO_BF16)
            launch_kernel(rmsnorm_vec_kernel<__nv_bfloat16>, out_rows, vec_threads, smem, stream, residual, (const __nv_bfloat16*)delta, rows, w, (__nv_bfloat16*)out, hidden, eps);
        else
            return SHISO_ERR_DTYPE;
        return launch_status();
    }
    if (act_dtype == SHISO_F32) {
        auto k = rmsnorm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(k, out_rows, threads, smem, stream, residual, (const float*)delta, rows, w, (float*)out, hidden, eps);
    } else if (act_dtype == SHISO_BF16) {
        auto k = rmsnorm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(k, out_rows, threads, smem, stream, residual, (const __nv_bfloat16*)delta, rows, w, (__nv_bfloat16*)out, hidden, eps);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}

// --------------------------------------------------------------------------- SwiGLU

template <typename AT>
__global__ void swiglu_kernel(const AT* __restrict__ gate_up, AT* __restrict__ out, int inter, long long total) {
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / inter;
    const int c = (int)(i - t * inter);
    const AT* row = gate_up + (size_t)t * 2 * inter;
    const float g = to_f32(row[c]);
    const float u = to_f32(row[inter + c]);
    const float silu = g / (1.0f + expf(-g));
    out[i] = from_f32<AT>(silu * u);
}

// Eight bfloat16 values per thread (inter a multiple of 8).
__global__ void swiglu_vec_kernel(const __nv_bfloat16* gate_up, __nv_bfloat16* out, int inter, long long total8) {
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = inter / 8;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    const __nv_bfloat16* row = gate_up + (size_t)t * 2 * inter;
    const uint4 graw = *reinterpret_cast<const uint4*>(row + c);
    const uint4 uraw = *reinterpret_cast<const uint4*>(row + inter + c);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    uint4 oraw;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
        op[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * inter + c) = oraw;
}

SHISO_API int shiso_swiglu(const void* gate_up, void* out, int act_dtype, int tokens, int inter, cudaStream_t stream) {
    const long long total = (long long)tokens * inter;
    if (total <= 0) return SHISO_OK;
    const unsigned blocks = ceil_div_u(total, 256);
    if (act_dtype == SHISO_BF16 && inter % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        launch_kernel(swiglu_vec_kernel, ceil_div_u(total / 8, 256), 256, 0, stream, (const __nv_bfloat16*)gate_up,
                      (__nv_bfloat16*)out, inter, total / 8);
        return launch_status();
    }
    if (act_dtype == SHISO_F32)
        launch_kernel(swiglu_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
