// Token selection on the device, one block per row of float logits.
//
// Greedy: the lowest id attaining the highest finite logit; a row with no finite entry
// yields id 0 (crates/shiso-engine/src/sampling.rs:91-154).
//
// Stochastic: the keyed rule of the reference (sampling.rs:720-862): over the candidates
// the request allows the token is argmax(logit / temperature + G(key, position, id)) with G
// a Gumbel variate from a hash of the three, so the draw depends only on the row, the
// key and the position - not on the batch or on how the work was cut.  The candidate set
// is described by thresholds so that no sort is needed:
//   top-k  keeps every token whose logit is >= the k-th largest logit (ties stay in);
//   top-p  keeps every token whose logit is >= the logit at which the mass, summed from
//          the largest logit down over the top-k set, first reaches top_p of that set;
//   min-p  keeps tokens with exp((l - max) / T) >= min_p.
// Masses are summed as 2^-40 fixed-point integers, so the sums and therefore the
// thresholds do not depend on the order in which threads add.
//
// Suppression: ids a request may never emit are set to -inf in its row before any pick
// (crates/shiso-engine/src/sampling.rs:156-174; kernels/cuda/sample/sample.cu:18-26).
//
// Status: a picking kernel may be given a place `status_out` (by convention the entry after
// the last pick); it moves the library's status word there and clears the word, so the host
// learns with the tokens, and without another copy or wait, whether a kernel of the step gave
// up on a bounded wait.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

struct Best {
    float v;
    int i;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ Best block_best(Best mine, Best* scratch /* 32 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        mine = better(mine, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    Best r = (lane < nwarps) ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, other);
    }
    return r;
}

__device__ __forceinline__ void hand_over_status(int* status_word, int* status_out) {
    if (status_out != nullptr && status_word != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0)
        *status_out = atomicExch(status_word, 0);
}

__global__ void suppress_kernel(float* __restrict__ logits, const int* __restrict__ rows, const int* __restrict__ ids,
                                int count, int num_rows, int vocab) {
    pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int r = rows[i], id = ids[i];
    if (r >= 0 && r < num_rows && id >= 0 && id < vocab) logits[(size_t)r * vocab + id] = -INFINITY;
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab,
                                                         int* status_word, int* status_out) {
    pdl_begin();
    hand_over_status(status_word, status_out);
    __shared__ Best scratch[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    Best mine{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (isfinite(v) && v > mine.v) mine = Best{v, i};  // ascending i: the first maximum stays
    }
    const Best r = block_best(mine, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = (r.i == 0x7fffffff) ? 0 : r.i;
}

// Greedy pick in two stages for wide vocabularies: a row is cut into chunks, one block each,
// so that a handful of rows still keeps many SMs reading; the second stage picks among the
// chunk winners (ascending chunk order, so the lower id still wins a tie).
__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const float* __restrict__ logits, float* __restrict__ best_v, int* __restrict__ best_i, int vocab,
                    int chunk_len, int chunks) {
    pdl_begin();
    __shared__ Best scratch[32];
    const int chunk = blockIdx.x, row_index = blockIdx.y;
    const float* row = logits + (size_t)row_index * vocab;
    const int begin = chunk * chunk_len, end = min(begin + chunk_len, vocab);
    Best mine{-INFINITY, 0x7fffffff};
    if (((vocab | chunk_len) & 3) == 0 && (((uintptr_t)logits) & 15) == 0) {
        // four values per load; a thread still meets its values in ascending order of index
        for (int i = begin + 4 * threadIdx.x; i < end; i += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            if (isfinite(v.x) && v.x > mine.v) mine = Best{v.x, i};
            if (isfinite(v.y) && v.y > mine.v) mine = Best{v.y, i + 1};
            if (isfinite(v.z) && v.z > mine.v) mine = Best{v.z, i + 2};
            if (isfinite(v.w) && v.w > mine.v) mine = Best{v.w, i + 3};
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            if (isfinite(v) && v > mine.v) mine = Best{v, i};
        }
    }
    const Best r = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        best_v[(size_t)row_index * chunks + chunk] = r.v;
        best_i[(size_t)row_index * chunks + chunk] = r.i;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ best_v, const int* __restrict__ best_i,
                                    int* __restrict__ out, int chunks, int* status_word, int* status_out) {
    pdl_begin();
    hand_over_status(status_word, status_out);
    const int row_index = blockIdx.x;
    Best mine{-INFINITY, 0x7fffffff};
    for (int c = threadIdx.x; c < chunks; c += 32) {
        const Best other{best_v[(size_t)row_index * chunks + c], best_i[(size_t)row_index * chunks + c]};
        mine = better(mine, other);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        mine = better(mine, other);
    }
    if (threadIdx.x == 0) out[row_index] = (mine.i == 0x7fffffff) ? 0 : mine.i;
}

// ---- keyed noise ------------------------------------------------------------------------

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// A uniform in (0, 1) from (key, position, id): three rounds of the splitmix64 finalizer,
// the top 24 bits, offset half a step from both ends (sampling.rs:893-912).
__device__ __forceinline__ float keyed_uniform(unsigned long long key, unsigned position, unsigned id) {
    unsigned long long x = mix64(key + 0x9E3779B97F4A7C15ull);
    x = mix64(x ^ ((unsigned long long)position * 0xD1B54A32D192ED03ull));
    x = mix64(x ^ (unsigned long long)id);
    return ((float)(x >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

// Order-preserving map float -> uint32 (larger float, larger key).
__device__ __forceinline__ unsigned orderable(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long fixed_mass(float scaled /* (l - max) / T <= 0 */) {
    return (unsigned long long)(expf(scaled) * 1099511627776.0f);  // 2^40
}

// Finds the largest key K such that sum over {key >= K} of weight >= target, by four
// 8-bit radix passes; weight is 1 (count, for top-k) or the fixed-point mass (top-p).
// Only entries with key >= floor_key take part.  All threads return the same K.
template <bool MASS>
__device__ unsigned radix_threshold(const float* __restrict__ row, int vocab, float max_logit, float inv_t,
                                    unsigned floor_key, unsigned long long target,
                                    unsigned long long* hist /* 256 */, unsigned* shared_u /* 2 */) {
    unsigned prefix = 0, prefix_mask = 0;
    unsigned long long above = 0;  // weight of entries whose key is above the current prefix bucket
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (!isfinite(v)) continue;
            const unsigned key = orderable(v);
            if (key < floor_key || (key & prefix_mask) != prefix) continue;
            const unsigned long long wgt = MASS ? fixed_mass((v - max_logit) * inv_t) : 1ull;
            atomicAdd(&hist[(key >> shift) & 0xffu], wgt);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long run = above;
            int pick = 0;
            for (int b = 255; b >= 0; --b) {
                if (run + hist[b] >= target) {
                    pick = b;
                    break;
                }
                run += hist[b];
                pick = b;  // falls to bucket 0 when the target is never reached
            }
            shared_u[0] = (unsigned)pick;
            // 64-bit value handed back through two words
            hist[0] = run;
        }
        __syncthreads();
        const unsigned pick = shared_u[0];
        above = hist[0];
        __syncthreads();
        prefix |= pick << shift;
        prefix_mask |= 0xffu << shift;
    }
    return prefix;
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const long long* __restrict__ keys, const int* __restrict__ positions, int* __restrict__ out, int vocab,
              int* status_word, int* status_out) {
    pdl_begin();
    hand_over_status(status_word, status_out);
    __shared__ Best scratch[32];
    __shared__ unsigned long long hist[256];
    __shared__ unsigned shared_u[2];
    __shared__ unsigned long long total_mass;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;

    Best mine{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (isfinite(v) && v > mine.v) mine = Best{v, i};
    }
    const Best top = block_best(mine, scratch);
    const float temp = temperature[r];
    if (top.i == 0x7fffffff || !(temp > 0.0f)) {
        if (threadIdx.x == 0) out[r] = (top.i == 0x7fffffff) ? 0 : top.i;
        return;
    }
    const float inv_t = 1.0f / temp;
    float p_keep = top_p[r];
    if (!(p_keep > 0.0f) || p_keep > 1.0f) p_keep = 1.0f;
    const float floor_p = fmaxf(min_p[r], 0.0f);
    int k = top_k[r];
    if (k < 0) k = 0;
    if (k > vocab) k = vocab;

    unsigned floor_key = 0;  // keep keys >= floor_key
    if (k > 0) floor_key = radix_threshold<false>(row, vocab, top.v, inv_t, 0u, (unsigned long long)k, hist, shared_u);
    if (p_keep < 1.0f) {
        if (threadIdx.x == 0) total_mass = 0;
        __syncthreads();
        unsigned long long part = 0;
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            if (isfinite(v) && orderable(v) >= floor_key) part += fixed_mass((v - top.v) * inv_t);
        }
        atomicAdd(&total_mass, part);
        __syncthreads();
        // smallest integer target with target / total >= p_keep, formed in double
        const unsigned long long target = (unsigned long long)ceil((double)p_keep * (double)total_mass);
        const unsigned nucleus = radix_threshold<true>(row, vocab, top.v, inv_t, floor_key, target, hist, shared_u);
        if (nucleus > floor_key) floor_key = nucleus;
    }
    const float log_floor = floor_p > 0.0f ? logf(floor_p) : -INFINITY;

    const unsigned long long key = (unsigned long long)keys[r];
    const unsigned position = (unsigned)positions[r];
    Best pick{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (!isfinite(v) || orderable(v) < floor_key) continue;
        const float scaled = (v - top.v) * inv_t;
        if (scaled < log_floor && i != top.i) continue;
        const float u = keyed_uniform(key, position, (unsigned)i);
        const float score = scaled - logf(-logf(u));
        if (score > pick.v) pick = Best{score, i};
    }
    const Best chosen = block_best(pick, scratch);
    if (threadIdx.x == 0) out[r] = (chosen.i == 0x7fffffff) ? top.i : chosen.i;
}

// Words from one buffer to another when one of the two is pinned host memory that the device
// reads or writes in place: a step's few tokens reach the host (and its few KB of row data the
// device) as loads and stores of a kernel in the stream, without a turn of the copy engine
// between two kernels.
__global__ void __launch_bounds__(256) copy_words_kernel(const int* __restrict__ src, int* __restrict__ dst, int n) {
    pdl_begin();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

}  // namespace

// `status_out` (may be null) receives the status word, which is cleared; see the file's head.
SHISO_API int shiso_argmax(const float* logits, int* out, int rows, int vocab, int* status_out, cudaStream_t stream) {
    if (rows <= 0) return SHISO_OK;
    if (vocab <= 0) return SHISO_ERR_SHAPE;
    launch_kernel(argmax_kernel, rows, THREADS, 0, stream, logits, out, vocab, status_out ? shiso_tc_status_word() : nullptr,
                  status_out);
    return launch_status();
}

// Sets logits[rows[i], ids[i]] to -inf for i < count.
SHISO_API int shiso_suppress(float* logits, const int* rows, const int* ids, int count, int num_rows, int vocab,
                             cudaStream_t stream) {
    if (count <= 0) return SHISO_OK;
    if (vocab <= 0 || num_rows <= 0) return SHISO_ERR_SHAPE;
    launch_kernel(suppress_kernel, ceil_div_u(count, 256), 256, 0, stream, logits, rows, ids, count, num_rows, vocab);
    return launch_status();
}

SHISO_API int shiso_sample(const float* logits, const float* temperature, const int* top_k, const float* top_p,
                           const float* min_p, const long long* keys, const int* positions, int* out, int rows,
                           int vocab, int* status_out, cudaStream_t stream) {
    if (rows <= 0) return SHISO_OK;
    if (vocab <= 0) return SHISO_ERR_SHAPE;
    launch_kernel(sample_kernel, rows, THREADS, 0, stream, logits, temperature, top_k, top_p, min_p, keys, positions, out, vocab,
                  status_out ? shiso_tc_status_word() : nullptr, status_out);
    return launch_status();
}

// Two-stage greedy pick; `scratch` holds rows * chunks floats followed by rows * chunks ints.
SHISO_API int shiso_argmax_chunked(const float* logits, int* out, float* scratch, int rows, int vocab, int chunks,
                                   int* status_out, cudaStream_t stream) {
    if (rows <= 0) return SHISO_OK;
    if (vocab <= 0 || chunks <= 0) return SHISO_ERR_SHAPE;
    const int chunk_len = ((vocab + chunks - 1) / chunks + 3) / 4 * 4;  // a multiple of four: 16-byte loads where the row allows
    float* best_v = scratch;
    int* best_i = (int*)(scratch + (size_t)rows * chunks);
    launch_kernel(argmax_chunk_kernel, dim3(chunks, rows), 256, 0, stream, logits, best_v, best_i, vocab, chunk_len, chunks);
    launch_kernel(argmax_final_kernel, rows, 32, 0, stream, best_v, best_i, out, chunks,
                  status_out ? shiso_tc_status_word() : nullptr, status_out);
    return launch_status();
}

// Copies `n` 32-bit words in a kernel.  `host_side` says which buffer is pinned host memory
// (1: the source, 2: the destination, 0: neither); its device address is asked of the runtime,
// and memory that the device cannot address is refused, so the caller can fall back to a copy.
SHISO_API int shiso_copy_words(const int* src, int* dst, int n, int host_side, cudaStream_t stream) {
    if (n <= 0) return SHISO_OK;
    void* mapped = nullptr;
    if (host_side == 1 || host_side == 2) {
        void* host = host_side == 1 ? (void*)src : (void*)dst;
        if (cudaHostGetDevicePointer(&mapped, host, 0) != cudaSuccess || mapped == nullptr) {
            cudaGetLastError();
            return SHISO_ERR_UNSUPPORTED;
        }
        if (host_side == 1) src = (const int*)mapped; else dst = (int*)mapped;
    } else if (host_side != 0) {
        return SHISO_ERR_SHAPE;
    }
    launch_kernel(copy_words_kernel, n <= 65536 ? ceil_div_u(n, 256) : 256, 256, 0, stream, src, dst, n);
    return launch_status();
}
