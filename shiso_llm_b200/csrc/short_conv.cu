// Gated short convolution over the rows of one step, every sequence with its own state.
//
// proj[t] = [b | c | x] (3H wide).  u = b * x is the gated input; the request's state
// keeps the last taps-1 values of u, oldest first, in float
// (kernels/metal/dense/dense_short_conv.metal:10-15,55,61-67).
//   y[t, ch] = c[t, ch] * (sum_j w[ch, j] * u[t - (taps-1) + j, ch] + bias[ch])
// with u before the portion's first row taken from the state.  The reference walks a
// portion serially, one thread a channel (.metal:45-60); here the output kernel is
// parallel over rows and channels, and a second kernel rewrites the states afterwards
// (stream order guarantees every read of the old state has finished).
//
// The sum runs j = 0 .. taps-1 in that order for every row, so a row's result does not
// depend on where the step was cut.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 8;

// u at relative time `rel` of a sequence whose rows start at `first`: from this step's
// rows when rel >= 0, else from the state (index taps-1+rel).
template <typename AT>
__device__ __forceinline__ float gated_input(const AT* __restrict__ proj, const float* __restrict__ state_row,
                                             int first, int rel, int ch, int hidden, int taps, long long state_stride_t) {
    if (rel >= 0) {
        const AT* row = proj + (size_t)(first + rel) * 3 * hidden;
        return to_f32(row[ch]) * to_f32(row[2 * hidden + ch]);
    }
    return state_row[(size_t)(taps - 1 + rel) * state_stride_t + ch];
}

template <typename AT>
__global__ void short_conv_out_kernel(const AT* __restrict__ proj, const float* __restrict__ w,
                                      const float* __restrict__ bias, const float* __restrict__ state,
                                      long long slot_stride, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ q_start, const int* __restrict__ slots,
                                      AT* __restrict__ y, int hidden, int taps) {
    pdl_begin();
    const int t = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (ch >= hidden) return;
    const int s = seq_of_token[t];
    const int first = q_start[s];
    const float* state_row = state + (size_t)slots[s] * slot_stride;
    const int rel_now = t - first;
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int rel = rel_now - (taps - 1) + j;
        const float u = gated_input(proj, state_row, first, rel, ch, hidden, taps, hidden);
        acc = fmaf(w[(size_t)ch * taps + j], u, acc);
    }
    if (bias) acc += bias[ch];
    const float c = to_f32(proj[(size_t)t * 3 * hidden + hidden + ch]);
    y[(size_t)t * hidden + ch] = from_f32<AT>(c * acc);
}

// bfloat16 rows, eight channels per thread (hidden a multiple of 8): 16-byte loads of b, c and x.
// Per channel the arithmetic and its order are those of the kernel above.
__global__ void short_conv_out_vec_kernel(const __nv_bfloat16* proj, const float* w, const float* bias,
                                          const float* state, long long slot_stride, const int* seq_of_token,
                                          const int* q_start, const int* slots, __nv_bfloat16* y, int hidden, int taps) {
    pdl_begin();
    const int t = blockIdx.x;
    const int ch = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (ch >= hidden) return;
    const int s = seq_of_token[t];
    const int first = q_start[s];
    const float* state_row = state + (size_t)slots[s] * slot_stride;
    const int rel_now = t - first;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int rel = rel_now - (taps - 1) + j;
        float u[8];
        if (rel >= 0) {
            const __nv_bfloat16* row = proj + (size_t)(first + rel) * 3 * hidden;
            const uint4 braw = *reinterpret_cast<const uint4*>(row + ch);
            const uint4 xraw = *reinterpret_cast<const uint4*>(row + 2 * hidden + ch);
            const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&braw);
            const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xraw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 b = __bfloat1622float2(bp[e]), x = __bfloat1622float2(xp[e]);
                u[2 * e] = b.x * x.x;
                u[2 * e + 1] = b.y * x.y;
            }
        } else {
            const float* sr = state_row + (size_t)(taps - 1 + rel) * hidden + ch;
            const float4 lo = *reinterpret_cast<const float4*>(sr), hi = *reinterpret_cast<const float4*>(sr + 4);
            u[0] = lo.x; u[1] = lo.y; u[2] = lo.z; u[3] = lo.w;
            u[4] = hi.x; u[5] = hi.y; u[6] = hi.z; u[7] = hi.w;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(w[(size_t)(ch + e) * taps + j], u[e], acc[e]);
    }
    const uint4 craw = *reinterpret_cast<const uint4*>(proj + (size_t)t * 3 * hidden + hidden + ch);
    const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&craw);
    uint4 oraw;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 c = __bfloat1622float2(cp[e]);
        float a0 = acc[2 * e], a1 = acc[2 * e + 1];
        if (bias) {
            a0 += bias[ch + 2 * e];
            a1 += bias[ch + 2 * e + 1];
        }
        op[e] = __floats2bfloat162_rn(c.x * a0, c.y * a1);
    }
    *reinterpret_cast<uint4*>(y + (size_t)t * hidden + ch) = oraw;
}

// For long portions: a thread owns eight channels and walks RUN consecutive rows with the
// window of gated inputs in registers, so every row of b, c and x is read once (the kernel
// above reads b and x once per tap) and the weights once per thread.  When the walk crosses
// into another sequence, or starts, the window is refilled from the rows or the state behind
// it.  Per channel the sum is the same fused multiply-adds in the same order as above.
constexpr int RUN = 16;

__device__ __forceinline__ void gated8(const uint4& braw, const uint4& xraw, float* u) {
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&braw);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xraw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 b = __bfloat1622float2(bp[e]), x = __bfloat1622float2(xp[e]);
        u[2 * e] = b.x * x.x;
        u[2 * e + 1] = b.y * x.y;
    }
}

template <int TAPS>
__global__ void __launch_bounds__(128)
short_conv_run_kernel(const __nv_bfloat16* proj, const float* __restrict__ w, const float* __restrict__ bias,
                      const float* state, long long slot_stride, const int* __restrict__ seq_of_token,
                      const int* __restrict__ q_start, const int* __restrict__ slots, __nv_bfloat16* y,
                      int hidden, int tokens) {
    pdl_begin();
    const int ch = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (ch >= hidden) return;
    const int t0 = blockIdx.x * RUN, t1 = min(tokens, t0 + RUN);
    float wr[TAPS][8], br[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[j][e] = w[(size_t)(ch + e) * TAPS + j];
        br[e] = bias ? bias[ch + e] : 0.0f;
    }
    float win[TAPS - 1][8];
    int cur_seq = -1;
    // The rows just before the run usually belong to the same sequence: they and their sequence
    // numbers are asked for together with the first rows, and when the numbers agree the window is
    // made of them; otherwise it is refilled below, two dependent lookups later.
    uint4 before_b[TAPS - 1], before_x[TAPS - 1];
    int before_seq[TAPS - 1];
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {
        const int t = t0 - (TAPS - 1) + j;
        before_seq[j] = t >= 0 ? seq_of_token[t] : -1;
        const __nv_bfloat16* row = proj + (size_t)(t >= 0 ? t : 0) * 3 * hidden + ch;
        before_b[j] = *reinterpret_cast<const uint4*>(row);
        before_x[j] = *reinterpret_cast<const uint4*>(row + 2 * hidden);
    }
    constexpr int AHEAD = 8;  // rows whose loads are in flight together
    for (int tb = t0; tb < t1; tb += AHEAD) {
        uint4 braw[AHEAD], craw[AHEAD], xraw[AHEAD];
        int seq_of[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const int t = min(tb + i, t1 - 1);
            seq_of[i] = seq_of_token[t];
            const __nv_bfloat16* row = proj + (size_t)t * 3 * hidden + ch;
            braw[i] = *reinterpret_cast<const uint4*>(row);
            craw[i] = *reinterpret_cast<const uint4*>(row + hidden);
            xraw[i] = *reinterpret_cast<const uint4*>(row + 2 * hidden);
        }
        if (tb == t0) {
            bool same = true;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) same = same && before_seq[j] == seq_of[0];
            if (same) {
                cur_seq = seq_of[0];
#pragma unroll
                for (int j = 0; j < TAPS - 1; ++j) gated8(before_b[j], before_x[j], win[j]);
            }
        }
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const int t = tb + i;
            if (t >= t1) break;
            const int s = seq_of[i];
            if (s != cur_seq) {
                cur_seq = s;
                const int first = q_start[s];
                const float* state_row = state + (size_t)slots[s] * slot_stride;
#pragma unroll
                for (int j = 0; j < TAPS - 1; ++j) {
                    const int rel = t - first - (TAPS - 1) + j;
                    if (rel >= 0) {
                        const __nv_bfloat16* row = proj + (size_t)(first + rel) * 3 * hidden + ch;
                        gated8(*reinterpret_cast<const uint4*>(row), *reinterpret_cast<const uint4*>(row + 2 * hidden), win[j]);
                    } else {
                        const float* sr = state_row + (size_t)(TAPS - 1 + rel) * hidden + ch;
                        const float4 lo = *reinterpret_cast<const float4*>(sr), hi = *reinterpret_cast<const float4*>(sr + 4);
                        win[j][0] = lo.x; win[j][1] = lo.y; win[j][2] = lo.z; win[j][3] = lo.w;
                        win[j][4] = hi.x; win[j][5] = hi.y; win[j][6] = hi.z; win[j][7] = hi.w;
                    }
                }
            }
            float u[8], acc[8];
            gated8(braw[i], xraw[i], u);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                acc[e] = 0.0f;
#pragma unroll
                for (int j = 0; j < TAPS - 1; ++j) acc[e] = fmaf(wr[j][e], win[j][e], acc[e]);
                acc[e] = fmaf(wr[TAPS - 1][e], u[e], acc[e]);
            }
            const __nv_bfloat162* cp = reinterpret_cast<const __nv_bfloat162*>(&craw[i]);
            uint4 oraw;
            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&oraw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 c = __bfloat1622float2(cp[e]);
                float a0 = acc[2 * e], a1 = acc[2 * e + 1];
                if (bias) {
                    a0 += br[2 * e];
                    a1 += br[2 * e + 1];
                }
                op[e] = __floats2bfloat162_rn(c.x * a0, c.y * a1);
            }
            *reinterpret_cast<uint4*>(y + (size_t)t * hidden + ch) = oraw;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
#pragma unroll
                for (int j = 0; j < TAPS - 2; ++j) win[j][e] = win[j + 1][e];
                win[TAPS - 2][e] = u[e];
            }
        }
    }
}

// New state = the last taps-1 values of (old state ++ this step's u).  One thread owns a
// (sequence, channel) pair and reads everything it needs before it writes.
template <typename AT>
__global__ void short_conv_state_kernel(const AT* __restrict__ proj, float* __restrict__ state,
                                        long long slot_stride, const int* __restrict__ q_start,
                                        const int* __restrict__ slots, int hidden, int taps) {
    pdl_begin();
    const int s = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (ch >= hidden) return;
    const int first = q_start[s];
    const int n = q_start[s + 1] - first;
    float* state_row = state + (size_t)slots[s] * slot_stride;
    float next[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int rel = n - (taps - 1) + j;
            next[j] = gated_input(proj, state_row, first, rel, ch, hidden, taps, hidden);
        }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
        if (j < taps - 1) state_row[(size_t)j * hidden + ch] = next[j];
}

// Both in one launch for steps whose sequences bring only a few rows (decode): one thread owns a
// (sequence, channel) pair, keeps the window of gated inputs in registers and walks the
// sequence's rows in order, as the reference's kernel does for a whole portion
// (kernels/metal/dense/dense_short_conv.metal:45-67).  Nothing else touches that pair's
// state, so reading and rewriting it in one kernel is safe.
template <typename AT>
__global__ void short_conv_serial_kernel(const AT* __restrict__ proj, const float* __restrict__ w,
                                         const float* __restrict__ bias, float* __restrict__ state,
                                         long long slot_stride, const int* __restrict__ q_start,
                                         const int* __restrict__ slots, AT* __restrict__ y, int hidden, int taps) {
    pdl_begin();
    const int s = blockIdx.x;
    const int ch = blockIdx.y * blockDim.x + threadIdx.x;
    if (ch >= hidden) return;
    const int first = q_start[s];
    const int n = q_start[s + 1] - first;
    float* state_row = state + (size_t)slots[s] * slot_stride;
    float window[MAX_TAPS], weight[MAX_TAPS];
#pragma unroll
    for (int j = 0; j < MAX_TAPS; ++j) {
        weight[j] = j < taps ? w[(size_t)ch * taps + j] : 0.0f;
        window[j] = j < taps - 1 ? state_row[(size_t)j * hidden + ch] : 0.0f;
    }
    const float b = bias ? bias[ch] : 0.0f;
    for (int i = 0; i < n; ++i) {
        const AT* row = proj + (size_t)(first + i) * 3 * hidden;
        const float u = to_f32(row[ch]) * to_f32(row[2 * hidden + ch]);
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j < taps) {
                const float v = j == taps - 1 ? u : window[j];
                acc = fmaf(weight[j], v, acc);
            }
        }
        y[(size_t)(first + i) * hidden + ch] = from_f32<AT>(to_f32(row[hidden + ch]) * (acc + b));
#pragma unroll
        for (int j = 0; j < MAX_TAPS - 1; ++j) {
            if (j < taps - 1) window[j] = j == taps - 2 ? u : window[j + 1];
        }
    }
#pragma unroll
    for (int j = 0; j < MAX_TAPS - 1; ++j)
        if (j < taps - 1) state_row[(size_t)j * hidden + ch] = window[j];
}

}  // namespace

// state: float [slots, taps-1, hidden] with `slot_stride` floats between slots (the rows
// of one slot are contiguous).
SHISO_API int shiso_short_conv(const void* proj, int act_dtype, const float* w, const float* bias, float* state,
                               long long slot_stride, const int* seq_of_token, const int* q_start,
                               const int* slots, void* y, int tokens, int seqs, int hidden, int taps,
                               int update_state, int max_rows_per_seq, cudaStream_t stream) {
    if (tokens <= 0 || seqs <= 0) return SHISO_OK;
    if (taps < 2 || taps > MAX_TAPS) return SHISO_ERR_SHAPE;
    const int threads = 128;
    if (update_state && max_rows_per_seq > 0 && max_rows_per_seq <= 4) {
        dim3 grid(seqs, ceil_div_u(hidden, threads));
        if (act_dtype == SHISO_F32)
            launch_kernel(short_conv_serial_kernel<float>, grid, threads, 0, stream, 
                (const float*)proj, w, bias, state, slot_stride, q_start, slots, (float*)y, hidden, taps);
        else if (act_dtype == SHISO_BF16)
            launch_kernel(short_conv_serial_kernel<__nv_bfloat16>, grid, threads, 0, stream, 
                (const __nv_bfloat16*)proj, w, bias, state, slot_stride, q_start, slots, (__nv_bfloat16*)y, hidden, taps);
        else
            return SHISO_ERR_DTYPE;
        return launch_status();
    }
    dim3 grid_out(tokens, ceil_div_u(hidden, threads));
    dim3 grid_state(seqs, ceil_div_u(hidden, threads));
    if (act_dtype == SHISO_F32) {
        launch_kernel(short_conv_out_kernel<float>, grid_out, threads, 0, stream, 
            (const float*)proj, w, bias, state, slot_stride, seq_of_token, q_start, slots, (float*)y, hidden, taps);
        if (update_state)
            launch_kernel(short_conv_state_kernel<float>, grid_state, threads, 0, stream, 
                (const float*)proj, state, slot_stride, q_start, slots, hidden, taps);
    } else if (act_dtype == SHISO_BF16) {
        const bool vec = hidden % 8 == 0 && slot_stride % 4 == 0 &&
                         (((uintptr_t)proj | (uintptr_t)y | (uintptr_t)state) & 15) == 0;
        const bool runs = vec && tokens >= 512 && taps >= 2 && taps <= 4;
        if (runs) {
            dim3 grid_run(ceil_div_u(tokens, RUN), ceil_div_u(hidden / 8, threads));
            auto launch_run = [&](auto kernel) {
                launch_kernel(kernel, grid_run, threads, 0, stream, (const __nv_bfloat16*)proj, w, bias,
                              (const float*)state, slot_stride, seq_of_token, q_start, slots, (__nv_bfloat16*)y, hidden, tokens);
            };
            if (taps == 2) launch_run(short_conv_run_kernel<2>);
            else if (taps == 3) launch_run(short_conv_run_kernel<3>);
            else launch_run(short_conv_run_kernel<4>);
        } else if (vec) {
            launch_kernel(short_conv_out_vec_kernel, dim3(tokens, ceil_div_u(hidden / 8, threads)), threads, 0, stream,
                          (const __nv_bfloat16*)proj, w, bias, (const float*)state, slot_stride, seq_of_token, q_start,
                          slots, (__nv_bfloat16*)y, hidden, taps);
        } else
        launch_kernel(short_conv_out_kernel<__nv_bfloat16>, grid_out, threads, 0, stream, 
            (const __nv_bfloat16*)proj, w, bias, state, slot_stride, seq_of_token, q_start, slots,
            (__nv_bfloat16*)y, hidden, taps);
        if (update_state)
            launch_kernel(short_conv_state_kernel<__nv_bfloat16>, grid_state, threads, 0, stream, 
                (const __nv_bfloat16*)proj, state, slot_stride, q_start, slots, hidden, taps);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}
