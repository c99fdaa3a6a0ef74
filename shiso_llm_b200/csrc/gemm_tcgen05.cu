// Y[T, N] = X[T, K] * W[N, K]^T for bfloat16 operands on the 5th-generation tensor cores.
//
// Layout of the work ("swap-AB"): the weight tile is the MMA's M operand (128 output
// features x 64 k per stage) and the token tile is its N operand (BN tokens x 64 k, BN =
// 16 .. 256), so one kernel serves a decode step (8 tokens: a 128 x 16 tile that streams
// the weights once) and a prompt portion (2,048 tokens: 128 x 256 tiles).  Both operands
// are K-major in shared memory, brought there by TMA with the 128-byte swizzle; the
// accumulator D[feature, token] lives in tensor memory (TMEM, 128 lanes x BN columns of
// float) and is read back with tcgen05.ld for the epilogue.  No multicast is used.
//
// Roles inside a CTA of 128 threads: lane 0 of warp 0 issues the TMA loads, lane 0 of warp 1
// issues tcgen05.mma and commits; all four warps run the epilogue (warp q owns TMEM lanes
// 32q .. 32q+31, i.e. features).  Stages are handed back and forth with mbarriers: `full`
// (TMA bytes landed) and `empty` (tcgen05.commit: the MMAs that read the stage are done).
//
// Small token counts leave too few feature tiles to fill 148 SMs, so the K dimension is split
// over a thread-block cluster of 2 to 8 CTAs, chosen so that the grid is one wave (48 feature
// tiles: 3 CTAs each).  Token j of the tile is summed by the CTA of rank j % size: every CTA
// pushes its partial values into that CTA's shared memory (remote stores into an inbox behind
// the stages), the cluster meets once, and each CTA adds up what it was sent in rank order, so
// the result does not depend on timing.  With a gate/up pair both accumulators travel and the
// summing CTA applies the activation.  (Clock stamps showed where the first version's 18 us for
// 64 tokens x 6144 x 2048 went: 4.7 us in the main loop, 3.6 us in a reduction that pulled its
// terms with remote loads between two cluster barriers, and 9 us outside the CTA's own timeline -
// a 176 KB CTA leaves no room for the next kernel's CTAs to start under its tail.  Three stages
// and the push took it to 9.3 us.)
//
// Every wait is bounded by a clock limit; a wait that runs out sets a status word that the
// host reads, frees the TMEM it holds and returns.
//
// The reference runs its prompt products through a scalar tile kernel or a dequantised
// plane and a vendor SGEMM in 256-token bands (crates/shiso-engine/src/projection.rs:949-1070,
// 1297-1304) and its decode products through matvec kernels (projection.rs:972-1069).
#include <cooperative_groups.h>

#include <type_traits>

#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace {

using namespace tc;

constexpr int THREADS = 128;

struct GemmParams {
    void* y;
    const float* bias;      // per output feature, or null
    int* status;            // set non-zero when a wait ran out
    int T, N, K;
    int k_blocks_per_split;  // BK-blocks each CTA of a cluster handles
    int out_f32;             // 1: float output, 0: bfloat16
    int inter;               // GLU kernels: rows of the gate (and of the up) matrix, and of the output
    // SCALED (scale_partials != null): the rows of x lack their RMS scale; token t's is
    // rsqrt(sum over c < scale_count of scale_partials[c * scale_stride + t] / K + scale_eps) and
    // multiplies the accumulators of its column.
    const float* scale_partials;
    int scale_count, scale_stride;
    float scale_eps;
    // INTO (res_in != null; plain products): res_out = res_in + product (+ bias), x_out =
    // bf16(res_out * norm_w) and into_partials[feature tile * T + t] = the sum of res_out^2 over
    // the tile's 128 features - the input of a SCALED product; y is not written.
    const float* res_in;
    float* res_out;
    const float* norm_w;
    __nv_bfloat16* x_out;
    float* into_partials;
    // rows of `y`, the stream, the bias and the norm weight may be read and written four features
    // at a time (their width is a multiple of 4 and their pointers are 16-byte aligned)
    int vec4;
};

constexpr int MAX_FUSED_BN = 64;  // token tiles of the SCALED / INTO modes (their scales lie in shared memory)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename OT>
__device__ __forceinline__ void store_out(OT* y, size_t at, float v);
template <> __device__ __forceinline__ void store_out<float>(float* y, size_t at, float v) { y[at] = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* y, size_t at, float v) { y[at] = __float2bfloat16_rn(v); }

// GLU: the weight is a [2 * inter, K] gate-over-up pair.  A CTA then loads the gate rows and
// the matching up rows of its 128 features, keeps two accumulators in TMEM (columns 0..BN-1
// and BN..2BN-1), and its epilogue writes silu(gate) * up - the token tile is read once for
// 256 weight rows and the [T, 2 * inter] intermediate never exists.
// (up to 64 tokens a CTA takes under half of an SM's shared memory, so that the CTAs of the next
// product in a chain of dependent launches can move in and start their loads under this one's tail)
template <int BN, int STAGES, int SPLITS, bool GLU>
__global__ void __launch_bounds__(THREADS, (BN <= 64 && !GLU) ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    constexpr int A_BYTES = BM * BK * 2;
    constexpr int A_TILES = GLU ? 2 : 1;
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_TILES * A_BYTES + B_BYTES;
    constexpr int ACC_COLS = A_TILES * BN;
    constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;  // a power of two >= 32

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // with K split over a cluster, an inbox for the partial sums the other CTAs push stands behind
    // the stages (not over them: a peer may push while this CTA's own loads are still landing)
    constexpr int INBOX_BYTES = SPLITS > 1 ? A_TILES * SPLITS * ((BN + SPLITS - 1) / SPLITS) * BM * 4 : 0;
    uint64_t* full = (uint64_t*)(smem + STAGES * STAGE_BYTES + INBOX_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum_bar = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum_bar + 1);
    int* failed = (int*)(tmem_slot + 1);
    float* scale_s = (float*)(failed + 1);  // [min(BN, MAX_FUSED_BN)] row scales of the SCALED mode
    float* square_s = scale_s + MAX_FUSED_BN;  // [4 warps][MAX_FUSED_BN] sums of squares of the INTO mode

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feature0 = blockIdx.x * BM;
    const int token0 = blockIdx.y * BN;
    const int split = SPLITS > 1 ? (int)blockIdx.z : 0;
    const int total_kb = (p.K + BK - 1) / BK;
    const int kb_begin = split * p.k_blocks_per_split;
    int kb_count = total_kb - kb_begin;
    if (kb_count > p.k_blocks_per_split) kb_count = p.k_blocks_per_split;
    if (kb_count < 0) kb_count = 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum_bar, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int feature = feature0 + warp * 32 + lane;
    const bool scaled = p.scale_partials != nullptr;
    const bool into = !GLU && p.res_in != nullptr;
    // INTO: what the epilogue needs from global memory is asked for under the main loop - the
    // norm weight and the stream's values of this CTA's first tokens (tokens first_own,
    // first_own + own_stride, ... of the tile).  The two lanes that run the main loop ask when
    // it suits them: the producer after its last load, the MMA issuer before its first MMA
    // (its operands cannot land before the predecessor is done either).
    constexpr int EARLY = 8;
    const int own_stride = SPLITS > 1 ? SPLITS : 1;
    int first_own = 0;
    if constexpr (SPLITS > 1) first_own = (int)cg::this_cluster().block_rank();
    float norm_weight = 0.0f;
    float early[EARLY];
    auto stream_value = [&](int token) {
        return (feature < p.N && token < p.T) ? p.res_in[(size_t)token * p.N + feature] : 0.0f;
    };
    // (Rows of a width that is no multiple of 4, or pointers off a 16-byte boundary, take the same
    // path with one element per load and store: p.vec4.)
    // With K split over a cluster the sums are finished by other threads than own the accumulator
    // rows: a warp takes tokens warp, warp + 4, .. of its CTA's share, a lane four consecutive
    // features of the tile (16-byte loads of the partial sums, one warp-wide sum of squares a token).
    constexpr int EARLY4 = 2;
    const int feature4 = feature0 + 4 * lane;
    float4 norm_weight4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 early4[EARLY4];
    // four consecutive floats from `limit`-wide rows; past the row's end zeros
    auto load4 = [&](const float* base, size_t row_offset, int first, int limit) {
        float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (p.vec4) {
            if (first < limit) r = *reinterpret_cast<const float4*>(base + row_offset + first);
        } else {
            if (first < limit) r.x = base[row_offset + first];
            if (first + 1 < limit) r.y = base[row_offset + first + 1];
            if (first + 2 < limit) r.z = base[row_offset + first + 2];
            if (first + 3 < limit) r.w = base[row_offset + first + 3];
        }
        return r;
    };
    auto stream_value4 = [&](int token) {
        return token < p.T ? load4(p.res_in, (size_t)token * p.N, feature4, p.N) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    };
    auto ask_early = [&]() {
        if (!into) return;
        pdl_wait();  // the stream is the predecessor's
        if constexpr (SPLITS > 1) {
            norm_weight4 = load4(p.norm_w, 0, feature4, p.N);
#pragma unroll
            for (int u = 0; u < EARLY4; ++u) early4[u] = stream_value4(token0 + (warp + 4 * u) * SPLITS + first_own);
        } else {
            norm_weight = feature < p.N ? p.norm_w[feature] : 0.0f;
#pragma unroll
            for (int u = 0; u < EARLY; ++u) early[u] = stream_value(token0 + first_own + u * own_stride);
        }
    };

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads, one stage per 64-wide k block.  Weights depend on no
        // predecessor, the activations do: the weights of every stage of the ring are asked for
        // before the dependency wait, so that they travel under the predecessor's tail.
        auto load_weights = [&](int i) {
            uint8_t* a = smem + (i % STAGES) * STAGE_BYTES;
            mbar_expect_tx(&full[i % STAGES], STAGE_BYTES);
            const int k = (kb_begin + i) * BK;
            tma_load_2d(a, &map_w, k, feature0, &full[i % STAGES]);
            if (GLU) tma_load_2d(a + A_BYTES, &map_w, k, p.inter + feature0, &full[i % STAGES]);
        };
        auto load_tokens = [&](int i) {
            tma_load_2d(smem + (i % STAGES) * STAGE_BYTES + A_TILES * A_BYTES, &map_x, (kb_begin + i) * BK, token0, &full[i % STAGES]);
        };
        const int ahead = kb_count < STAGES ? kb_count : STAGES;
        for (int i = 0; i < ahead; ++i) load_weights(i);
        pdl_wait();
        for (int i = 0; i < ahead; ++i) load_tokens(i);
        for (int i = ahead; i < kb_count; ++i) {
            if (!mbar_wait(&empty[i % STAGES], ((i / STAGES) - 1) & 1)) {
                *failed = 1;
                break;
            }
            load_weights(i);
            load_tokens(i);
        }
        ask_early();
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        ask_early();
        const uint32_t idesc = umma_idesc(BM, BN);
        bool ok = true;
        for (int i = 0; i < kb_count && ok; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(&full[s], (i / STAGES) & 1)) {
                *failed = 1;
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
            const uint32_t b_addr = a_addr + A_TILES * A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t a_desc = umma_desc(a_addr + k * UMMA_K * 2);
                const uint64_t b_desc = umma_desc(b_addr + k * UMMA_K * 2);
                umma_bf16(tmem_base, a_desc, b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                if (GLU) {
                    const uint64_t up_desc = umma_desc(a_addr + A_BYTES + k * UMMA_K * 2);
                    umma_bf16(tmem_base + BN, up_desc, b_desc, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
            }
            umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
        }
        umma_commit(accum_bar);      // the accumulator is complete once every MMA is done
    } else {
        ask_early();
    }
    if (warp >= 2 && scaled) {
        // ---- the row scales, while the main loop runs (the sums of squares are the predecessor's)
        pdl_wait();
        for (int j = threadIdx.x - 64; j < BN && j < MAX_FUSED_BN; j += 64) {
            float sum = 0.0f;
            if (token0 + j < p.T) {
                const float* mine = p.scale_partials + token0 + j;
                int c = 0;
                for (; c + 8 <= p.scale_count; c += 8) {  // eight loads in flight, added in index order
                    float part[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) part[u] = mine[(size_t)(c + u) * p.scale_stride];
#pragma unroll
                    for (int u = 0; u < 8; ++u) sum += part[u];
                }
                for (; c < p.scale_count; ++c) sum += mine[(size_t)c * p.scale_stride];
            }
            scale_s[j] = rsqrtf(sum / (float)p.K + p.scale_eps);
        }
    }
    __syncwarp();

    // ---- epilogue: every thread owns one feature (TMEM lane), columns are tokens
    pdl_wait();  // nothing is written before the predecessor has finished
    bool ready = true;
    if (kb_count > 0) ready = mbar_wait(accum_bar, 0);
    if (!ready) *failed = 1;
    pdl_trigger();  // the main loop is over: the successor may be scheduled while the epilogue runs
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool bad = *failed != 0;
    if (bad && threadIdx.x == 0 && p.status) atomicExch(p.status, 1);

    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    // INTO: one token's value of this thread's feature joins the stream; all lanes of the warp
    // call it together (the sum of squares is taken over the warp's 32 features)
    auto join_stream = [&](int token, float v, float before) {
        float r = 0.0f;
        if (feature < p.N && token < p.T) {
            const size_t at = (size_t)token * p.N + feature;
            r = before + v;
            p.res_out[at] = r;
            p.x_out[at] = __float2bfloat16_rn(r * norm_weight);
        }
        const float square = warp_sum(r * r);
        if (lane == 0) square_s[warp * MAX_FUSED_BN + (token - token0) % MAX_FUSED_BN] = square;
    };
    // after the tokens of this CTA have joined: the four warps' sums of squares, added in warp order
    auto leave_squares = [&](int stride, int first) {  // this CTA's tokens of the tile: first, first + stride, ...
        __syncthreads();
        for (int j = first + (int)threadIdx.x * stride; j < BN && j < MAX_FUSED_BN; j += THREADS * stride) {
            if (token0 + j >= p.T) break;
            const float sum = square_s[j] + square_s[MAX_FUSED_BN + j] + square_s[2 * MAX_FUSED_BN + j] + square_s[3 * MAX_FUSED_BN + j];
            p.into_partials[(size_t)blockIdx.x * p.T + token0 + j] = sum;
        }
    };

    if constexpr (GLU && SPLITS == 1) {
        if (!bad) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                float gate[8], up[8];  // the loads are warp-wide; rows past `inter` are dropped at the store
                tmem_ld8(lane_addr + c, gate);
                tmem_ld8(lane_addr + BN + c, up);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int token = token0 + c + j;
                    if (token < p.T && feature < p.inter) {
                        if (scaled) {
                            const float sc = scale_s[(c + j) % MAX_FUSED_BN];
                            gate[j] *= sc;
                            up[j] *= sc;
                        }
                        const float v = silu_times(gate[j], up[j]);
                        const size_t at = (size_t)token * p.inter + feature;
                        if (p.out_f32) store_out<float>((float*)p.y, at, v);
                        else store_out<__nv_bfloat16>((__nv_bfloat16*)p.y, at, v);
                    }
                }
            }
        }
    } else if constexpr (SPLITS == 1) {
        if (!bad) {
            const float b = (p.bias && feature < p.N) ? p.bias[feature] : 0.0f;
#pragma unroll 1
            for (int c = 0; c < BN; c += 8) {
                float v[8];
                if (kb_count > 0) {
                    tmem_ld8(lane_addr + c, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                }
                if (scaled) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] *= scale_s[(c + j) % MAX_FUSED_BN];
                }
                if (into) {
                    float before[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) before[j] = c == 0 ? early[j] : stream_value(token0 + c + j);
#pragma unroll
                    for (int j = 0; j < 8; ++j) join_stream(token0 + c + j, v[j] + b, before[j]);
                } else if (feature < p.N) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int token = token0 + c + j;
                        if (token < p.T) {
                            const size_t at = (size_t)token * p.N + feature;
                            if (p.out_f32) store_out<float>((float*)p.y, at, v[j] + b);
                            else store_out<__nv_bfloat16>((__nv_bfloat16*)p.y, at, v[j] + b);
                        }
                    }
                }
            }
            if (into) leave_squares(1, 0);  // `bad` and `into` are the same in every thread
        }
    } else {
        // Token j is summed by the CTA of rank j % SPLITS.  Every CTA pushes its partial values
        // into the shared memory of the CTA that sums them (remote stores), the cluster meets
        // once, and each CTA adds up what it was sent in rank order: no remote loads, and nobody
        // reads a CTA's memory after the meeting, so a CTA may leave as soon as it is done.
        cg::cluster_group cluster = cg::this_cluster();
        // With a gate/up pair both accumulators travel, and the CTA that has the sums applies
        // the activation.
        constexpr int OWN = (BN + SPLITS - 1) / SPLITS;  // tokens a CTA sums
        float* inbox = (float*)(smem + STAGES * STAGE_BYTES);  // [A_TILES][SPLITS][OWN][BM]
        const unsigned rank = cluster.block_rank();
        float* target[SPLITS];
#pragma unroll
        for (int r = 0; r < SPLITS; ++r) target[r] = cluster.map_shared_rank(inbox, r) + (size_t)rank * OWN * BM;
#pragma unroll
        for (int t = 0; t < A_TILES; ++t) {
#pragma unroll
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (kb_count > 0 && !bad) {
                    tmem_ld16(lane_addr + t * BN + c, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    target[(c + j) % SPLITS][(size_t)t * SPLITS * OWN * BM + ((c + j) / SPLITS) * BM + warp * 32 + lane] = v[j];
            }
        }
        cluster.sync();
        const int out_rows = GLU ? p.inter : p.N;
        // Token `i` of this CTA's share (i = warp, warp + 4, ..), four features a lane; `pair` of
        // them at a time, all their partial sums asked for before the first is used.  False past
        // the share, the tile or the step (the same in every lane of the warp).
        const bool live4 = feature4 < out_rows;
        float4 bias4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (!GLU && p.bias) bias4 = load4(p.bias, 0, feature4, out_rows);
        const float4* inbox4 = reinterpret_cast<const float4*>(inbox);
        // four values at `at` = row start + feature4 of `limit`-wide rows
        auto store4_f32 = [&](float* base, size_t at, float4 v, int limit) {
            if (p.vec4) {
                *reinterpret_cast<float4*>(base + at) = v;
            } else {
                base[at] = v.x;
                if (feature4 + 1 < limit) base[at + 1] = v.y;
                if (feature4 + 2 < limit) base[at + 2] = v.z;
                if (feature4 + 3 < limit) base[at + 3] = v.w;
            }
        };
        auto store4_bf16 = [&](__nv_bfloat16* base, size_t at, float4 v, int limit) {
            if (p.vec4) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                *reinterpret_cast<uint2*>(base + at) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
                base[at] = __float2bfloat16_rn(v.x);
                if (feature4 + 1 < limit) base[at + 1] = __float2bfloat16_rn(v.y);
                if (feature4 + 2 < limit) base[at + 2] = __float2bfloat16_rn(v.z);
                if (feature4 + 3 < limit) base[at + 3] = __float2bfloat16_rn(v.w);
            }
        };
        auto finish_pair = [&](int u0, const float4* before) {
            float4 part[2][A_TILES][SPLITS];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = warp + 4 * (u0 + u);
#pragma unroll
                for (int t = 0; t < A_TILES; ++t)
#pragma unroll
                    for (int r = 0; r < SPLITS; ++r)
                        part[u][t][r] = i < OWN ? inbox4[((((size_t)t * SPLITS + r) * OWN + i) * BM) / 4 + lane] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int i = warp + 4 * (u0 + u);
                const int j = i * SPLITS + (int)rank;
                if (i >= OWN || j >= BN || token0 + j >= p.T) return false;
                const int token = token0 + j;
                float4 sum[A_TILES];
#pragma unroll
                for (int t = 0; t < A_TILES; ++t) {
                    sum[t] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int r = 0; r < SPLITS; ++r) {  // rank order
                        sum[t].x += part[u][t][r].x;
                        sum[t].y += part[u][t][r].y;
                        sum[t].z += part[u][t][r].z;
                        sum[t].w += part[u][t][r].w;
                    }
                    if (scaled) {
                        const float sc = scale_s[j % MAX_FUSED_BN];
                        sum[t].x *= sc; sum[t].y *= sc; sum[t].z *= sc; sum[t].w *= sc;
                    }
                }
                float4 v;
                if (GLU) {
                    v = make_float4(silu_times(sum[0].x, sum[A_TILES - 1].x), silu_times(sum[0].y, sum[A_TILES - 1].y),
                                    silu_times(sum[0].z, sum[A_TILES - 1].z), silu_times(sum[0].w, sum[A_TILES - 1].w));
                } else {
                    v = make_float4(sum[0].x + bias4.x, sum[0].y + bias4.y, sum[0].z + bias4.z, sum[0].w + bias4.w);
                }
                if (into) {
                    float4 r4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (live4) {
                        const size_t at = (size_t)token * p.N + feature4;
                        r4 = make_float4(before[u].x + v.x, before[u].y + v.y, before[u].z + v.z, before[u].w + v.w);
                        // (features past the row's end: v and the stream's value are zero there)
                        store4_f32(p.res_out, at, r4, p.N);
                        store4_bf16(p.x_out, at, make_float4(r4.x * norm_weight4.x, r4.y * norm_weight4.y, r4.z * norm_weight4.z, r4.w * norm_weight4.w), p.N);
                    }
                    // the token's sum of squares over the tile's 128 features: one warp has them all
                    const float square = warp_sum((r4.x * r4.x + r4.y * r4.y) + (r4.z * r4.z + r4.w * r4.w));
                    if (lane == 0) p.into_partials[(size_t)blockIdx.x * p.T + token] = square;
                } else if (live4) {
                    const size_t at = (size_t)token * out_rows + feature4;
                    if (p.out_f32) store4_f32((float*)p.y, at, v, out_rows);
                    else store4_bf16((__nv_bfloat16*)p.y, at, v, out_rows);
                }
            }
            return true;
        };
        constexpr int PER_WARP = (OWN + 3) / 4;  // tokens a warp may have to finish
        bool more = finish_pair(0, early4);      // (EARLY4 == 2: the first pair's stream values are here)
        for (int u0 = 2; u0 < PER_WARP && more; u0 += 2) {
            float4 before[2];
#pragma unroll
            for (int u = 0; u < 2; ++u)
                before[u] = into ? stream_value4(token0 + (warp + 4 * (u0 + u)) * SPLITS + (int)rank) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            more = finish_pair(u0, before);
        }

    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------- host side

constexpr int SPLIT_STAGES = 6, WHOLE_STAGES = 8;  // wanted; see fit_stages

// Stages of a CTA: for plain products as many (up to `wanted`) as leave room for a second CTA on
// the SM, for gate/up pairs, whose CTA has an SM to itself anyway, as many as fit.
constexpr int fit_stages(int wanted, int bn, int splits, bool glu) {
    const int stage = (glu ? 2 : 1) * BM * BK * 2 + bn * BK * 2;
    const int inbox = splits > 1 ? (glu ? 2 : 1) * splits * ((bn + splits - 1) / splits) * BM * 4 : 0;
    const int room = glu ? 227 * 1024 : 113 * 1024;
    int stages = wanted;
    while (stages > 3 && stages * stage + inbox + 2560 > room) --stages;
    return stages;
}

template <int BN, int WANTED_STAGES, int SPLITS, bool GLU = false>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, GemmParams p, cudaStream_t stream) {
    constexpr int STAGES = fit_stages(WANTED_STAGES, BN, SPLITS, GLU);
    constexpr int STAGE_BYTES = (GLU ? 2 : 1) * BM * BK * 2 + BN * BK * 2;
    constexpr int PARTIAL_BYTES = SPLITS > 1 ? (GLU ? 2 : 1) * SPLITS * ((BN + SPLITS - 1) / SPLITS) * BM * 4 : 0;
    constexpr int TILE_BYTES = STAGES * STAGE_BYTES + PARTIAL_BYTES;
    constexpr int SMEM = TILE_BYTES + 1024 /* alignment */ + 1536 /* barriers, flags, row scales, sums of squares */;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, SPLITS, GLU>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div_u(GLU ? p.inter : p.N, BM), ceil_div_u(p.T, BN), SPLITS);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = SPLITS;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = shiso_pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    {
        const int out_rows = GLU ? p.inter : p.N;
        const uintptr_t pointers = (uintptr_t)p.y | (uintptr_t)p.bias | (uintptr_t)p.res_in | (uintptr_t)p.res_out |
                                   (uintptr_t)p.norm_w | (uintptr_t)p.x_out;
        p.vec4 = (out_rows % 4 == 0 && (pointers & 15) == 0) ? 1 : 0;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, mx, p);
    return (int)e;
}

}  // namespace

int* shiso_tc_status_word() {
    static int* word = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaMalloc(&word, sizeof(int)) == cudaSuccess) cudaMemset(word, 0, sizeof(int));
        else word = nullptr;
    });
    return word;
}

// Whether the tensor-core kernel takes this problem (bfloat16 operands, rows 16-byte aligned).
SHISO_API int shiso_gemm_tcgen05_supported(int K, const void* x, const void* w) {
    if (K % 8 != 0 || K < 8) return 0;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return 0;
    return encode_fn() != nullptr ? 1 : 0;
}

// Reads and clears the status word: non-zero when a bounded wait inside a kernel ran out.
SHISO_API int shiso_gemm_tcgen05_status() {
    int* word = shiso_tc_status_word();
    if (!word) return -1;
    int host = 0;
    if (cudaMemcpy(&host, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (host) cudaMemset(word, 0, sizeof(int));
    return host;
}

// Tokens per CTA (the MMA's N operand).  Up to 192 tokens run as tiles of at most 64: such a
// CTA is under half an SM, two are resident together and the next product's CTAs start under
// this one's tail, and K is split over fewer CTAs.  Measured on a chain of the four products of
// a 2048-wide layer: 128 tokens as one tile of 128 took 87 us a layer, as two tiles of 64 60 us;
// 192 tokens as three tiles 64 us against 98 us in the kernels for long portions; from four
// token tiles on the grid is more than one wave and those kernels are faster.
static inline int token_tile(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 192 ? 64 : 256; }

namespace {

GemmParams blank_params(int T, int N, int K) {
    GemmParams p = {};
    p.status = shiso_tc_status_word();
    p.T = T;
    p.N = N;
    p.K = K;
    p.k_blocks_per_split = (K + BK - 1) / BK;
    return p;
}

int sm_count_of_device() {
    static int sm_count = 0;
    if (sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    }
    return sm_count;
}

// A plain product (p.inter == 0), with whatever epilogue mode p carries.
int run_plain(GemmParams p, const void* x, const void* w, int sm_count, cudaStream_t stream, int tile_override = 0) {
    const int T = p.T, N = p.N, K = p.K;
    const int total_kb = (K + BK - 1) / BK;
    const int bn = tile_override > 0 ? tile_override : token_tile(T);
    CUtensorMap mw, mx;
    if (!tensor_map(w, N, K, BM, &mw) || !tensor_map(x, T, K, bn, &mx)) return SHISO_ERR_UNSUPPORTED;

    if (bn == 256) return launch<256, 4, 1>(mw, mx, p, stream);
    // Few tokens: split K over a cluster so that the grid covers the SMs, up to the two CTAs that are
    // resident on each (every CTA keeps >= 2 k blocks; 48 feature tiles take 5 CTAs each, 240 CTAs:
    // decode at batch 16 / 32 / 64 gained 2.2 / 3.8 / 1.8 % over one CTA per SM).
    const int tiles = (int)ceil_div_u(N, BM) * (int)ceil_div_u(T, bn);
    // (portions of several token tiles: two CTAs are resident per SM and a long K is worth splitting
    // further - 2048 x 5632 at 576 rows: 31.2 us whole, 22.2 us in two parts, 288 CTAs - but clusters of
    // more than two on a grid near the 296 places wait for a second wave: 2,304 of K in 4 parts took
    // 12.5 us as 256 CTAs and 22.1 us as 288)
    const int room = 2 * sm_count;
    int splits = room / (tiles > 0 ? tiles : 1);
    splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
    while (splits > 2 && tiles * splits > 7 * sm_count / 4) --splits;
    while (splits > 1 && total_kb / splits < (tile_override > 0 ? 8 : 2)) --splits;
    p.k_blocks_per_split = (total_kb + splits - 1) / splits;
    // More tiles than the two CTAs an SM holds with deep rings, but no more than four an SM: rings of
    // two stages, so that every tile is resident at once instead of a second, partly empty wave
    // (the head's 512 tiles of 128 features on 148 SMs).
    const bool one_wave_of_four = splits == 1 && tiles > room && tiles <= 4 * sm_count && tile_override == 0;
#define SHISO_PICK(BN_)                                                        \
    if (one_wave_of_four) return launch<BN_, 2, 1>(mw, mx, p, stream);         \
    switch (splits) {                                                          \
        case 1: return launch<BN_, WHOLE_STAGES, 1>(mw, mx, p, stream);                   \
        case 2: return launch<BN_, SPLIT_STAGES, 2>(mw, mx, p, stream);                   \
        case 3: return launch<BN_, SPLIT_STAGES, 3>(mw, mx, p, stream);                   \
        case 4: return launch<BN_, SPLIT_STAGES, 4>(mw, mx, p, stream);                   \
        case 5: return launch<BN_, SPLIT_STAGES, 5>(mw, mx, p, stream);                   \
        case 6: return launch<BN_, SPLIT_STAGES, 6>(mw, mx, p, stream);                   \
        case 7: return launch<BN_, SPLIT_STAGES, 7>(mw, mx, p, stream);                   \
        default: return launch<BN_, SPLIT_STAGES, 8>(mw, mx, p, stream);                  \
    }
    if (bn == 16) { SHISO_PICK(16) }
    if (bn == 32) { SHISO_PICK(32) }
    SHISO_PICK(64)
#undef SHISO_PICK
}

// silu(x gate^T) * (x up^T) for w = [gate; up] of shape [2 * p.inter, K], p.N == 2 * p.inter.
int run_glu(GemmParams p, const void* x, const void* w, cudaStream_t stream) {
    const int T = p.T, K = p.K, inter = p.inter;
    const int bn = token_tile(T);
    CUtensorMap mw, mx;
    if (!tensor_map(w, 2 * inter, K, BM, &mw) || !tensor_map(x, T, K, bn, &mx)) return SHISO_ERR_UNSUPPORTED;
    if (bn == 256) return launch<256, 3, 1, true>(mw, mx, p, stream);
    // Few tokens: K split over a cluster of up to 4 CTAs, as for plain products (one wave over the SMs).
    const int sm_count = sm_count_of_device();
    const int total_kb = (K + BK - 1) / BK;
    const int tiles = (int)ceil_div_u(inter, BM) * (int)ceil_div_u(T, bn);
    int splits = sm_count / (tiles > 0 ? tiles : 1);
    splits = splits < 1 ? 1 : (splits > 4 ? 4 : splits);
    while (splits > 1 && total_kb / splits < 2) --splits;
    p.k_blocks_per_split = (total_kb + splits - 1) / splits;
#define SHISO_PICK_GLU(BN_)                                                          \
    switch (splits) {                                                                \
        case 1: return launch<BN_, WHOLE_STAGES, 1, true>(mw, mx, p, stream);                   \
        case 2: return launch<BN_, SPLIT_STAGES, 2, true>(mw, mx, p, stream);                   \
        case 3: return launch<BN_, SPLIT_STAGES, 3, true>(mw, mx, p, stream);                   \
        default: return launch<BN_, SPLIT_STAGES, 4, true>(mw, mx, p, stream);                  \
    }
    if (bn == 16) { SHISO_PICK_GLU(16) }
    if (bn == 32) { SHISO_PICK_GLU(32) }
    SHISO_PICK_GLU(64)
#undef SHISO_PICK_GLU
}

}  // namespace

// x [T, K] bf16, w [N, K] bf16, y [T, N] bf16 (y_dtype 1) or float (y_dtype 0).
SHISO_API int shiso_gemm_tcgen05(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T, int N,
                                 int K, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (!shiso_gemm_tcgen05_supported(K, x, w)) return SHISO_ERR_UNSUPPORTED;
    GemmParams p = blank_params(T, N, K);
    p.y = y;
    p.bias = bias;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    return run_plain(p, x, w, sm_count, stream);
}

// The same product with token tiles of 64 whatever T is.  For portions of a few hundred rows and a
// matrix of few rows the kernels for long portions have a handful of 256 x 256 tiles for 148 SMs
// (2,048 x 5632 at 512 rows: 16 tiles, 29.8 us measured on the 1,024-wide shape); here the same
// product is ceil(N / 128) x ceil(T / 64) CTAs, with K split over a cluster while they are few.
// The caller decides (kernels/ops.py).
SHISO_API int shiso_gemm_tcgen05_tokens64(const void* x, const void* w, const float* bias, void* y, int y_dtype, int T,
                                          int N, int K, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (!shiso_gemm_tcgen05_supported(K, x, w)) return SHISO_ERR_UNSUPPORTED;
    GemmParams p = blank_params(T, N, K);
    p.y = y;
    p.bias = bias;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    return run_plain(p, x, w, sm_count, stream, 64);
}

// silu(x gate^T) * (x up^T) for w = [gate; up] of shape [2 * inter, K]; y [T, inter].
SHISO_API int shiso_gemm_tcgen05_swiglu(const void* x, const void* w, void* y, int y_dtype, int T, int inter, int K,
                                        cudaStream_t stream) {
    if (T <= 0 || inter <= 0) return SHISO_OK;
    if (!shiso_gemm_tcgen05_supported(K, x, w)) return SHISO_ERR_UNSUPPORTED;
    GemmParams p = blank_params(T, 2 * inter, K);
    p.y = y;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    p.inter = inter;
    return run_glu(p, x, w, stream);
}

// Rows of the fused-norm pair below: token tiles of at most 64.  Up to 192 rows they are this
// kernel's own tiles; a plain product takes up to 1,024 rows as tiles of 64 (the shapes
// shiso_gemm_tcgen05_tokens64 is for), a gate/up pair does not.
SHISO_API int shiso_gemm_tcgen05_fused_max_tokens(void) { return 192; }
SHISO_API int shiso_gemm_tcgen05_fused_max_tokens64(void) { return 1024; }

// Rows of T floats of `partials_out` that shiso_gemm_tcgen05_into writes for N features.
SHISO_API int shiso_gemm_tcgen05_into_partial_rows(int N) { return (N + BM - 1) / BM; }

// A block's output projection into the residual stream, for 1..192 rows: res_out = res_in +
// x w^T (+ bias) (float [T, N]; res_in is not changed), x_out = bf16(res_out * next_norm_w)
// [T, N], and partials_out[c * T + t] (c < ceil(N / 128)) whose sum over c is the sum of
// squares of res_out's row t: what shiso_gemm_tcgen05_scaled takes in place of normed rows.
SHISO_API int shiso_gemm_tcgen05_into(const void* x, const void* w, const float* bias, const float* res_in,
                                      float* res_out, const float* next_norm_w, void* x_out, float* partials_out, int T,
                                      int N, int K, int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    if (T > shiso_gemm_tcgen05_fused_max_tokens64() || !res_in || !res_out || !next_norm_w || !x_out || !partials_out)
        return SHISO_ERR_UNSUPPORTED;
    if (!shiso_gemm_tcgen05_supported(K, x, w)) return SHISO_ERR_UNSUPPORTED;
    GemmParams p = blank_params(T, N, K);
    p.bias = bias;
    p.res_in = res_in;
    p.res_out = res_out;
    p.norm_w = next_norm_w;
    p.x_out = (__nv_bfloat16*)x_out;
    p.into_partials = partials_out;
    return run_plain(p, x, w, sm_count, stream, T > shiso_gemm_tcgen05_fused_max_tokens() ? 64 : 0);
}

// y = (x * rsqrt(mean square + eps)) w^T for rows x [T, K] that lack their RMS scale (x_out of
// the call above; mean square of row t = sum over c < partial_count of partials[c * stride + t]
// / K), 1..192 rows; with inter > 0 the gate/up pair and SwiGLU as in shiso_gemm_tcgen05_swiglu.
SHISO_API int shiso_gemm_tcgen05_scaled(const void* x, const float* partials, int partial_count, int partial_stride,
                                        float eps, const void* w, void* y, int y_dtype, int T, int N, int K, int inter,
                                        int sm_count, cudaStream_t stream) {
    if (T <= 0 || N <= 0) return SHISO_OK;
    const bool tiles64 = T > shiso_gemm_tcgen05_fused_max_tokens();
    if (T > (inter > 0 ? shiso_gemm_tcgen05_fused_max_tokens() : shiso_gemm_tcgen05_fused_max_tokens64()) || !partials ||
        partial_count <= 0 || partial_stride < T)
        return SHISO_ERR_UNSUPPORTED;
    if (inter > 0 && N != 2 * inter) return SHISO_ERR_SHAPE;
    if (!shiso_gemm_tcgen05_supported(K, x, w)) return SHISO_ERR_UNSUPPORTED;
    GemmParams p = blank_params(T, N, K);
    p.y = y;
    p.out_f32 = y_dtype == SHISO_F32 ? 1 : 0;
    p.inter = inter;
    p.scale_partials = partials;
    p.scale_count = partial_count;
    p.scale_stride = partial_stride;
    p.scale_eps = eps;
    return inter > 0 ? run_glu(p, x, w, stream) : run_plain(p, x, w, sm_count, stream, tiles64 ? 64 : 0);
}
