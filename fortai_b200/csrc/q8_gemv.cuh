// Batch-1 Q8_0 x Q8_0 matrix-vector kernels for sm_100a.
//
// What they replace in the reference (backend/cuda/fortai_cuda_backend.cu):
//   q8_gemv_one_warp :64-86, q8_gemv_four_warp :88-126, launch_q8 :139-147,
//   q8_gemv_fused4 :149-190, q8_gemv_silu_product + qwen_silu_product :331-384,
//   qwen_quantize_q8 :483-498 (folded into the GEMV prologue for fp32 input).
//
// Arithmetic (identical per block to the reference GPU kernels):
//   dot_b  = sum_{i<32} qw[b][i] * qa[b][i]            exact int32 (dp4a)
//   out    = sum_b fmaf(half(dw[b]) * half(da[b]), float(dot_b), acc)
// Each lane owns 16-byte half-blocks; the two halves of a block sit in adjacent
// lanes and are joined with one shuffle before the scale is applied, so the
// value that gets scaled is the exact int32 block dot.  Lane partial sums are
// combined with a butterfly; only the fp32 summation order differs from the CPU
// path.
//
// This is HBM-streaming integer/byte work (about 1.9 int-ops per weight byte),
// so no tensor cores: the design goal is bytes in flight.  Two variants:
//   direct  persistent warps, each lane issues U 16-byte no-allocate loads per
//           row before consuming any of them;
//   ring    one producer thread per CTA feeds a shared-memory ring of row tiles
//           with 1-D bulk asynchronous copies (the TMA engine) completed on
//           mbarriers; eight consumer warps dequant-and-dot out of shared
//           memory.  Every barrier wait is bounded and reports a status word.
#pragma once

#include "q8_common.cuh"

namespace fortai_b200 {

constexpr int kMaxSegments = 4;
constexpr int kMaxPeers = 8;
constexpr int kGemvWarps = 8;
constexpr int kGemvThreads = kGemvWarps * 32;

enum GemvEpilogue : int {
    kEpiPlain = 0,      // out[row] = dot
    kEpiSiluPair = 1,   // segments: 0 = gate, 1 = up; out[row] = silu(gate.x) * (up.x)
    kEpiBlockDots = 2,  // int32 out[row * blocks + b] = exact block dot
    kEpiPeers = 3,      // plain, stored into every peer's output vector
    kEpiStacked = 4     // pipelined kernel only: plain over up to four stacked matrices
};

enum ActivationKind : int {
    kActQ8 = 0,      // width/32 blocks of 34 bytes (GGUF Q8_0)
    kActF32 = 1,     // width floats, quantized in the prologue
    kActPlanar = 2   // the shared-memory image itself, prepared once in global memory
};

struct GemvParams {
    const uint8_t *weights[kMaxSegments];
    float *outputs[kMaxSegments];
    int rows[kMaxSegments];
    int segments;
    int total_rows;
    int width;
    int blocks;
    int row_stride;
    const void *activation;
    int *status;
    // When the successor in the stream may be scheduled (programmatic dependent launch).
    // Zero: after the row loop, so its launch overlaps this grid's tail only (the default for
    // every GEMV but the one with a residual epilogue, which a many-row projection follows).
    // Non-zero: as soon as every CTA of this grid runs.  That lets a successor request its
    // first weights earlier (the same 9728 x 2560 product back to back: 5.6 us against
    // 6.7 us), but its CTAs take whatever slots are free at that moment, piled onto the SMs
    // with room; a successor of few CTAs then runs on part of the machine (1024 x 3840
    // after 7680 x 1024: 5.1 us against 4.3 us; the 1024-wide FFN 8.4 us against 6.6 us),
    // and whole decode steps are 1-3 % slower.
    int trigger_early;
    float *peer_outputs[kMaxPeers];
    int peers;
    int first_row;  // element offset of this shard inside the peers' vectors
    // fused all-gather (sequence != 0): flag words in every rank's memory
    unsigned *peer_flags[kMaxPeers];   // peer_flags[p][my_rank] is written with `sequence`
    unsigned *my_flags;                // this rank's own flag array, one word per peer
    unsigned *cta_counter;             // device word, zero between launches
    unsigned sequence;
    int my_rank;
    long long flag_wait_clocks;        // how long the tail waits for a peer's flag (SM clocks)
    int overlap_ok;                    // the only "peer" is this process: dependent launch allowed
    // optional fusions of the caller's glue (null = off): an RMS norm of the fp32
    // activation with learned scale in the prologue, and out[row] = dot + residual[row]
    // in the plain epilogue (residual may be the output vector itself)
    const float *norm_weights;
    float norm_epsilon;
    const float *residual;
    // optional, half-block kernel only: the first `conv_rows` output rows are channels of a
    // causal depthwise convolution (window conv_kernel, history in conv_state) followed by
    // SiLU - the gated-delta-net layer's step between its input projections and its state
    // update, done by the lane that holds the finished dot product
    const float *conv_weights;
    float *conv_state;
    int conv_rows;
    int conv_kernel;
};

// One channel of the causal depthwise convolution over the last `kernel` inputs, SiLU, and
// the shift of that channel's history (conv_state is (kernel - 1) x channels, oldest first).
// Same arithmetic as the reference's CPU layer (src/models/qwen35/fortai_qwen35_cpu.f90:856-879).
__device__ __forceinline__ float conv_silu_channel(const float *__restrict__ conv_weights,
    float *__restrict__ conv_state, int channels, int kernel, int c, float now) {
    float acc = 0.0f;
    for (int slot = 0; slot < kernel - 1; ++slot) {
        const float held = conv_state[slot * channels + c];
        acc += conv_weights[c * kernel + slot] * held;
        if (slot > 0) conv_state[(slot - 1) * channels + c] = held;
    }
    acc += conv_weights[c * kernel + kernel - 1] * now;
    conv_state[(kernel - 2) * channels + c] = now;
    return silu_ieee(acc);
}

// Tail of a peer-output GEMV: turns "every rank stored its slice everywhere" into "this
// launch is complete only when every rank's slice has arrived here", without a second
// kernel.  Every CTA publishes its stores system-wide and counts itself; in the last one,
// one lane per peer raises this rank's flag in that peer's memory and then waits, for at
// most about one second, until that peer has raised its flag here.  A wait that runs out writes a
// status word and returns; the kernel never spins without a bound.  All ranks must run
// on different GPUs (they wait on one another).
__device__ __forceinline__ void peer_allgather_tail(const GemvParams &p) {
    if (p.sequence == 0) return;
    __shared__ int is_last_cta;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned arrived = atomicAdd(p.cta_counter, 1u);
        is_last_cta = arrived == gridDim.x - 1;
        if (is_last_cta) {
            *p.cta_counter = 0;                   // ready for the next launch
            __threadfence_system();
        }
    }
    __syncthreads();
    if (!is_last_cta || threadIdx.x >= p.peers) return;
    // one lane per peer: raise this rank's flag there, then wait for that peer's flag here
    const int peer = threadIdx.x;
    unsigned *remote = p.peer_flags[peer] + p.my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(p.sequence) : "memory");
    const unsigned *local = p.my_flags + peer;
    const long long start = clock64();
    const long long limit = p.flag_wait_clocks;   // about a second of SM clocks by default
    for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(local) : "memory");
        // sequence numbers only grow; the signed difference survives wrap-around
        if (static_cast<int>(seen - p.sequence) >= 0) break;
        if (clock64() - start > limit) {
            atomicExch(p.status, kStatusPeerFlagTimeout);
            break;
        }
    }
}

// Shared-memory image of the activation: `width` int8 quants, then `blocks`
// floats holding half(da[b]).
__host__ __device__ inline size_t activation_smem_bytes(int width, int blocks) {
    return (static_cast<size_t>(width) + static_cast<size_t>(blocks) * 4 + 15) & ~size_t(15);
}

// 1 / sqrt(mean(x^2) + epsilon) over `width` floats, by all threads of the CTA.  Sum of
// squares in double and the rest in float, as the reference's RMS norm does it
// (src/models/qwen35/fortai_qwen35_cpu.f90:1422-1427, backend/cuda/fortai_cuda_backend.cu:518-537).
__device__ __forceinline__ float rms_inverse_scale(const float *x, int width, float epsilon, int tid,
    int threads) {
    __shared__ double rms_partial[32];
    double sum = 0.0;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int g = tid; g < (width >> 2); g += threads) {
        const float4 v = x4[g];
        sum += static_cast<double>(v.x) * v.x + static_cast<double>(v.y) * v.y +
            static_cast<double>(v.z) * v.z + static_cast<double>(v.w) * v.w;
    }
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    if ((tid & 31) == 0) rms_partial[tid >> 5] = sum;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (threads + 31) / 32; ++w) total += rms_partial[w];
    return 1.0f / sqrtf(static_cast<float>(total / static_cast<double>(width)) + epsilon);
}

template <int ACT>
__device__ __forceinline__ void stage_activation(const void *activation, int width, int blocks,
    uint8_t *smem, int tid, int threads, const float *norm_weights = nullptr,
    float norm_epsilon = 0.0f) {
    int8_t *act_q = reinterpret_cast<int8_t *>(smem);
    float *act_s = reinterpret_cast<float *>(smem + width);
    if (ACT == kActPlanar) {
        // long vectors are quantized once by q8_planar_prepare_kernel; every CTA only
        // copies the finished image (16-byte loads) instead of redoing the work
        const int4 *src = static_cast<const int4 *>(activation);
        int4 *dst = reinterpret_cast<int4 *>(smem);
        const int count = static_cast<int>(activation_smem_bytes(width, blocks) >> 4);
        for (int i = tid; i < count; i += threads) dst[i] = src[i];
    } else if (ACT == kActQ8) {
        // 17 two-byte words per block: word 0 is the scale, words 1..16 the quants.
        const uint16_t *raw = static_cast<const uint16_t *>(activation);
        uint16_t *act_q16 = reinterpret_cast<uint16_t *>(act_q);
        const int words = blocks * 17;
        for (int i = tid; i < words; i += threads) {
            const int b = i / 17;
            const int j = i - b * 17;
            const uint16_t v = raw[i];
            if (j == 0) act_s[b] = half_bits_to_float(v);
            else act_q16[b * 16 + (j - 1)] = v;
        }
    } else {
        // fp32 -> Q8_0, eight lanes per block: every thread takes four consecutive
        // floats (one 16-byte load), the block maximum is three shuffles within the
        // 8-lane group, and the four quants leave as one 32-bit store.  All loads of
        // a pass are issued before the first shuffle.  Same arithmetic, hence the
        // same bytes, as quantize_lane.
        const float4 *x4 = static_cast<const float4 *>(activation);
        uint32_t *act_q32 = reinterpret_cast<uint32_t *>(act_q);
        const int groups = width >> 2;              // float4 count; 8 per block
        const float4 *w4 = reinterpret_cast<const float4 *>(norm_weights);
        const float inverse_rms = norm_weights
            ? rms_inverse_scale(static_cast<const float *>(activation), width, norm_epsilon, tid,
                  threads)
            : 1.0f;
        constexpr int kPasses = 4;
        for (int g0 = tid; g0 - tid < groups; g0 += threads * kPasses) {
            float4 v[kPasses];
#pragma unroll
            for (int k = 0; k < kPasses; ++k) {
                const int g = g0 + k * threads;
                v[k] = g < groups ? x4[g] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (norm_weights && g < groups) {
                    // (x * inverse) * weight, each product rounded, as the norm kernel does
                    const float4 w = w4[g];
                    v[k].x = __fmul_rn(__fmul_rn(v[k].x, inverse_rms), w.x);
                    v[k].y = __fmul_rn(__fmul_rn(v[k].y, inverse_rms), w.y);
                    v[k].z = __fmul_rn(__fmul_rn(v[k].z, inverse_rms), w.z);
                    v[k].w = __fmul_rn(__fmul_rn(v[k].w, inverse_rms), w.w);
                }
            }
#pragma unroll
            for (int k = 0; k < kPasses; ++k) {
                const int g = g0 + k * threads;
                float amax = fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)),
                    fmaxf(fabsf(v[k].z), fabsf(v[k].w)));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                const float scale = __fdiv_rn(amax, 127.0f);
                const float inverse = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                const int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v[k].x, inverse))));
                const int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v[k].y, inverse))));
                const int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v[k].z, inverse))));
                const int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v[k].w, inverse))));
                if (g < groups) {
                    act_q32[g] = static_cast<uint32_t>(q0 & 0xff) |
                        (static_cast<uint32_t>(q1 & 0xff) << 8) |
                        (static_cast<uint32_t>(q2 & 0xff) << 16) |
                        (static_cast<uint32_t>(q3 & 0xff) << 24);
                    if ((g & 7) == 0)
                        act_s[g >> 3] = half_bits_to_float(
                            __half_as_ushort(__float2half_rn(scale)));
                }
            }
        }
    }
}

// NR rows at once from global memory.  All 16-byte loads of a pass are issued
// before the first one is consumed.
template <int NR, int U, bool BLOCKDOTS>
__device__ __forceinline__ void rows_dot_global(const uint8_t *const (&base)[NR],
    const int4 *__restrict__ act_q, const float *__restrict__ act_s, int width, int nchunks,
    int lane, float (&acc)[NR], int32_t *const (&dots)[NR]) {
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.0f;
    for (int c0 = 0; c0 < nchunks; c0 += 32 * U) {
        int4 w[NR][U];
        uint16_t d[NR][U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = c0 + u * 32 + lane;
            const bool ok = idx < nchunks;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                if (ok) {
                    w[r][u] = ldg_stream_16(base[r] + static_cast<size_t>(idx) * 16);
                    d[r][u] = ldg_stream_u16(base[r] + width + (idx >> 1) * 2);
                } else {
                    w[r][u] = make_int4(0, 0, 0, 0);
                    d[r][u] = 0;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = c0 + u * 32 + lane;
            const bool ok = idx < nchunks;
            const int4 a = ok ? act_q[idx] : make_int4(0, 0, 0, 0);
            const float sa = (ok && !(lane & 1)) ? act_s[idx >> 1] : 0.0f;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                int dot = dot16(w[r][u], a);
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                acc[r] = fmaf(half_bits_to_float(d[r][u]) * sa, static_cast<float>(dot), acc[r]);
                if (BLOCKDOTS && ok && !(lane & 1)) dots[r][idx >> 1] = dot;
            }
        }
    }
}

// --------------------------------------------------------------------------
// direct variant
// --------------------------------------------------------------------------
template <int U, int NR, int ACT, int EPI>
__global__ void __launch_bounds__(kGemvThreads)
q8_gemv_direct_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    if (p.trigger_early) grid_dependents_may_launch();
    grid_dependency_wait();      // the activation is the previous kernel's output
    stage_activation<ACT>(p.activation, p.width, p.blocks, gemv_smem, threadIdx.x, kGemvThreads,
        p.norm_weights, p.norm_epsilon);
    __syncthreads();
    const int4 *act_q = reinterpret_cast<const int4 *>(gemv_smem);
    const float *act_s = reinterpret_cast<const float *>(gemv_smem + p.width);
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * kGemvWarps + (threadIdx.x >> 5);
    const int warps = gridDim.x * kGemvWarps;
    const int nchunks = p.width >> 4;
    const size_t stride = static_cast<size_t>(p.row_stride);

    if (EPI == kEpiSiluPair) {
        // NR is 2 here: the gate row and the up row of the same index.
        for (int row = warp; row < p.total_rows; row += warps) {
            const uint8_t *base[2] = {p.weights[0] + row * stride, p.weights[1] + row * stride};
            int32_t *none[2] = {nullptr, nullptr};
            float acc[2];
            rows_dot_global<2, U, false>(base, act_q, act_s, p.width, nchunks, lane, acc, none);
            const float gate = warp_sum(acc[0]);
            const float up = warp_sum(acc[1]);
            if (lane == 0) p.outputs[0][row] = silu_mul(gate, up);
        }
        return;
    }

    for (int first = warp * NR; first < p.total_rows; first += warps * NR) {
        const uint8_t *base[NR];
        float *out[NR];
        int32_t *dots[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            int row = first + r;
            if (row >= p.total_rows) row = first;  // duplicate work, no store
            int seg = 0;
            int local = row;
            if (EPI == kEpiPlain) {
#pragma unroll
                for (int s = 0; s < kMaxSegments - 1; ++s)
                    if (seg == s && s + 1 < p.segments && local >= p.rows[s]) {
                        local -= p.rows[s];
                        seg = s + 1;
                    }
            }
            base[r] = p.weights[seg] + local * stride;
            out[r] = p.outputs[seg] + local;
            dots[r] = EPI == kEpiBlockDots
                ? reinterpret_cast<int32_t *>(p.outputs[0]) + static_cast<size_t>(local) * p.blocks
                : nullptr;
        }
        float acc[NR];
        rows_dot_global<NR, U, EPI == kEpiBlockDots>(base, act_q, act_s, p.width, nchunks, lane,
            acc, dots);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const float total = warp_sum(acc[r]);
            const int row = first + r;
            if (lane == 0 && row < p.total_rows) {
                if (EPI == kEpiPlain) {
                    float value = p.residual ? total + p.residual[row] : total;
                    if (p.conv_weights && row < p.conv_rows)
                        value = conv_silu_channel(p.conv_weights, p.conv_state, p.conv_rows,
                            p.conv_kernel, row, value);
                    *out[r] = value;
                } else if (EPI == kEpiPeers) {
                    for (int peer = 0; peer < p.peers; ++peer)
                        p.peer_outputs[peer][p.first_row + row] = total;
                }
            }
        }
    }
    grid_dependents_may_launch();
    if (EPI == kEpiPeers) peer_allgather_tail(p);
}

// --------------------------------------------------------------------------
// split-row variant: few rows, long rows (FFN down projections)
// --------------------------------------------------------------------------
// With fewer rows than resident warps (5120 rows of 18.5 KB on 4736 warps) a
// warp-per-row grid leaves most of the machine idle in its last round.  Here SPLIT
// adjacent warps of a CTA share a row: each takes a contiguous K-slice (a whole
// number of blocks), and the SPLIT partial sums meet in shared memory.  Same lane
// mapping and arithmetic as the half-block kernel; only the fp32 summation order
// differs.
template <int SPLIT, int ACT, int EPI>
__global__ void __launch_bounds__(kGemvThreads)
q8_gemv_splitrow_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    __shared__ float partial[kGemvWarps];
    stage_activation<ACT>(p.activation, p.width, p.blocks, gemv_smem, threadIdx.x, kGemvThreads);
    __syncthreads();
    const int4 *act_q = reinterpret_cast<const int4 *>(gemv_smem);
    const float *act_s = reinterpret_cast<const float *>(gemv_smem + p.width);
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    constexpr int ROWS_PER_ROUND = kGemvWarps / SPLIT;
    constexpr int U = 8;
    const int slice = warp % SPLIT;
    const int blocks_per_slice = (p.blocks + SPLIT - 1) / SPLIT;
    const int chunk_begin = min(p.blocks, slice * blocks_per_slice) * 2;
    const int chunk_end = min(p.blocks, (slice + 1) * blocks_per_slice) * 2;
    const size_t stride = static_cast<size_t>(p.row_stride);

    for (int first = blockIdx.x * ROWS_PER_ROUND; first < p.total_rows;
         first += gridDim.x * ROWS_PER_ROUND) {
        const int row = first + warp / SPLIT;
        const bool row_ok = row < p.total_rows;
        const uint8_t *base = p.weights[0] + static_cast<size_t>(row_ok ? row : first) * stride;
        float acc = 0.0f;
        for (int c0 = chunk_begin; c0 < chunk_end; c0 += 32 * U) {
            int4 w[U];
            uint16_t d[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = c0 + u * 32 + lane;
                if (idx < chunk_end) {
                    w[u] = ldg_stream_16(base + static_cast<size_t>(idx) * 16);
                    d[u] = ldg_stream_u16(base + p.width + (idx >> 1) * 2);
                } else {
                    w[u] = make_int4(0, 0, 0, 0);
                    d[u] = 0;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int idx = c0 + u * 32 + lane;
                const bool ok = idx < chunk_end;
                const int4 a = ok ? act_q[idx] : make_int4(0, 0, 0, 0);
                const float sa = ok ? act_s[idx >> 1] : 0.0f;
                acc = fmaf(half_bits_to_float(d[u]) * sa, static_cast<float>(dot16(w[u], a)), acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) partial[warp] = acc;
        __syncthreads();
        if (lane == 0 && slice == 0 && row_ok) {
            float total = 0.0f;
#pragma unroll
            for (int k = 0; k < SPLIT; ++k) total += partial[warp + k];
            if (EPI == kEpiPeers) {
                for (int peer = 0; peer < p.peers; ++peer)
                    p.peer_outputs[peer][p.first_row + row] = total;
            } else {
                p.outputs[0][row] = total;
            }
        }
        __syncthreads();
    }
    if (EPI == kEpiPeers) peer_allgather_tail(p);
}

// --------------------------------------------------------------------------
// pipelined variant: two rows in flight per warp, one request for a row's scales
// --------------------------------------------------------------------------
// Same lane mapping as the half-block kernel (lane l owns 16-byte chunks l,
// l + 32, ...; CPL chunks per lane, exact: width == 512 * CPL), rebuilt around
// what a bare read kernel of the same access pattern showed on B200: the weight
// stream itself runs at 7.1 TB/s, and what slows a GEMV down is (a) the number of
// separate load requests - five 2-byte scale loads per row cost 9 % - and (b) the
// time during which a warp has nothing in flight.  Hence:
//  * a row's fp16 scales (2 * B bytes, contiguous behind its quants) are fetched by
//    ONE 16-byte load on lanes < 2 * CPL and handed to the other lanes through a
//    per-warp shared-memory slot when the row is consumed;
//  * register double buffering: the loads of the row after next are issued before
//    a row is consumed, and the first two rows are requested before the activation
//    is staged, so the quantize prologue runs under a full memory pipeline;
//  * no predicates and no per-chunk address arithmetic (one pointer per row, all
//    chunk offsets are immediates);
//  * each lane scales its own exact int32 half-block dot (no shuffle per chunk):
//    out = sum over half-blocks of fmaf(half(dw) * half(da), float(dot_half), acc).
// ROWS is 1 (plain / peers) or 2 (gate row + up row with the SiLU epilogue).
template <int CPL>
struct RowRegs {
    int4 w[CPL];
    int4 scales;   // lanes < 2 * CPL: eight fp16 scales of this row
};

template <int CPL>
__device__ __forceinline__ void row_issue(RowRegs<CPL> &regs, const uint8_t *row, int lane,
    int width) {
#pragma unroll
    for (int u = 0; u < CPL; ++u) regs.w[u] = ldg_stream_16(row + lane * 16 + u * 512);
    if (lane < 2 * CPL) regs.scales = ldg_stream_16(row + width + lane * 16);
}

template <int CPL>
__device__ __forceinline__ float row_consume(const RowRegs<CPL> &regs, const int4 *act_lane,
    const float *scale_lane, uint8_t *slot, int lane) {
    if (lane < 2 * CPL) *reinterpret_cast<int4 *>(slot + lane * 16) = regs.scales;
    __syncwarp();
    float acc = 0.0f;
#pragma unroll
    for (int u = 0; u < CPL; ++u) {
        const uint16_t dw = *reinterpret_cast<const uint16_t *>(slot + ((lane >> 1) + u * 16) * 2);
        const int4 a = act_lane[u * 32];
        const float sa = scale_lane[u * 16];
        acc = fmaf(half_bits_to_float(dw) * sa, static_cast<float>(dot16(regs.w[u], a)), acc);
    }
    __syncwarp();
    return acc;
}

// Shared memory of the pipelined kernel: the activation image, then one scale slot
// per (warp, row-of-the-pair).
__host__ __device__ inline size_t pipelined_smem_bytes(int width, int blocks, int cpl, int rows) {
    return activation_smem_bytes(width, blocks) +
        static_cast<size_t>(kGemvWarps) * rows * (2 * cpl * 16);
}

// Row `row` of up to four matrices stacked one after the other (the fused projections of
// a layer): which matrix, which of its rows, and where that row starts.
__device__ __forceinline__ const uint8_t *stacked_row(const GemvParams &p, int row, size_t stride,
    int *segment, int *local) {
    int seg = 0, at = row;
#pragma unroll
    for (int s = 0; s < kMaxSegments - 1; ++s)
        if (seg == s && s + 1 < p.segments && at >= p.rows[s]) {
            at -= p.rows[s];
            seg = s + 1;
        }
    *segment = seg;
    *local = at;
    return p.weights[seg] + at * stride;
}

// DEPTH is the number of rows a warp keeps in flight: 1 = the next row is
// requested right after the current one has been consumed (64 registers, four
// CTAs per SM for CPL = 5), 2 = it is requested one row earlier (register double
// buffering, fewer resident warps).
template <int CPL, int ACT, int EPI, int DEPTH>
__global__ void __launch_bounds__(kGemvThreads)
q8_gemv_pipelined_kernel(const __grid_constant__ GemvParams p) {
    if (p.trigger_early) grid_dependents_may_launch();
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    constexpr int ROWS = EPI == kEpiSiluPair ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    const size_t stride = static_cast<size_t>(p.row_stride);
    uint8_t *slots = gemv_smem + activation_smem_bytes(p.width, p.blocks) +
        warp_in_cta * ROWS * (2 * CPL * 16);

    // Row assignment.  Ordinary outputs: grid-stride over warps (warp g takes rows g,
    // g + W, ...).  Peer outputs: each CTA takes one contiguous block of rows, collects
    // its results in shared memory and stores them to every peer as whole 128-byte lines
    // at the end - one NVLink packet per 32 rows instead of one per row.
    int row, row_step, row_end, cta_first = 0;
    if (EPI == kEpiPeers) {
        const int per_cta = (p.total_rows + gridDim.x - 1) / gridDim.x;
        cta_first = blockIdx.x * per_cta;
        row = cta_first + warp_in_cta;
        row_step = kGemvWarps;
        row_end = min(p.total_rows, cta_first + per_cta);
    } else {
        row = blockIdx.x * kGemvWarps + warp_in_cta;
        row_step = gridDim.x * kGemvWarps;
        row_end = p.total_rows;
    }
    const size_t step = stride * row_step;
    float *staged = reinterpret_cast<float *>(gemv_smem +
        pipelined_smem_bytes(p.width, p.blocks, CPL, ROWS));

    // several stacked matrices (plain epilogue, one row in flight): the row's matrix and
    // local index are looked up per row instead of stepping one base pointer
    constexpr bool stacked = EPI == kEpiStacked;
    int segment = 0, local = row;
    const uint8_t *base[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) base[r] = p.weights[r] + row * stride;
    if (stacked && row < row_end) base[0] = stacked_row(p, row, stride, &segment, &local);
    RowRegs<CPL> cur[ROWS], next[DEPTH == 2 ? ROWS : 1];
    // the first row(s) are requested before the activation is staged, so the
    // quantize prologue runs under a full memory pipeline
    if (row < row_end) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) row_issue<CPL>(cur[r], base[r], lane, p.width);
    }
    if (DEPTH == 2 && row + row_step < row_end) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) row_issue<CPL>(next[r], base[r] + step, lane, p.width);
    }

    // the weight requests above do not depend on the previous kernel; everything below does
    grid_dependency_wait();
    stage_activation<ACT>(p.activation, p.width, p.blocks, gemv_smem, threadIdx.x, kGemvThreads,
        p.norm_weights, p.norm_epsilon);
    __syncthreads();
    const int4 *act_lane = reinterpret_cast<const int4 *>(gemv_smem) + lane;
    const float *scale_lane = reinterpret_cast<const float *>(gemv_smem + p.width) + (lane >> 1);

    while (row < row_end) {
        float partial[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            partial[r] = row_consume<CPL>(cur[r], act_lane, scale_lane,
                slots + r * (2 * CPL * 16), lane);
        const int finished = row, finished_segment = segment, finished_local = local;
        row += row_step;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) base[r] += step;
        if (stacked && row < row_end) base[0] = stacked_row(p, row, stride, &segment, &local);
        if (DEPTH == 1) {
            // registers of `cur` are free again: request the next row before reducing
            if (row < row_end) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r) row_issue<CPL>(cur[r], base[r], lane, p.width);
            }
        }
        float total[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) total[r] = warp_sum(partial[r]);
        if (lane == 0) {
            if (EPI == kEpiSiluPair) {
                p.outputs[0][finished] = silu_mul(total[0], total[ROWS - 1]);
            } else if (EPI == kEpiPeers) {
                staged[finished - cta_first] = total[0];
            } else if (stacked) {
                float value = total[0];
                if (p.conv_weights && finished < p.conv_rows)
                    value = conv_silu_channel(p.conv_weights, p.conv_state, p.conv_rows,
                        p.conv_kernel, finished, value);
                p.outputs[finished_segment][finished_local] = value;
            } else {
                p.outputs[0][finished] = p.residual ? total[0] + p.residual[finished] : total[0];
            }
        }
        if (DEPTH == 2) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) cur[r] = next[r];
            if (row + row_step < row_end) {
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    row_issue<CPL>(next[r], base[r] + step, lane, p.width);
            }
        }
    }
    grid_dependents_may_launch();
    if (EPI == kEpiPeers) {
        __syncthreads();
        const int count = row_end - cta_first;
        for (int peer = 0; peer < p.peers; ++peer) {
            float *dst = p.peer_outputs[peer] + p.first_row + cta_first;
            for (int i = threadIdx.x; i < count; i += kGemvThreads) dst[i] = staged[i];
        }
    }
    if (EPI == kEpiPeers) peer_allgather_tail(p);
}

// --------------------------------------------------------------------------
// block-per-lane variant: one 32-byte load fetches a whole Q8_0 block
// --------------------------------------------------------------------------
// Lane l owns blocks l, l + 32, ... of a row, so every int32 block dot is formed
// inside one lane (eight dp4a) and no shuffle is needed before scaling.  With
// P > 0 the row has at most 32 * P blocks and the lane's share of the quantized
// activation (P blocks, 9 registers each) stays in registers for the whole
// kernel; with P == 0 the activation is read from shared memory.  Compared with
// the half-block kernel above this issues about a quarter of the instructions
// per weight byte, which is what keeps the SM clock up under the power cap.
struct Block32 {
    int4 lo, hi;
};

__device__ __forceinline__ Block32 ldg_stream_32(const void *address) {
    Block32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.s32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x),
                   "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                 : "l"(address));
    return v;
}

__device__ __forceinline__ int dot32(const Block32 &w, const Block32 &a) {
    return dot16(w.hi, a.hi) + dot16(w.lo, a.lo);
}

template <int P, int NR, int ACT, int EPI>
__global__ void __launch_bounds__(kGemvThreads)
q8_gemv_block_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    stage_activation<ACT>(p.activation, p.width, p.blocks, gemv_smem, threadIdx.x, kGemvThreads);
    __syncthreads();
    const int4 *act_q = reinterpret_cast<const int4 *>(gemv_smem);
    const float *act_s = reinterpret_cast<const float *>(gemv_smem + p.width);
    const int lane = threadIdx.x & 31;
    const int warp = blockIdx.x * kGemvWarps + (threadIdx.x >> 5);
    const int warps = gridDim.x * kGemvWarps;
    const int blocks = p.blocks;
    const size_t stride = static_cast<size_t>(p.row_stride);
    constexpr int PR = P > 0 ? P : 1;
    constexpr int ROWS_AT_ONCE = EPI == kEpiSiluPair ? 2 : NR;

    // register image of this lane's activation blocks (P > 0 only)
    Block32 a_reg[PR];
    float sa_reg[PR];
    if (P > 0) {
#pragma unroll
        for (int u = 0; u < PR; ++u) {
            const int b = u * 32 + lane;
            const bool ok = b < blocks;
            a_reg[u].lo = ok ? act_q[2 * b] : make_int4(0, 0, 0, 0);
            a_reg[u].hi = ok ? act_q[2 * b + 1] : make_int4(0, 0, 0, 0);
            sa_reg[u] = ok ? act_s[b] : 0.0f;
        }
    }
    const int lane_q = lane * 32;   // byte offset of the lane's first block in a row
    const int lane_s = p.width + lane * 2;

    for (int first = warp * NR; first < p.total_rows; first += warps * NR) {
        const uint8_t *base[ROWS_AT_ONCE];
        int local_row[ROWS_AT_ONCE];
        int seg_of[ROWS_AT_ONCE];
#pragma unroll
        for (int r = 0; r < ROWS_AT_ONCE; ++r) {
            if (EPI == kEpiSiluPair) {
                local_row[r] = first;
                seg_of[r] = r;
            } else {
                int row = first + r;
                if (row >= p.total_rows) row = first;
                int seg = 0;
                if (EPI == kEpiPlain && p.segments > 1) {
#pragma unroll
                    for (int s = 0; s < kMaxSegments - 1; ++s)
                        if (seg == s && s + 1 < p.segments && row >= p.rows[s]) {
                            row -= p.rows[s];
                            seg = s + 1;
                        }
                }
                local_row[r] = row;
                seg_of[r] = seg;
            }
            base[r] = p.weights[seg_of[r]] + local_row[r] * stride;
        }
        float acc[ROWS_AT_ONCE];
#pragma unroll
        for (int r = 0; r < ROWS_AT_ONCE; ++r) acc[r] = 0.0f;

        if (P > 0) {
            Block32 w[ROWS_AT_ONCE][PR];
            uint16_t d[ROWS_AT_ONCE][PR];
#pragma unroll
            for (int u = 0; u < PR; ++u) {
                // only the last pass can be ragged
                const bool ok = (u + 1 < PR) || (u * 32 + lane < blocks);
#pragma unroll
                for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                    if (ok) {
                        w[r][u] = ldg_stream_32(base[r] + lane_q + u * 1024);
                        d[r][u] = ldg_stream_u16(base[r] + lane_s + u * 64);
                    } else {
                        w[r][u].lo = w[r][u].hi = make_int4(0, 0, 0, 0);
                        d[r][u] = 0;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < PR; ++u) {
#pragma unroll
                for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                    const int dot = dot32(w[r][u], a_reg[u]);
                    acc[r] = fmaf(half_bits_to_float(d[r][u]) * sa_reg[u],
                        static_cast<float>(dot), acc[r]);
                    if (EPI == kEpiBlockDots && u * 32 + lane < blocks)
                        reinterpret_cast<int32_t *>(p.outputs[0])[
                            static_cast<size_t>(local_row[r]) * blocks + u * 32 + lane] = dot;
                }
            }
        } else {
            constexpr int U = 4;
            for (int b0 = 0; b0 < blocks; b0 += 32 * U) {
                Block32 w[ROWS_AT_ONCE][U];
                uint16_t d[ROWS_AT_ONCE][U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int b = b0 + u * 32 + lane;
                    const bool ok = b < blocks;
#pragma unroll
                    for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                        if (ok) {
                            w[r][u] = ldg_stream_32(base[r] + static_cast<size_t>(b) * 32);
                            d[r][u] = ldg_stream_u16(base[r] + p.width + b * 2);
                        } else {
                            w[r][u].lo = w[r][u].hi = make_int4(0, 0, 0, 0);
                            d[r][u] = 0;
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int b = b0 + u * 32 + lane;
                    const bool ok = b < blocks;
                    Block32 a;
                    a.lo = ok ? act_q[2 * b] : make_int4(0, 0, 0, 0);
                    a.hi = ok ? act_q[2 * b + 1] : make_int4(0, 0, 0, 0);
                    const float sa = ok ? act_s[b] : 0.0f;
#pragma unroll
                    for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                        const int dot = dot32(w[r][u], a);
                        acc[r] = fmaf(half_bits_to_float(d[r][u]) * sa, static_cast<float>(dot),
                            acc[r]);
                        if (EPI == kEpiBlockDots && ok)
                            reinterpret_cast<int32_t *>(p.outputs[0])[
                                static_cast<size_t>(local_row[r]) * blocks + b] = dot;
                    }
                }
            }
        }

        if (EPI == kEpiSiluPair) {
            const float gate = warp_sum(acc[0]);
            const float up = warp_sum(acc[ROWS_AT_ONCE - 1]);
            if (lane == 0) p.outputs[0][first] = silu_mul(gate, up);
        } else {
#pragma unroll
            for (int r = 0; r < ROWS_AT_ONCE; ++r) {
                const float total = warp_sum(acc[r]);
                if (lane == 0 && first + r < p.total_rows) {
                    if (EPI == kEpiPlain) {
                        p.outputs[seg_of[r]][local_row[r]] = total;
                    } else if (EPI == kEpiPeers) {
                        for (int peer = 0; peer < p.peers; ++peer)
                            p.peer_outputs[peer][p.first_row + local_row[r]] = total;
                    }
                }
            }
        }
    }
}

// --------------------------------------------------------------------------
// ring variant
// --------------------------------------------------------------------------
constexpr int kRingConsumerWarps = 8;
constexpr int kRingThreads = (kRingConsumerWarps + 1) * 32;
constexpr int kRingMaxStages = 16;

struct RingConfig {
    int stages;         // 2..kRingMaxStages
    int rows_per_tile;  // rows of one matrix per stage
    int stage_bytes;    // rows_per_tile * row_stride * (2 for the SiLU pair)
    int tiles;          // ceil(total_rows / rows_per_tile)
};

__host__ __device__ inline size_t ring_smem_bytes(int width, int blocks, const RingConfig &cfg) {
    size_t bytes = activation_smem_bytes(width, blocks);
    bytes += 2 * kRingMaxStages * sizeof(uint64_t);
    bytes = (bytes + 127) & ~size_t(127);
    return bytes + static_cast<size_t>(cfg.stages) * cfg.stage_bytes;
}

__device__ __forceinline__ float row_dot_shared(const uint8_t *row, const int4 *act_q,
    const float *act_s, int width, int nchunks, int lane) {
    float acc = 0.0f;
    const int passes = (nchunks + 31) >> 5;
#pragma unroll 4
    for (int pass = 0; pass < passes; ++pass) {
        const int idx = pass * 32 + lane;
        const bool ok = idx < nchunks;
        const int safe = ok ? idx : 0;
        const int4 w = *reinterpret_cast<const int4 *>(row + safe * 16);
        const uint16_t d = *reinterpret_cast<const uint16_t *>(row + width + (safe >> 1) * 2);
        const int4 a = act_q[safe];
        const float sa = (ok && !(lane & 1)) ? act_s[safe >> 1] : 0.0f;
        int dot = ok ? dot16(w, a) : 0;
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        acc = fmaf(half_bits_to_float(d) * sa, static_cast<float>(dot), acc);
    }
    return acc;
}

template <int ACT, int EPI>
__global__ void __launch_bounds__(kRingThreads, 1)
q8_gemv_ring_kernel(const __grid_constant__ GemvParams p, const __grid_constant__ RingConfig cfg) {
    extern __shared__ __align__(128) uint8_t ring_smem[];
    const size_t act_bytes = activation_smem_bytes(p.width, p.blocks);
    uint64_t *full = reinterpret_cast<uint64_t *>(ring_smem + act_bytes);
    uint64_t *empty = full + kRingMaxStages;
    uint8_t *stages = ring_smem +
        ((act_bytes + 2 * kRingMaxStages * sizeof(uint64_t) + 127) & ~size_t(127));
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const size_t stride = static_cast<size_t>(p.row_stride);
    const int copies = EPI == kEpiSiluPair ? 2 : 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < cfg.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kRingConsumerWarps);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // ---------------- producer: one thread drives the copy engine --------------
    // It first arms every stage once (no waits are needed for the first lap), so
    // weight tiles are in flight while the whole CTA stages the activation; only
    // after the CTA-wide barrier does it enter the steady state, where each refill
    // waits for the consumers to release the stage.
    const bool producer = warp == kRingConsumerWarps && lane == 0;
    int issued = 0;
    int next_tile = blockIdx.x;
    auto issue = [&](int tile, int s) {
        const int first_row = tile * cfg.rows_per_tile;
        const int rows = min(cfg.rows_per_tile, p.total_rows - first_row);
        const uint32_t bytes = static_cast<uint32_t>(rows * stride);
        uint8_t *dst = stages + static_cast<size_t>(s) * cfg.stage_bytes;
        mbar_arrive_expect_tx(&full[s], bytes * copies);
        bulk_copy_g2s(dst, p.weights[0] + first_row * stride, bytes, &full[s]);
        if (copies == 2)
            bulk_copy_g2s(dst + cfg.rows_per_tile * stride, p.weights[1] + first_row * stride,
                bytes, &full[s]);
    };
    if (producer) {
        for (; next_tile < cfg.tiles && issued < cfg.stages; next_tile += gridDim.x, ++issued)
            issue(next_tile, issued);
    }

    stage_activation<ACT>(p.activation, p.width, p.blocks, ring_smem, threadIdx.x, kRingThreads);
    __syncthreads();

    if (producer) {
        bool gave_up = false;
        for (; next_tile < cfg.tiles; next_tile += gridDim.x, ++issued) {
            const int s = issued % cfg.stages;
            const int use = issued / cfg.stages;
            if (!mbar_wait_bounded(&empty[s], (use - 1) & 1)) {
                atomicExch(p.status, kStatusRingProducerTimeout);
                atomicExch(&abort_flag, 1);
                gave_up = true;
                break;
            }
            if (*reinterpret_cast<volatile int *>(&abort_flag)) {
                gave_up = true;
                break;
            }
            issue(next_tile, s);
        }
        if (gave_up) {
            // Let copies that are still in flight land before the CTA's shared
            // memory is released: wait (bounded) on the full barrier of every
            // stage that was armed in the last lap.
            const int lap = issued < cfg.stages ? issued : cfg.stages;
            for (int k = 0; k < lap; ++k) {
                const int n = issued - 1 - k;
                mbar_wait_bounded(&full[n % cfg.stages], (n / cfg.stages) & 1, 1u << 16);
            }
        }
    }

    if (warp < kRingConsumerWarps) {
        const int4 *act_q = reinterpret_cast<const int4 *>(ring_smem);
        const float *act_s = reinterpret_cast<const float *>(ring_smem + p.width);
        const int nchunks = p.width >> 4;
        int consumed = 0;
        for (int tile = blockIdx.x; tile < cfg.tiles; tile += gridDim.x, ++consumed) {
            const int s = consumed % cfg.stages;
            const int use = consumed / cfg.stages;
            bool ready = true;
            if (lane == 0) {
                ready = mbar_wait_bounded(&full[s], use & 1);
                if (!ready) {
                    atomicExch(p.status, kStatusRingConsumerTimeout);
                    atomicExch(&abort_flag, 1);
                }
            }
            ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
            if (!ready || *reinterpret_cast<volatile int *>(&abort_flag)) break;
            // lane 0 observed the phase; the others re-check once, which returns
            // at once and gives each lane its own acquire of the copied bytes
            mbar_wait_bounded(&full[s], use & 1, 1u << 10);
            const uint8_t *tile_base = stages + static_cast<size_t>(s) * cfg.stage_bytes;
            const int first_row = tile * cfg.rows_per_tile;
            const int rows = min(cfg.rows_per_tile, p.total_rows - first_row);
            for (int r = warp; r < rows; r += kRingConsumerWarps) {
                const float a0 = warp_sum(row_dot_shared(tile_base + r * stride, act_q, act_s,
                    p.width, nchunks, lane));
                if (EPI == kEpiSiluPair) {
                    const float a1 = warp_sum(row_dot_shared(
                        tile_base + (cfg.rows_per_tile + r) * stride, act_q, act_s, p.width,
                        nchunks, lane));
                    if (lane == 0) p.outputs[0][first_row + r] = silu_mul(a0, a1);
                } else if (EPI == kEpiPeers) {
                    if (lane == 0)
                        for (int peer = 0; peer < p.peers; ++peer)
                            p.peer_outputs[peer][p.first_row + first_row + r] = a0;
                } else {
                    if (lane == 0) p.outputs[0][first_row + r] = a0;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
    }
}

// `count` 16-byte pieces from page-locked host memory (through its device alias) into
// device memory: the host-call path's replacement for a copy-engine transfer of a few
// kilobytes.  Its dependent, the GEMV, may start at once.
__global__ void __launch_bounds__(256)
q8_fetch_kernel(const float4 *__restrict__ source, float4 *__restrict__ destination, int count) {
    grid_dependents_may_launch();
    for (int i = threadIdx.x; i < count; i += blockDim.x) destination[i] = source[i];
}

// --------------------------------------------------------------------------
// standalone quantizer: one warp per block of 32 floats
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
q8_quantize_kernel(const float *__restrict__ input, uint8_t *__restrict__ output, long long blocks) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long long warp = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const long long warps = static_cast<long long>(gridDim.x) * 8;
    for (long long b = warp; b < blocks; b += warps) {
        uint16_t bits;
        const int q = quantize_lane(input[b * kBlockElems + lane], &bits);
        uint8_t *dst = output + b * kBlockBytes;
        dst[2 + lane] = static_cast<uint8_t>(q);
        if (lane == 0) *reinterpret_cast<uint16_t *>(dst) = bits;
    }
}

// --------------------------------------------------------------------------
// activation image prepared once in global memory (long vectors)
// --------------------------------------------------------------------------
// One warp per block: fp32 -> (quants, scale) or GGUF Q8_0 block -> (quants, scale),
// written in the layout the GEMV kernels keep in shared memory.
template <int ACT>
__global__ void __launch_bounds__(256)
q8_planar_prepare_kernel(const void *__restrict__ activation, int width, int blocks,
    uint8_t *__restrict__ image) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    int8_t *act_q = reinterpret_cast<int8_t *>(image);
    float *act_s = reinterpret_cast<float *>(image + width);
    const int lane = threadIdx.x & 31;
    for (int b = blockIdx.x * 8 + (threadIdx.x >> 5); b < blocks; b += gridDim.x * 8) {
        if (ACT == kActF32) {
            uint16_t bits;
            const int q = quantize_lane(
                static_cast<const float *>(activation)[b * kBlockElems + lane], &bits);
            act_q[b * kBlockElems + lane] = static_cast<int8_t>(q);
            if (lane == 0) act_s[b] = half_bits_to_float(bits);
        } else {
            const uint8_t *block = static_cast<const uint8_t *>(activation) +
                static_cast<size_t>(b) * kBlockBytes;
            act_q[b * kBlockElems + lane] = static_cast<int8_t>(block[2 + lane]);
            if (lane == 0)
                act_s[b] = half_bits_to_float(*reinterpret_cast<const uint16_t *>(block));
        }
    }
}

// --------------------------------------------------------------------------
// upload-time re-layout: GGUF blocks -> row-planar device rows
// --------------------------------------------------------------------------
// One thread per (row, block) of the destination.  src_blocks is the block count
// of a full source row; [first_block, first_block + blocks) is the slice kept.
__global__ void __launch_bounds__(256)
q8_repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int rows,
    int src_blocks, int first_block, int blocks, int row_stride) {
    const long long total = static_cast<long long>(rows) * blocks;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / blocks);
        const int b = static_cast<int>(i - static_cast<long long>(row) * blocks);
        const uint16_t *in = reinterpret_cast<const uint16_t *>(
            src + (static_cast<size_t>(row) * src_blocks + first_block + b) * kBlockBytes);
        uint8_t *out_row = dst + static_cast<size_t>(row) * row_stride;
        uint32_t q[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            q[k] = static_cast<uint32_t>(in[1 + 2 * k]) |
                (static_cast<uint32_t>(in[2 + 2 * k]) << 16);
        uint4 *out_q = reinterpret_cast<uint4 *>(out_row + b * kBlockElems);
        out_q[0] = make_uint4(q[0], q[1], q[2], q[3]);
        out_q[1] = make_uint4(q[4], q[5], q[6], q[7]);
        reinterpret_cast<uint16_t *>(out_row + blocks * kBlockElems)[b] = in[0];
    }
}

// Dequantize one row of a row-planar matrix (embedding lookup; reference
// qwen_embedding_lookup_q8, backend.cu:500-510).
__global__ void __launch_bounds__(256)
q8_dequantize_row_kernel(const uint8_t *__restrict__ weights, long long row, int width,
    int row_stride, float *__restrict__ output) {
    const int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= width) return;
    const uint8_t *base = weights + static_cast<size_t>(row) * row_stride;
    const float scale = half_bits_to_float(
        reinterpret_cast<const uint16_t *>(base + width)[index >> 5]);
    output[index] = scale * static_cast<float>(static_cast<int8_t>(base[index]));
}

}  // namespace fortai_b200
