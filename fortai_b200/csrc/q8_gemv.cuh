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
// so no tensor cores: the design goal is bytes in flight.  Three kernels:
//   pipelined   persistent warps, one row (or gate/up row pair) per warp at a time, the
//               next row requested while the current one is reduced; widths that are a
//               whole number of 512-element granules (the default where it applies);
//   slice       the same inner loop over K-slices of a row shared by 2, 4 or 8 warps,
//               for few long rows;
//   half-block  (q8_gemv_direct_kernel) any width, U loads per lane in flight; also
//               carries the int32 block-dot probe and the convolution epilogue.
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

enum PeerExchange : int { kExchangeOff = 0, kExchangeLastCta = 1, kExchangeCounters = 2 };

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
    // fused all-gather (exchange != kExchangeOff): flag words in every rank's memory
    unsigned *peer_flags[kMaxPeers];   // peer_flags[p][my_rank] belongs to this rank
    unsigned *my_flags;                // this rank's own flag array, one word per peer
    unsigned *cta_counter;             // device word, zero between launches
    unsigned sequence;                 // this launch's number among the rank's exchanging launches
    int exchange;                      // kExchangeOff, kExchangeLastCta or kExchangeCounters
    int my_rank;
    long long flag_wait_clocks;        // how long the tail waits for a peer's flag (SM clocks)
    int overlap_ok;                    // the only "peer" is this process: dependent launch allowed
    // all-gather without flags (ll_sequence != 0): peer_outputs[p] is rank p's array of
    // (value, call number) pairs, ll_output this rank's plain vector of ll_total floats
    unsigned ll_sequence;
    float *ll_output;
    int ll_total;
    // ll_reduce > 0: the pair arrays hold ll_reduce slots of ll_total pairs, slot r filled by
    // rank r (this rank's own slot too); the tail adds the slots in order into ll_output
    int ll_reduce;
    // peer outputs of the pipelined kernel: a warp stores its results every `peer_flush`
    // finished rows (a power of two up to 32; 0 = 32).  32 rows make one 128-byte line per
    // store (NVLink peers); 8 keep a slow link (a page-locked host vector behind PCIe) busy
    // throughout the kernel instead of handing it the whole vector at the end.
    int peer_flush;
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
// kernel.  Two protocols (GemvParams::exchange), both on one 32-bit word per (receiver,
// sender) pair that starts at zero, and both bounded: a wait that runs out writes a status
// word and returns.  All ranks must run on different GPUs (they wait on one another).
//   kExchangeCounters  every CTA, once its stores are issued, adds its share of 2^20 to this
//       rank's word in every peer's memory (a system-wide fence orders the CTA's stores
//       before the adds; nothing comes back).  A launch adds exactly 2^20 per sender,
//       whatever its grid, so the n-th launch on a set of words is complete at a receiver
//       when the word has reached n * 2^20 (modulo 2^32); n comes from the rank's own word,
//       not from the host, so a launch can be replayed from a CUDA graph.  CTA 0 waits, one
//       lane per peer.  After the last row the critical path is one release and one trip
//       over the link.
//   kExchangeLastCta   every CTA publishes its stores system-wide and counts itself in a
//       device word; the last one writes the call's sequence number to the peers and waits
//       for theirs.  Needs no remote atomic: used when the "peer" is page-locked host memory.
constexpr unsigned kExchangeUnitsLog2 = 20;

__device__ __forceinline__ void peer_wait_word(const GemvParams &p, const unsigned *word,
    unsigned target) {
    const long long start = clock64();
    for (;;) {
        unsigned seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(word) : "memory");
        // the words only grow; the signed difference survives wrap-around
        if (static_cast<int>(seen - target) >= 0) break;
        if (clock64() - start > p.flag_wait_clocks) {   // about a second of SM clocks by default
            atomicExch(p.status, kStatusPeerFlagTimeout);
            break;
        }
    }
}

__device__ __forceinline__ void peer_allgather_tail(const GemvParams &p) {
    if (p.exchange == kExchangeOff) return;
    if (p.exchange == kExchangeCounters) {
        __syncthreads();                              // the whole CTA's stores are issued
        if (threadIdx.x < 32) {
            // one system-wide fence for the CTA (by lane 0, handed to the warp), then one
            // relaxed add per peer: a release on every add would fence once per peer
            if (threadIdx.x == 0) __threadfence_system();
            __syncwarp();
            if (threadIdx.x < p.peers) {
                // CTA 0 derives the launch's target from this rank's own word BEFORE adding
                // its share: all earlier launches of this rank have completed (stream order),
                // so the word holds (launches so far) * 2^20 plus what other CTAs of this
                // launch have added, which stays below 2^20 as long as this CTA's share is
                // missing.
                unsigned target = 0;
                if (blockIdx.x == 0) {
                    unsigned own;
                    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];"
                                 : "=r"(own) : "l"(p.my_flags + p.my_rank) : "memory");
                    target = ((own >> kExchangeUnitsLog2) + 1u) << kExchangeUnitsLog2;
                }
                const unsigned long long units = 1ull << kExchangeUnitsLog2;
                const unsigned share = static_cast<unsigned>(
                    (blockIdx.x + 1ull) * units / gridDim.x - blockIdx.x * units / gridDim.x);
                unsigned *remote = p.peer_flags[threadIdx.x] + p.my_rank;
                asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(remote), "r"(share)
                             : "memory");
                if (blockIdx.x == 0) peer_wait_word(p, p.my_flags + threadIdx.x, target);
            }
        }
        return;
    }
    __shared__ int is_last_cta;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned arrived = atomicAdd(p.cta_counter, 1u);
        is_last_cta = arrived == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last_cta) return;
    // one lane per peer: raise this rank's flag there, then wait for that peer's flag here
    if (threadIdx.x < p.peers) {
        unsigned *remote = p.peer_flags[threadIdx.x] + p.my_rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(p.sequence)
                     : "memory");
    }
    if (threadIdx.x == 0) *p.cta_counter = 0;         // ready for the next launch in the stream
    if (threadIdx.x < p.peers) peer_wait_word(p, p.my_flags + threadIdx.x, p.sequence);
}

// All-gather in which the data carries its own flag (the scheme of NCCL's low-latency
// protocol): a result travels as one aligned 8-byte store of (value bits, call number), which
// arrives whole, so the sender needs no fence and raises no flag, and the receiver knows a
// value has arrived when the number beside it is this call's.  After its rows every CTA helps
// to collect: it polls the pairs of the other ranks' slices in this rank's own array (bounded:
// a pair that does not arrive ends in a status word) and writes the values into the plain
// output vector.  The own slice goes there directly.  After the last row the critical path is
// one trip over the link.
__device__ __forceinline__ void ll_store(float *pairs, int index, float value, unsigned sequence) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(
                     reinterpret_cast<uint2 *>(pairs) + index),
                 "r"(__float_as_uint(value)), "r"(sequence)
                 : "memory");
}

// One result of this rank into every rank's memory: pairs for the others, the plain vector here.
__device__ __forceinline__ void peer_store(const GemvParams &p, int index, float value) {
    if (p.ll_sequence == 0) {
        for (int peer = 0; peer < p.peers; ++peer) p.peer_outputs[peer][index] = value;
        return;
    }
    for (int peer = 0; peer < p.peers; ++peer) {
        if (peer == p.my_rank && p.ll_reduce == 0) p.ll_output[index] = value;
        else ll_store(p.peer_outputs[peer], index, value, p.ll_sequence);
    }
}

// Bounded wait for pair `index` of this rank's own array; false when it ran out.
__device__ __forceinline__ bool ll_wait(const GemvParams &p, const uint2 *pairs, int index,
    long long start, float *value) {
    unsigned bits, number;
    for (;;) {
        asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];"
                     : "=r"(bits), "=r"(number) : "l"(pairs + index) : "memory");
        if (number == p.ll_sequence) break;
        if (clock64() - start > p.flag_wait_clocks) {
            atomicExch(p.status, kStatusPeerFlagTimeout);
            return false;
        }
    }
    *value = __uint_as_float(bits);
    return true;
}

__device__ __forceinline__ void ll_gather_tail(const GemvParams &p) {
    const long long start = clock64();
    const uint2 *pairs = reinterpret_cast<const uint2 *>(p.peer_outputs[p.my_rank]);
    if (p.ll_reduce > 0) {
        // partial vectors: out[i] = slot 0 + slot 1 + ... in slot order, the same on every rank
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.ll_total;
             i += gridDim.x * blockDim.x) {
            float total = 0.0f;
            for (int slot = 0; slot < p.ll_reduce; ++slot) {
                float value;
                if (!ll_wait(p, pairs, slot * p.ll_total + i, start, &value)) return;
                total = slot == 0 ? value : total + value;
            }
            p.ll_output[i] = total;
        }
        return;
    }
    const int own_begin = p.first_row, own_end = p.first_row + p.total_rows;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < p.ll_total;
         i += gridDim.x * blockDim.x) {
        if (i >= own_begin && i < own_end) continue;
        float value;
        if (!ll_wait(p, pairs, i, start, &value)) return;
        p.ll_output[i] = value;
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
                    peer_store(p, p.first_row + row, total);
                }
            }
        }
    }
    grid_dependents_may_launch();
    if (EPI == kEpiPeers) {
        if (p.ll_sequence) ll_gather_tail(p);
        else peer_allgather_tail(p);
    }
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
    // g + W, ...).  Peer outputs: warp g of the grid takes the contiguous run
    // [g * R / W, (g + 1) * R / W) - run lengths differ by at most one row, as with the
    // grid-stride order - keeps its results in its lanes (row i of the run in lane i mod 32)
    // and stores them to every peer a group at a time, so that the link carries whole
    // sectors or lines, spread over the kernel's duration.
    int row, row_step, row_end, warp_first = 0;
    // (Pairs with one other rank keep the ordinary row order, one 8-byte store per row:
    // 36.4 against 38.0 us per step on two GPUs.
    // With more peers a store per row and peer is too many small packets: 24.3 against 18.0 us
    // on eight GPUs.)
    const bool runs = EPI == kEpiPeers && (p.ll_sequence == 0 || p.peers > 2);
    if (runs) {
        const long long warps = static_cast<long long>(gridDim.x) * kGemvWarps;
        const long long g = static_cast<long long>(blockIdx.x) * kGemvWarps + warp_in_cta;
        warp_first = static_cast<int>(g * p.total_rows / warps);
        row = warp_first;
        row_step = 1;
        row_end = static_cast<int>((g + 1) * p.total_rows / warps);
    } else {
        row = blockIdx.x * kGemvWarps + warp_in_cta;
        row_step = gridDim.x * kGemvWarps;
        row_end = p.total_rows;
    }
    const size_t step = stride * row_step;
    const int flush_mask = (p.peer_flush > 0 ? p.peer_flush : 32) - 1;
    float held = 0.0f;
    int flushed = 0;

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
        if (runs) {
            // every lane holds the sum (butterfly); lane i mod 32 keeps row i of the run
            const int done = finished - warp_first + 1;
            if (lane == ((done - 1) & 31)) held = total[0];
            if ((done & flush_mask) == 0 || row >= row_end) {
                const int mine = flushed + ((lane - flushed) & 31);
                if (mine < done) {
                    peer_store(p, p.first_row + warp_first + mine, held);
                }
                flushed = done;
            }
        } else if (lane == 0) {
            if (EPI == kEpiSiluPair) {
                p.outputs[0][finished] = silu_mul(total[0], total[ROWS - 1]);
            } else if (EPI == kEpiPeers) {
                peer_store(p, p.first_row + finished, total[0]);
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
        if (p.ll_sequence) ll_gather_tail(p);
        else peer_allgather_tail(p);
    }
}

// --------------------------------------------------------------------------
// slice variant: few long rows (FFN down projections)
// --------------------------------------------------------------------------
// 5120 rows of 18.5 KB on 4736 resident warps are 1.08 rounds of a warp-per-row grid, and
// one warp cannot keep enough of an 18 KB row in flight.  Here SPLIT adjacent warps of a CTA
// share a row, as the reference's long-row kernel does with four warps
// (backend/cuda/fortai_cuda_backend.cu:88-126): each takes a contiguous slice of whole
// 512-element granules (at most G of them, the counts differing by at most one), with the
// pipelined kernel's structure - one request for the slice's scales, immediate offsets, the
// next row's slice requested as soon as the registers are free.  The SPLIT partial sums meet
// in shared memory and are added in slice order by the first warp of the row, so the result
// does not depend on timing.  Per half-block the arithmetic is that of the pipelined kernel.
template <int G>
__device__ __forceinline__ void slice_issue(RowRegs<G> &regs, const uint8_t *quants,
    const uint8_t *scales, int lane, int count) {
#pragma unroll
    for (int u = 0; u < G; ++u)
        if (u < count) regs.w[u] = ldg_stream_16(quants + u * 512);
    if (lane < 2 * count) regs.scales = ldg_stream_16(scales);
}

template <int G>
__device__ __forceinline__ float slice_consume(const RowRegs<G> &regs, const int4 *act_lane,
    const float *scale_lane, uint8_t *slot, int lane, int count) {
    if (lane < 2 * count) *reinterpret_cast<int4 *>(slot + lane * 16) = regs.scales;
    __syncwarp();
    float acc = 0.0f;
#pragma unroll
    for (int u = 0; u < G; ++u) {
        if (u < count) {
            const uint16_t dw =
                *reinterpret_cast<const uint16_t *>(slot + ((lane >> 1) + u * 16) * 2);
            const int4 a = act_lane[u * 32];
            const float sa = scale_lane[u * 16];
            acc = fmaf(half_bits_to_float(dw) * sa, static_cast<float>(dot16(regs.w[u], a)), acc);
        }
    }
    __syncwarp();
    return acc;
}

__host__ __device__ inline size_t slice_smem_bytes(int width, int blocks, int granules) {
    return activation_smem_bytes(width, blocks) +
        static_cast<size_t>(kGemvWarps) * (2 * granules * 16);
}

template <int G, int SPLIT, int ACT, int EPI>
__global__ void __launch_bounds__(kGemvThreads)
q8_gemv_slice_kernel(const __grid_constant__ GemvParams p) {
    if (p.trigger_early) grid_dependents_may_launch();
    extern __shared__ __align__(16) uint8_t gemv_smem[];
    __shared__ float partial[2][kGemvWarps];
    constexpr int ROWS_PER_ROUND = kGemvWarps / SPLIT;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int slice = warp % SPLIT;
    const int group = warp / SPLIT;
    const int granules = p.width >> 9;
    const int begin = slice * granules / SPLIT;
    const int count = (slice + 1) * granules / SPLIT - begin;      // <= G by the launcher
    const size_t stride = static_cast<size_t>(p.row_stride);
    uint8_t *slot = gemv_smem + activation_smem_bytes(p.width, p.blocks) + warp * (2 * G * 16);

    int row = blockIdx.x * ROWS_PER_ROUND + group;
    const int row_step = gridDim.x * ROWS_PER_ROUND;
    const size_t step = stride * row_step;
    const uint8_t *quants = p.weights[0] + row * stride + begin * 512 + lane * 16;
    const uint8_t *scales = p.weights[0] + row * stride + p.width + begin * 32 + lane * 16;
    RowRegs<G> cur;
    if (row < p.total_rows) slice_issue<G>(cur, quants, scales, lane, count);

    // the weight requests above do not depend on the previous kernel; everything below does
    grid_dependency_wait();
    stage_activation<ACT>(p.activation, p.width, p.blocks, gemv_smem, threadIdx.x, kGemvThreads);
    __syncthreads();
    const int4 *act_lane = reinterpret_cast<const int4 *>(gemv_smem) + begin * 32 + lane;
    const float *scale_lane =
        reinterpret_cast<const float *>(gemv_smem + p.width) + begin * 16 + (lane >> 1);

    int round = 0;
    while (row < p.total_rows) {
        float acc = slice_consume<G>(cur, act_lane, scale_lane, slot, lane, count);
        const int finished = row;
        row += row_step;
        quants += step;
        scales += step;
        if (row < p.total_rows) slice_issue<G>(cur, quants, scales, lane, count);
        acc = warp_sum(acc);
        if (lane == 0) partial[round & 1][warp] = acc;
        // the SPLIT warps of this row meet; two slots by round parity make one barrier enough
        asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(SPLIT * 32) : "memory");
        if (slice == 0 && lane == 0) {
            float total = partial[round & 1][warp];
#pragma unroll
            for (int s = 1; s < SPLIT; ++s) total += partial[round & 1][warp + s];
            if (EPI == kEpiPeers) {
                // few rows (a partial output vector): one word per row and peer
                peer_store(p, p.first_row + finished, total);
            } else {
                p.outputs[0][finished] = p.residual ? total + p.residual[finished] : total;
            }
        }
        ++round;
    }
    grid_dependents_may_launch();
    if (EPI == kEpiPeers) {
        if (p.ll_sequence) ll_gather_tail(p);
        else peer_allgather_tail(p);
    }
}

// `count` 16-byte pieces from page-locked host memory (through its device alias) into
// device memory: the host-call path's replacement for a copy-engine transfer of a few
// kilobytes.  Its dependent, the GEMV, may start at once.
__global__ void __launch_bounds__(1024)
q8_fetch_kernel(const float4 *__restrict__ source, float4 *__restrict__ destination, int count) {
    grid_dependents_may_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) destination[i] = source[i];
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
