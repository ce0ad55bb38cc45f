// Batched Q8_0 x Q8_0 product for multi-token prefill: tcgen05 tensor cores fed with the
// int8 quants widened to binary16, block dots exact in fp32, accumulators in TMEM.
//
// out[t][r] = sum_b half(dw[r][b]) * half(da[t][b]) * (sum_i qw[r][b][i] * qa[t][b][i])
//
// The reference has no batched call (one token per forward,
// src/models/qwen35/fortai_qwen35_cpu.f90:591); parity is defined as `tokens` independent
// reference matvecs (src/fortai_gguf_runtime.f90:424-465), and the per-(token, row, block)
// integer dots are the loop of src/backend/cpu/fortai_q8_dot.c:277-279.
//
// Why binary16 operands for an int8 product.  Every Q8_0 block has its own pair of scales,
// so a block's 32-element dot has to leave the tensor core before the next block is added
// to it, and every element of the accumulator tile costs CUDA-core work once per block.
// With kind::i8 that work is an int32 -> fp32 conversion (a quarter-rate instruction), a
// multiply and a fused multiply-add; the conversions alone take longer than the MMAs.  The
// quants are integers in [-127, 127], exact in binary16; their products and the sum of 32
// of them (|dot| <= 516 128 < 2^24) are exact in the fp32 accumulator of kind::f16.  The
// accumulator therefore holds the block dot already as a float: no conversion, and the
// int32 block dots that the parity probe returns are these floats converted back, exact.
// The tensor core runs at half its int8 rate, which is still twice as fast as the
// CUDA cores can scale what it produces.
//
// Tile: 128 weight rows (MMA M, TMEM lanes) x TN tokens (MMA N, TMEM columns), TN = 256
// for long prompts (an MMA takes 128 cycles whatever N is, so N = 256 is the only shape at
// full rate), 128 or 64 for short ones.  Two K = 16 MMAs per Q8_0 block.
//
//   warp 0        TMA producer: per stage (2 blocks = 64 K) the raw int8 weight tile
//                 (128 rows x 64 bytes) and the binary16 activation tile (TN x 64, 128-byte
//                 swizzle); per 8 blocks the activation scales (8 x TN floats)
//   warp 1        TMEM allocation, MMA issue (one elected thread), commits
//   warps 2..3    weight converters: int8 -> binary16 into the swizzled K-major operand tile
//   warps 4..11   epilogue: warp w owns TMEM lanes 32*(w%4).. and half of the token columns;
//                 TN/2 fp32 accumulators per thread, packed f32x2 multiply and FMA
//
// Registers: the first warpgroup gives registers back (setmaxnreg) so that the epilogue
// warpgroups can hold 128 accumulators and two 32-column slabs of a TMEM load per thread.
//
// The grid is persistent (one CTA per SM); work is split in units of one stage of one tile
// so that every CTA gets the same number of units, and a tile that two CTAs share is
// completed with atomic adds onto zeroed output.  All waits on mbarriers are bounded; a wait
// that gives up records a status word, raises the CTA's abort flag, and every role falls
// through to the common exit, where the TMEM allocation is released.
#pragma once

#include <cuda.h>

#include "q8_mmq.cuh"

namespace fortai_b200 {

constexpr int kPfTileRows = 128;
constexpr int kPfStageBlocks = 2;           // 64 K per stage: one 128-byte swizzle row of binary16
constexpr int kPfStageK = kPfStageBlocks * kBlockElems;
constexpr int kPfStages = 3;
constexpr int kPfChunkBlocks = 8;           // activation-scale chunk: 8 blocks x TN tokens
constexpr int kPfChunks = 3;
#ifndef FORTAI_PF_EPILOGUE_WARPS
#define FORTAI_PF_EPILOGUE_WARPS 16
#endif
#ifndef FORTAI_PF_SLAB_BUFFERS
#define FORTAI_PF_SLAB_BUFFERS 1
#endif
constexpr int kPfEpilogueWarps = FORTAI_PF_EPILOGUE_WARPS;   // 8 or 16: 4 TMEM lane quadrants x column groups
constexpr int kPfThreads = (4 + kPfEpilogueWarps) * 32;
#ifndef FORTAI_PF_PRODUCER_REGS
#define FORTAI_PF_PRODUCER_REGS 40
#endif
#ifndef FORTAI_PF_EPILOGUE_REGS
#define FORTAI_PF_EPILOGUE_REGS 104
#endif
#ifndef FORTAI_PF_SLAB
#define FORTAI_PF_SLAB 16
#endif
constexpr int kPfProducerRegs = FORTAI_PF_PRODUCER_REGS;   // registers per thread of the first warpgroup after the hand-over
constexpr int kPfEpilogueRegs = FORTAI_PF_EPILOGUE_REGS;   // and of the two epilogue warpgroups
constexpr int kPfSlab = FORTAI_PF_SLAB;                    // TMEM columns per tcgen05.ld
constexpr int kPfRawBytes = kPfTileRows * kPfStageK;            // int8 weight tile as loaded
constexpr int kPfW16Bytes = kPfTileRows * kPfStageK * 2;        // the same tile in binary16

__host__ __device__ constexpr int pf_stage_bytes(int tn) {
    return kPfW16Bytes + tn * kPfStageK * 2 + kPfRawBytes;
}
__host__ __device__ constexpr int pf_chunk_bytes(int tn) { return kPfChunkBlocks * tn * 4; }
__host__ __device__ constexpr int pf_tmem_buffers(int tn) { return tn >= 256 ? 2 : 4; }

inline int pf_tile_tokens(int tokens) { return tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256; }

inline int pf_padded_tokens(int tokens) {
    const int tn = pf_tile_tokens(tokens);
    return (tokens + tn - 1) / tn * tn;
}

// Planar activation image in scratch:
//   [ tokens_padded x width binary16 quants ][ blocks x tokens_padded float scales ]
inline size_t pf_scratch_bytes(int width, int tokens) {
    const size_t padded = static_cast<size_t>(pf_padded_tokens(tokens));
    return padded * width * 2 + padded * (width / kBlockElems) * sizeof(float);
}

inline bool pf_supported(int rows, int width, int tokens, int min_tokens) {
    const int threshold = min_tokens > 0 ? min_tokens : 33;
    return tokens >= threshold && width % kPfStageK == 0 && rows >= 1;
}

#ifdef FORTAI_PF_TRACE
// Debug builds only: clock64 stamps of CTA 0's roles (producer, MMA, converter, epilogue).
constexpr int kPfTraceEvents = 96;
__device__ long long g_pf_trace[4][kPfTraceEvents][6];
#define PF_STAMP(role, n, slot) \
    do { if (blockIdx.x == 0 && (n) < kPfTraceEvents) g_pf_trace[role][n][slot] = clock64(); } while (0)
#else
#define PF_STAMP(role, n, slot) do { } while (0)
#endif

struct PfWeightsPlan {
    bool ready = false;
    CUtensorMap weights_map;    // raw int8 quant plane, boxes of 128 rows x 64 bytes
};

struct PfParams {
    const uint8_t *weights;     // row-planar weight rows (for the fp16 scale plane)
    int rows;
    int width;
    int blocks;
    int row_stride;
    int tokens;
    int padded_tokens;
    int tiles_n;                // row tiles
    int tiles;                  // row tiles x token tiles
    int stages_per_tile;        // blocks / 2
    float *output;              // [tokens][rows]
    int32_t *block_dots;        // optional [tokens][rows][blocks]
    int *status;
};

struct PfShared {
    uint64_t full[kPfStages];           // TMA bytes of a stage have landed
    uint64_t converted[kPfStages];      // binary16 weight tile written
    uint64_t empty[kPfStages];          // the stage's MMAs have finished reading
    uint64_t tmem_full[4];
    uint64_t tmem_empty[4];
    uint64_t scale_full[kPfChunks];
    uint64_t scale_empty[kPfChunks];
    uint32_t tmem_base;
    int abort_flag;
};

// D(tmem) (+)= A(smem) * B(smem)^T, binary16 x binary16 -> fp32.
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
    uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor of kind::f16: D = f32, A = B = f16, both K-major.
__host__ __device__ constexpr uint32_t pf_instr_desc(int m, int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Four int8 -> two binary16 pairs, exact: the byte with its sign bit flipped is q + 128;
// OR-ed under the exponent of 1024 it is the binary16 number 1024 + 128 + q, and one packed
// subtraction of 1152 leaves q.
__device__ __forceinline__ void widen4(uint32_t q4, uint32_t &lo, uint32_t &hi) {
    const uint32_t biased = q4 ^ 0x80808080u;
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(biased), "r"(0x64646464u));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(biased), "r"(0x64646464u));
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(0x64806480u));
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(0x64806480u));
}

__device__ __forceinline__ unsigned long long pack_bits(uint32_t lo, uint32_t hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_load_slab(uint32_t taddr, uint32_t (&v)[32]) { tmem_load_32(taddr, v); }
__device__ __forceinline__ void tmem_load_slab(uint32_t taddr, uint32_t (&v)[16]) { tmem_load_16(taddr, v); }

template <int REGS>
__device__ __forceinline__ void regs_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void regs_claim() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

template <int TN, bool DOTS>
__global__ void __launch_bounds__(kPfThreads, 1)
q8_prefill_kernel(const __grid_constant__ CUtensorMap weights_map,
    const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap scale_map,
    const __grid_constant__ PfParams p) {
    constexpr int kStageBytes = pf_stage_bytes(TN);
    constexpr int kChunkBytes = pf_chunk_bytes(TN);
    constexpr int kBufs = pf_tmem_buffers(TN);
    constexpr int kBufStride = 512 / kBufs;             // TMEM columns per accumulator buffer
    constexpr uint32_t kStageTx = kPfRawBytes + TN * kPfStageK * 2;

    extern __shared__ uint8_t pf_smem_raw[];
    // [stages x (W16 16 KB | A16 TN*128 | raw 8 KB)] [scale chunks] [barriers]; swizzled
    // tiles start on 1024-byte boundaries (the launch reserves the slack).
    uint8_t *smem = pf_smem_raw + ((1024u - (smem_u32(pf_smem_raw) & 1023u)) & 1023u);
    uint8_t *scale_base = smem + kPfStages * kStageBytes;
    PfShared *sh = reinterpret_cast<PfShared *>(scale_base + kPfChunks * kChunkBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh->abort_flag;

    const long long total_units = static_cast<long long>(p.tiles) * p.stages_per_tile;
    const long long unit_begin = mmq_unit_begin(total_units, gridDim.x, blockIdx.x);
    const long long unit_end = mmq_unit_begin(total_units, gridDim.x, blockIdx.x + 1);
    const int unit_count = static_cast<int>(unit_end - unit_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPfStages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->converted[s], kPfEpilogueWarps);
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(&sh->tmem_full[b], 1);
            mbar_init(&sh->tmem_empty[b], kPfEpilogueWarps);
        }
        for (int c = 0; c < kPfChunks; ++c) {
            mbar_init(&sh->scale_full[c], 1);
            mbar_init(&sh->scale_empty[c], kPfEpilogueWarps);
        }
        sh->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    // everything above may run under the prepare kernel; the activation image, its scales
    // and the zeroed split tiles are that kernel's output
    grid_dependency_wait();

    if (warp < 4) {
        regs_release<kPfProducerRegs>();
        if (warp == 0) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                int armed = 0;          // stages armed so far (ring position)
                int chunks = 0;         // scale chunks armed so far
                bool failed = false;
                for (long long u = unit_begin; u < unit_end && !failed;) {
                    const int tile = static_cast<int>(u / p.stages_per_tile);
                    const int first_stage = static_cast<int>(u -
                        static_cast<long long>(tile) * p.stages_per_tile);
                    const long long tile_end = static_cast<long long>(tile + 1) * p.stages_per_tile;
                    const int count = static_cast<int>((tile_end < unit_end ? tile_end : unit_end) - u);
                    const int row0 = (tile % p.tiles_n) * kPfTileRows;
                    const int token0 = (tile / p.tiles_n) * TN;
                    for (int i = 0; i < count; ++i) {
                        const int st = first_stage + i;
                        const int kb = st * kPfStageBlocks;
                        if (i == 0 || (kb & (kPfChunkBlocks - 1)) == 0) {
                            const int c = chunks % kPfChunks;
                            const int use = chunks / kPfChunks;
                            if (use > 0 && !mbar_wait_bounded(&sh->scale_empty[c], (use - 1) & 1)) {
                                atomicExch(p.status, kStatusMmqLoadTimeout);
                                *abort_flag = 1;
                                failed = true;
                                break;
                            }
                            mbar_arrive_expect_tx(&sh->scale_full[c], kChunkBytes);
                            tma_load_2d(scale_base + c * kChunkBytes, &scale_map, token0,
                                kb & ~(kPfChunkBlocks - 1), &sh->scale_full[c]);
                            ++chunks;
                        }
                        const int s = armed % kPfStages;
                        const int use = armed / kPfStages;
                        PF_STAMP(0, armed, 0);
                        if (use > 0 && !mbar_wait_bounded(&sh->empty[s], (use - 1) & 1)) {
                            atomicExch(p.status, kStatusMmqLoadTimeout);
                            *abort_flag = 1;
                            failed = true;
                            break;
                        }
                        if (*abort_flag) {
                            failed = true;
                            break;
                        }
                        uint8_t *stage = smem + s * kStageBytes;
                        mbar_arrive_expect_tx(&sh->full[s], kStageTx);
                        tma_load_2d(stage + kPfW16Bytes + TN * kPfStageK * 2, &weights_map,
                            st * kPfStageK, row0, &sh->full[s]);
                        tma_load_2d(stage + kPfW16Bytes, &act_map, st * kPfStageK, token0,
                            &sh->full[s]);
                        PF_STAMP(0, armed, 1);
                        ++armed;
                    }
                    u += count;
                }
                if (failed || *abort_flag) {
                    // let the loads that are still in flight land before the CTA ends
                    const int lap = armed < kPfStages ? armed : kPfStages;
                    for (int k = 0; k < lap; ++k) {
                        const int n = armed - 1 - k;
                        mbar_wait_bounded(&sh->full[n % kPfStages], (n / kPfStages) & 1, 1u << 16);
                    }
                    const int clap = chunks < kPfChunks ? chunks : kPfChunks;
                    for (int k = 0; k < clap; ++k) {
                        const int n = chunks - 1 - k;
                        mbar_wait_bounded(&sh->scale_full[n % kPfChunks], (n / kPfChunks) & 1,
                            1u << 16);
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------ MMA issuer --------------------------------
            if (lane == 0) {
                const uint32_t idesc = pf_instr_desc(kPfTileRows, TN);
                bool failed = false;
                int issued = 0;         // blocks issued (TMEM ring position)
                for (int consumed = 0; consumed < unit_count && !failed; ++consumed) {
                    const int s = consumed % kPfStages;
                    const uint32_t parity = (consumed / kPfStages) & 1;
                    PF_STAMP(1, consumed, 0);
                    if (!mbar_wait_bounded(&sh->full[s], parity)) {
                        atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    PF_STAMP(1, consumed, 1);
                    if (!mbar_wait_bounded(&sh->converted[s], parity)) {
                        atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    tc_fence_after();
                    PF_STAMP(1, consumed, 2);
                    const uint8_t *stage = smem + s * kStageBytes;
                    const uint64_t desc_w = smem_desc_k_major_sw128(stage);
                    const uint64_t desc_a = smem_desc_k_major_sw128(stage + kPfW16Bytes);
#pragma unroll
                    for (int j = 0; j < kPfStageBlocks; ++j, ++issued) {
                        const int buf = issued % kBufs;
                        const int use = issued / kBufs;
                        if (use > 0) {
                            if (!mbar_wait_bounded(&sh->tmem_empty[buf], (use - 1) & 1)) {
                                atomicExch(p.status, kStatusMmqDrainTimeout);
                                *abort_flag = 1;
                                failed = true;
                                break;
                            }
                            tc_fence_after();
                        }
                        if (*abort_flag) {
                            failed = true;
                            break;
                        }
                        // a block is 64 bytes of the 128-byte swizzled row: two K = 16 steps
                        // of 32 bytes, +2 each in the descriptor's 16-byte units
                        const uint32_t d = tmem_base + buf * kBufStride;
                        if (j == 0) PF_STAMP(1, consumed, 3);
                        mma_f16(d, desc_w + 4 * j, desc_a + 4 * j, idesc, 0u);
                        mma_f16(d, desc_w + 4 * j + 2, desc_a + 4 * j + 2, idesc, 1u);
                        mma_commit(&sh->tmem_full[buf]);
                    }
                    if (!failed) mma_commit(&sh->empty[s]);
                    PF_STAMP(1, consumed, 4);
                }
            }
        }
    } else {
        // ---------------- weight conversion + epilogue (warps 4..) -------------------
        regs_claim<kPfEpilogueRegs>();
        const int ew = warp - 4;
        const int et = threadIdx.x - 128;           // 0 .. 32 * kPfEpilogueWarps - 1
        const int quadrant = warp & 3;              // TMEM lanes this warp may touch
        constexpr int kGroups = kPfEpilogueWarps / 4;
        constexpr int kCols = TN / kGroups;         // token columns of this warp
        constexpr int kSlab = kCols < kPfSlab ? kCols : kPfSlab;
        const int col0 = (ew >> 2) * kCols;
        constexpr int kPairs = kCols / 2;
        constexpr int kSlabs = kCols / kSlab;
        constexpr int kP = kSlab / 2;
        unsigned long long acc[kPairs];             // fp32 accumulators, packed in pairs
        bool failed = false;
        int drained = 0;        // accumulators drained (TMEM ring position)
        int chunks = 0;         // scale chunks taken so far
        int converted = 0;      // stages converted so far

        // int8 -> binary16 of one stage's weight tile: 16 raw bytes (16 K of one row) per
        // thread and step, into the 128-byte swizzled K-major tile the MMA reads.
        auto convert_stage = [&]() -> bool {
            const int s = converted % kPfStages;
            if (et == 0) PF_STAMP(2, converted, 0);
            if (!mbar_wait_bounded(&sh->full[s], (converted / kPfStages) & 1)) {
                if (lane == 0) atomicExch(p.status, kStatusMmqLoadTimeout);
                *abort_flag = 1;
                return false;
            }
            if (et == 0) PF_STAMP(2, converted, 1);
            uint8_t *stage = smem + s * kStageBytes;
            const uint8_t *raw = stage + kPfW16Bytes + TN * kPfStageK * 2;
            constexpr int kUnits = kPfRawBytes / 16;
            constexpr int kThreads = kPfEpilogueWarps * 32;
#pragma unroll
            for (int q = 0; q < kUnits / kThreads; ++q) {
                const int unit = et + kThreads * q;
                const int r = unit >> 2;
                const int c16 = unit & 3;
                const uint4 x = *reinterpret_cast<const uint4 *>(raw + r * kPfStageK + c16 * 16);
                uint4 h0, h1;
                widen4(x.x, h0.x, h0.y);
                widen4(x.y, h0.z, h0.w);
                widen4(x.z, h1.x, h1.y);
                widen4(x.w, h1.z, h1.w);
                // 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r & 7)
                uint8_t *row = stage + r * 128;
                *reinterpret_cast<uint4 *>(row + (((2 * c16) ^ (r & 7)) << 4)) = h0;
                *reinterpret_cast<uint4 *>(row + (((2 * c16 + 1) ^ (r & 7)) << 4)) = h1;
            }
            // generic-proxy writes must be visible to the tensor core's async-proxy reads
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->converted[s]);
            if (et == 0) PF_STAMP(2, converted, 2);
            ++converted;
            return true;
        };

        // conversion runs two stages ahead of the drain
        for (int k = 0; k < 2 && k < unit_count && !failed; ++k) failed = !convert_stage();

        for (long long u = unit_begin; u < unit_end && !failed;) {
            const int tile = static_cast<int>(u / p.stages_per_tile);
            const int first_stage = static_cast<int>(u - static_cast<long long>(tile) *
                p.stages_per_tile);
            const long long tile_end = static_cast<long long>(tile + 1) * p.stages_per_tile;
            const int count = static_cast<int>((tile_end < unit_end ? tile_end : unit_end) - u);
            const int row0 = (tile % p.tiles_n) * kPfTileRows;
            const int token0 = (tile / p.tiles_n) * TN;
            const int row = row0 + quadrant * 32 + lane;
            const bool row_ok = row < p.rows;
            const uint8_t *scale_plane = p.weights +
                static_cast<size_t>(row_ok ? row : 0) * p.row_stride + p.width;
#pragma unroll
            for (int i = 0; i < kPairs; ++i) acc[i] = 0ull;
            // the two fp16 weight scales of a stage are 4 aligned bytes of the row's scale
            // plane, fetched one stage ahead
            uint32_t dw_next = *reinterpret_cast<const uint32_t *>(scale_plane +
                first_stage * kPfStageBlocks * 2);
            int chunk = 0;

            for (int i = 0; i < count && !failed; ++i) {
                const int st = first_stage + i;
                const int kb = st * kPfStageBlocks;
                if (i == 0 || (kb & (kPfChunkBlocks - 1)) == 0) {
                    chunk = chunks % kPfChunks;
                    if (!mbar_wait_bounded(&sh->scale_full[chunk], (chunks / kPfChunks) & 1)) {
                        if (lane == 0) atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        failed = true;
                        break;
                    }
                    ++chunks;
                }
                const uint32_t dw_pair = dw_next;
                if (i + 1 < count)
                    dw_next = *reinterpret_cast<const uint32_t *>(scale_plane +
                        (st + 1) * kPfStageBlocks * 2);
#pragma unroll
                for (int j = 0; j < kPfStageBlocks; ++j, ++drained) {
                    const int buf = drained % kBufs;
                    const uint32_t parity = (drained / kBufs) & 1;
                    const uint32_t taddr = tmem_base +
                        (static_cast<uint32_t>(quadrant * 32) << 16) + buf * kBufStride + col0;
                    if (et == 0) PF_STAMP(3, drained, 0);
                    if (!mbar_wait_bounded(&sh->tmem_full[buf], parity)) {
                        if (lane == 0) atomicExch(p.status, kStatusMmqMmaTimeout);
                        *abort_flag = 1;
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    if (et == 0) PF_STAMP(3, drained, 1);
                    const float dw = half_bits_to_float(
                        static_cast<uint16_t>(j ? (dw_pair >> 16) : (dw_pair & 0xffffu)));
                    const unsigned long long dw2 = pack2(dw, dw);
                    const float *da_row = reinterpret_cast<const float *>(scale_base +
                        chunk * kChunkBytes) + ((kb + j) & (kPfChunkBlocks - 1)) * TN + col0;
                    // Slabs of kSlab columns; with two buffers the next slab is requested
                    // before this one is worked on.  The accumulator buffer goes back to the
                    // MMA warp as soon as the last slab has left TMEM.
                    constexpr int kDepth = FORTAI_PF_SLAB_BUFFERS;
                    uint32_t v[kDepth][kSlab];
                    if (kDepth == 2) tmem_load_slab(taddr, v[0]);
#pragma unroll
                    for (int h = 0; h < kSlabs; ++h) {
                        if (kDepth == 1) tmem_load_slab(taddr + kSlab * h, v[0]);
                        tmem_load_wait();
                        if (kDepth == 2 && h + 1 < kSlabs)
                            tmem_load_slab(taddr + kSlab * (h + 1), v[(h + 1) & 1]);
                        if (h + 1 == kSlabs) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
                            if (et == 0) PF_STAMP(3, drained, 2);
                        }
                        const uint32_t (&vv)[kSlab] = v[kDepth == 2 ? (h & 1) : 0];
#ifndef FORTAI_PF_NO_MATH
                        const ulonglong2 *da = reinterpret_cast<const ulonglong2 *>(da_row + kSlab * h);
#pragma unroll
                        for (int q = 0; q < kSlab / 4; ++q) {
                            const ulonglong2 a = da[q];
#ifdef FORTAI_PF_SCALAR
                            float a0, a1, a2, a3, c0, c1, c2, c3;
                            unpack2(a.x, a0, a1);
                            unpack2(a.y, a2, a3);
                            unpack2(acc[kP * h + 2 * q], c0, c1);
                            unpack2(acc[kP * h + 2 * q + 1], c2, c3);
                            c0 = fmaf(__uint_as_float(vv[4 * q]), dw * a0, c0);
                            c1 = fmaf(__uint_as_float(vv[4 * q + 1]), dw * a1, c1);
                            c2 = fmaf(__uint_as_float(vv[4 * q + 2]), dw * a2, c2);
                            c3 = fmaf(__uint_as_float(vv[4 * q + 3]), dw * a3, c3);
                            acc[kP * h + 2 * q] = pack2(c0, c1);
                            acc[kP * h + 2 * q + 1] = pack2(c2, c3);
#else
                            acc[kP * h + 2 * q] = fma2(pack_bits(vv[4 * q], vv[4 * q + 1]),
                                mul2(dw2, a.x), acc[kP * h + 2 * q]);
                            acc[kP * h + 2 * q + 1] = fma2(pack_bits(vv[4 * q + 2], vv[4 * q + 3]),
                                mul2(dw2, a.y), acc[kP * h + 2 * q + 1]);
#endif
                        }
#else
                        acc[h] ^= vv[0];
#endif
                        if (DOTS && row_ok) {
#pragma unroll
                            for (int e = 0; e < kSlab; ++e) {
                                const int t0 = token0 + col0 + kSlab * h + e;
                                if (t0 < p.tokens)
                                    p.block_dots[(static_cast<size_t>(t0) * p.rows + row) *
                                        p.blocks + kb + j] = __float2int_rn(__uint_as_float(vv[e]));
                            }
                        }
                    }
                    if (et == 0) PF_STAMP(3, drained, 3);
                }
                if (!failed && (((kb + kPfStageBlocks) & (kPfChunkBlocks - 1)) == 0 ||
                        i == count - 1)) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->scale_empty[chunk]);
                }
                if (!failed && converted < unit_count) failed = !convert_stage();
            }
            if (!failed && row_ok && p.output) {
                const bool split = count != p.stages_per_tile;
#pragma unroll
                for (int e = 0; e < kPairs; ++e) {
                    const int t = token0 + col0 + 2 * e;
                    float lo, hi;
                    unpack2(acc[e], lo, hi);
                    float *dst = p.output + static_cast<size_t>(t) * p.rows + row;
                    if (split) {
                        if (t < p.tokens) atomicAdd(dst, lo);
                        if (t + 1 < p.tokens) atomicAdd(dst + p.rows, hi);
                    } else {
                        if (t < p.tokens) *dst = lo;
                        if (t + 1 < p.tokens) dst[p.rows] = hi;
                    }
                }
            }
            u += count;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- activation image of several tokens, quants widened to binary16 ---------------------
// quants[token][width] binary16 and scales[block][padded_tokens] float for `padded_tokens`
// rows (rows >= tokens are zero), from fp32 rows (ACT == 1: eight lanes per Q8_0 block, same
// arithmetic and bytes as quantize_lane) or from GGUF Q8_0 rows (ACT == 0).  Also zeroes the
// output of every split tile (their pieces arrive as atomic adds).
template <int ACT>
__global__ void __launch_bounds__(256)
pf_prepare_kernel(const void *__restrict__ activation, int tokens, int padded_tokens, int width,
    __half *__restrict__ quants, float *__restrict__ scales, float *__restrict__ output, int rows,
    int tile_tokens, int tiles_n, int tiles, int stages_per_tile, int product_grid) {
    grid_dependents_may_launch();
    const int blocks = width / kBlockElems;
    if (ACT == 1) {
        const float4 *x4 = static_cast<const float4 *>(activation);
        uint2 *q64 = reinterpret_cast<uint2 *>(quants);
        const int groups = width >> 2;                       // float4 per token, 8 per block
        const long long total = static_cast<long long>(padded_tokens) * groups;
        const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
        // warp-uniform trip count: the shuffles below need all 32 lanes
        for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x; base < total;
             base += stride) {
            const long long at = base + threadIdx.x;
            const bool valid = at < total;
            const int token = valid ? static_cast<int>(at / groups) : 0;
            const int g = valid ? static_cast<int>(at - static_cast<long long>(token) * groups) : 0;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (valid && token < tokens) v = x4[static_cast<size_t>(token) * groups + g];
            float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            const float scale = __fdiv_rn(amax, 127.0f);
            const float inverse = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            const int q0 = max(-128, min(127, __float2int_rn(__fmul_rn(v.x, inverse))));
            const int q1 = max(-128, min(127, __float2int_rn(__fmul_rn(v.y, inverse))));
            const int q2 = max(-128, min(127, __float2int_rn(__fmul_rn(v.z, inverse))));
            const int q3 = max(-128, min(127, __float2int_rn(__fmul_rn(v.w, inverse))));
            if (valid) {
                const __half2 lo = __floats2half2_rn(static_cast<float>(q0), static_cast<float>(q1));
                const __half2 hi = __floats2half2_rn(static_cast<float>(q2), static_cast<float>(q3));
                q64[static_cast<size_t>(token) * groups + g] = make_uint2(
                    *reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
                if ((g & 7) == 0)
                    scales[static_cast<size_t>(g >> 3) * padded_tokens + token] =
                        half_bits_to_float(__half_as_ushort(__float2half_rn(scale)));
            }
        }
    } else {
        const int lane = threadIdx.x & 31;
        const long long total = static_cast<long long>(padded_tokens) * blocks;
        for (long long i = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); i < total;
             i += static_cast<long long>(gridDim.x) * 8) {
            const int token = static_cast<int>(i / blocks);
            const int b = static_cast<int>(i - static_cast<long long>(token) * blocks);
            int q = 0;
            float scale = 0.0f;
            if (token < tokens) {
                const uint8_t *block = static_cast<const uint8_t *>(activation) +
                    (static_cast<size_t>(token) * blocks + b) * kBlockBytes;
                q = static_cast<int8_t>(block[2 + lane]);
                scale = half_bits_to_float(*reinterpret_cast<const uint16_t *>(block));
            }
            quants[static_cast<size_t>(token) * width + b * kBlockElems + lane] =
                __float2half_rn(static_cast<float>(q));
            if (lane == 0) scales[static_cast<size_t>(b) * padded_tokens + token] = scale;
        }
    }
    if (!output) return;
    const long long total_units = static_cast<long long>(tiles) * stages_per_tile;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        if (!mmq_tile_is_split(total_units, product_grid, stages_per_tile, tile)) continue;
        const int row0 = (tile % tiles_n) * kPfTileRows;
        const int token0 = (tile / tiles_n) * tile_tokens;
        for (int i = threadIdx.x; i < kPfTileRows * tile_tokens; i += blockDim.x) {
            const int r = row0 + (i & (kPfTileRows - 1));
            const int t = token0 + i / kPfTileRows;
            if (r < rows && t < tokens) output[static_cast<size_t>(t) * rows + r] = 0.0f;
        }
    }
}

// ---- host side ----------------------------------------------------------------
// uint8 matrix `rows` x `width` bytes, row pitch `pitch`; boxes of 128 rows x 64 bytes, dense.
inline bool pf_make_raw_map(CUtensorMap *map, const void *base, int rows, int width, size_t pitch) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
    const cuuint32_t box[2] = {kPfStageK, kPfTileRows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

// binary16 matrix `rows` x `width`, dense; boxes of `box_rows` rows x 64 elements, 128-byte swizzle.
inline bool pf_make_act_map(CUtensorMap *map, const void *base, int rows, int width, int box_rows) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(width) * 2};
    const cuuint32_t box[2] = {kPfStageK, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

// fp32 matrix `rows` (blocks) x `cols` (tokens), dense; boxes of 8 rows x `box_cols`, no swizzle.
inline bool pf_make_scale_map(CUtensorMap *map, const void *base, int rows, int cols, int box_cols) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(float)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), kPfChunkBlocks};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims,
               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

inline cudaError_t pf_reserve(void **aux, size_t *aux_bytes, int width, int tokens) {
    const size_t want = pf_scratch_bytes(width, tokens);
    if (want <= *aux_bytes) return cudaSuccess;
    cudaError_t error = cudaFree(*aux);
    *aux = nullptr;
    *aux_bytes = 0;
    if (error != cudaSuccess) return error;
    error = cudaMalloc(aux, want);
    if (error == cudaSuccess) *aux_bytes = want;
    return error;
}

inline size_t pf_smem_bytes(int tn) {
    return static_cast<size_t>(kPfStages) * pf_stage_bytes(tn) +
        static_cast<size_t>(kPfChunks) * pf_chunk_bytes(tn) + sizeof(PfShared) + 64 + 1024;
}

template <int TN, bool DOTS>
inline cudaError_t pf_launch(const cudaLaunchConfig_t &config, const CUtensorMap &weights_map,
    const CUtensorMap &act_map, const CUtensorMap &scale_map, const PfParams &p) {
    static bool configured[16] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 16 && !configured[device]) {
        // The register hand-over inside the kernel (setmaxnreg) only works if the CTA was
        // given the pool it redistributes; a build that allocates fewer registers per
        // thread would wait for registers that never come, so refuse it here.
        cudaFuncAttributes attributes;
        cudaError_t error = cudaFuncGetAttributes(&attributes, q8_prefill_kernel<TN, DOTS>);
        if (error != cudaSuccess) return error;
        if (attributes.numRegs * kPfThreads < 128 * kPfProducerRegs + 32 * kPfEpilogueWarps * kPfEpilogueRegs)
            return cudaErrorLaunchOutOfResources;
        error = cudaFuncSetAttribute(q8_prefill_kernel<TN, DOTS>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pf_smem_bytes(TN)));
        if (error != cudaSuccess) return error;
        configured[device] = true;
    }
    return cudaLaunchKernelEx(&config, q8_prefill_kernel<TN, DOTS>, weights_map, act_map,
        scale_map, p);
}

// activation: fp32 [tokens][width] (act == 1) or Q8_0 blocks (act == 0), device memory.
inline cudaError_t pf_enqueue(cudaStream_t stream, int sm_count, int *status, PfWeightsPlan *plan,
    const uint8_t *weights, int rows, int width, int row_stride, const void *activation, int act,
    int tokens, float *output, int32_t *block_dots, void **aux, size_t *aux_bytes,
    uint64_t *launches) {
    const int blocks = width / kBlockElems;
    const int tn = pf_tile_tokens(tokens);
    const int padded = pf_padded_tokens(tokens);
    cudaError_t error = pf_reserve(aux, aux_bytes, width, tokens);
    if (error != cudaSuccess) return error;
    __half *quants = static_cast<__half *>(*aux);
    float *scales = reinterpret_cast<float *>(quants + static_cast<size_t>(padded) * width);
    if (!plan->ready) {
        if (!pf_make_raw_map(&plan->weights_map, weights, rows, width, row_stride))
            return cudaErrorNotSupported;
        plan->ready = true;
    }
    CUtensorMap act_map, scale_map;
    if (!pf_make_act_map(&act_map, quants, padded, width, tn)) return cudaErrorNotSupported;
    if (!pf_make_scale_map(&scale_map, scales, blocks, padded, tn)) return cudaErrorNotSupported;

    PfParams p = {};
    p.weights = weights;
    p.rows = rows;
    p.width = width;
    p.blocks = blocks;
    p.row_stride = row_stride;
    p.tokens = tokens;
    p.padded_tokens = padded;
    p.tiles_n = (rows + kPfTileRows - 1) / kPfTileRows;
    p.tiles = p.tiles_n * (padded / tn);
    p.stages_per_tile = blocks / kPfStageBlocks;
    p.output = output;
    p.block_dots = block_dots;
    p.status = status;
    const long long total_units = static_cast<long long>(p.tiles) * p.stages_per_tile;
    const int grid = static_cast<int>(std::min<long long>(sm_count, total_units));
    {
        const long long work = act == 1 ? static_cast<long long>(padded) * (width / 4) / 256
                                        : static_cast<long long>(padded) * blocks / 8;
        const int prep_grid = static_cast<int>(std::max<long long>(1,
            std::min<long long>(work + 1, static_cast<long long>(sm_count) * 8)));
        if (act == 1)
            pf_prepare_kernel<1><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                quants, scales, output, rows, tn, p.tiles_n, p.tiles, p.stages_per_tile, grid);
        else
            pf_prepare_kernel<0><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                quants, scales, output, rows, tn, p.tiles_n, p.tiles, p.stages_per_tile, grid);
        ++*launches;
        error = cudaGetLastError();
        if (error != cudaSuccess) return error;
    }
    // the product kernel may start (barriers, TMEM, descriptors) under the prepare kernel
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kPfThreads);
    config.dynamicSmemBytes = pf_smem_bytes(tn);
    config.stream = stream;
    cudaLaunchAttribute overlap = {};
    overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    overlap.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &overlap;
    config.numAttrs = 1;
    const bool dots = block_dots != nullptr;
    if (tn == 256)
        error = dots ? pf_launch<256, true>(config, plan->weights_map, act_map, scale_map, p)
                     : pf_launch<256, false>(config, plan->weights_map, act_map, scale_map, p);
    else if (tn == 128)
        error = dots ? pf_launch<128, true>(config, plan->weights_map, act_map, scale_map, p)
                     : pf_launch<128, false>(config, plan->weights_map, act_map, scale_map, p);
    else
        error = dots ? pf_launch<64, true>(config, plan->weights_map, act_map, scale_map, p)
                     : pf_launch<64, false>(config, plan->weights_map, act_map, scale_map, p);
    if (error != cudaSuccess) return error;
    ++*launches;
    return cudaGetLastError();
}

}  // namespace fortai_b200
