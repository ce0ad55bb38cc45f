// Batched Q8_0 x Q8_0 product for multi-token prefill on the sm_100a tensor cores.
//
// out[t][r] = sum_b half(dw[r][b]) * half(da[t][b]) * (sum_i qw[r][b][i] * qa[t][b][i])
//
// The reference has no batched call (one token per forward,
// src/models/qwen35/fortai_qwen35_cpu.f90:591); parity is defined as `tokens`
// independent reference matvecs (src/fortai_gguf_runtime.f90:424-465), and the
// per-(token, row, block) int32 dots are the loop of
// src/backend/cpu/fortai_q8_dot.c:277-279.
//
// Mapping.  One `tcgen05.mma.kind::i8` has K = 32, exactly one Q8_0 block, so
// each MMA yields the exact int32 block dots of a 128 (weight rows) x 128
// (tokens) tile, written to a fresh TMEM accumulator (no accumulation across
// blocks, because every block has its own pair of scales).  Epilogue warps pull
// the accumulator out with tcgen05.ld, convert, scale by dw * da and add into
// fp32 registers, while the next blocks' MMAs run into the other TMEM buffers.
//
//   warp 0        TMA producer: 2-D tiled loads (128B swizzle) of 128 rows x 128
//                 K-bytes of weights and of activations per stage (= 4 blocks), and
//                 one 2-D load of activation scales per 16 blocks
//   warp 1        TMEM allocation, MMA issue (one elected thread), commits
//   warps 2..9    epilogue: warp w owns TMEM lanes 32*(w%4).. and 64 of the 128
//                 token columns; 64 fp32 accumulators per thread, updated with
//                 packed f32x2 multiply and fused multiply-add
//
// The grid is persistent (one CTA per SM); work is split in units of one stage of
// one tile so that every CTA gets the same number of units, and a tile that two
// CTAs share is completed with atomic adds onto zeroed output.
//
// TMEM: 512 columns = 4 accumulator buffers of 128 int32 columns.  All waits on
// mbarriers are bounded; a wait that gives up records a status word, raises the
// CTA's abort flag, and every role falls through to the common exit, where the
// TMEM allocation is released.
#pragma once

#include <cuda.h>

#ifndef FORTAI_MMQ_SPIN_WAITS
#define FORTAI_MMQ_SPIN_WAITS 0
#endif

#include "q8_common.cuh"

namespace fortai_b200 {

#ifdef FORTAI_MMQ_TRACE
// Debug builds only: clock64 stamps of CTA 0's three roles, for the first kTraceEvents
// hand-offs of each kind (role, event, slot).
constexpr int kTraceEvents = 96;
__device__ long long g_mmq_trace[3][kTraceEvents][6];
#define MMQ_STAMP(role, n, slot) \
    do { if (blockIdx.x == 0 && (n) < kTraceEvents) g_mmq_trace[role][n][slot] = clock64(); } while (0)
#else
#define MMQ_STAMP(role, n, slot) do { } while (0)
#endif

// Hand-offs between the roles of the kernel (see FORTAI_MMQ_SPIN_WAITS above).
__device__ __forceinline__ bool mmq_wait(uint64_t *bar, uint32_t parity) {
#if FORTAI_MMQ_SPIN_WAITS
    return mbar_wait_spin_bounded(bar, parity);
#else
    return mbar_wait_bounded(bar, parity);
#endif
}

constexpr int kMmqTileRows = 128;     // weight rows per CTA (MMA M)
constexpr int kMmqTileTokens = 128;   // tokens per CTA (MMA N)
constexpr int kMmqStageBlocks = 4;    // Q8_0 blocks per pipeline stage (128 K-bytes)
constexpr int kMmqStages = 4;
constexpr int kMmqTmemBuffers = 4;
#ifndef FORTAI_MMQ_EPILOGUE_WARPS
#define FORTAI_MMQ_EPILOGUE_WARPS 8
#endif
// Four TMEM lane quadrants x (128 / kMmqWarpColumns) column groups.  Eight warps of 64
// columns rather than sixteen of 32: the fixed cost of a drain step (barrier wait, fences,
// the load itself, the weight scale) is paid per warp and buffer, and ten warps may use
// 168 registers each where eighteen are held to 96.
constexpr int kMmqEpilogueWarps = FORTAI_MMQ_EPILOGUE_WARPS;
constexpr int kMmqWarpColumns = kMmqTileTokens / (kMmqEpilogueWarps / 4);
constexpr int kMmqThreads = (2 + kMmqEpilogueWarps) * 32;
constexpr int kMmqStageBytes = (kMmqTileRows + kMmqTileTokens) * 128;

struct MmqWeightsPlan {
    bool ready = false;
    CUtensorMap weights_map;
};

// ---- planar activation image in scratch -------------------------------------
//   [ tokens_padded x width int8 quants ][ blocks x tokens_padded float scales ]
// The scale plane is block-major so that a tile's 128 scales of one block are
// contiguous.
inline int mmq_padded_tokens(int tokens) {
    return (tokens + kMmqTileTokens - 1) / kMmqTileTokens * kMmqTileTokens;
}

inline size_t mmq_scratch_bytes(int width, int tokens) {
    const size_t padded = static_cast<size_t>(mmq_padded_tokens(tokens));
    return padded * width + padded * (width / kBlockElems) * sizeof(float);
}

inline bool mmq_supported(int rows, int width, int tokens, int min_tokens) {
    const int threshold = min_tokens > 0 ? min_tokens : 65;
    return tokens >= threshold && width % (kMmqStageBlocks * kBlockElems) == 0 && rows >= 1;
}

// ---- tcgen05 / TMA wrappers ---------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y,
    uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D(tmem) = A(smem) * B(smem)^T, int8 x int8 -> int32, fresh accumulator.
// (Tried and dropped: keeping the bias 0x4B400000 in every accumulator so that the int32
// result is already the float 12582912 + dot and the convert becomes one exact packed
// subtraction.  Restoring the bias with tcgen05.st after every drain lengthened the time a
// buffer is held and the kernel went from 93 us to 113 us at M = 512.)
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
    uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(0u)
        : "memory");
}

// Arrive on an mbarrier once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
          "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
          "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are
// 128 bytes apart, groups of 8 rows 1024 bytes apart (the stride byte offset);
// the leading byte offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(const void *tile) {
    uint64_t desc = (smem_u32(tile) >> 4) & 0x3fffu;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;   // stride byte offset
    desc |= 1ull << 46;                               // descriptor version for tcgen05
    desc |= 2ull << 61;                               // SWIZZLE_128B
    return desc;
}

// Instruction descriptor of kind::i8: D = s32, A = B = s8, both K-major.
__host__ __device__ constexpr uint32_t mmq_instr_desc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
        (static_cast<uint32_t>(m >> 4) << 24);
}

struct MmqParams {
    const uint8_t *weights;     // row-planar weight rows (for the fp16 scale plane)
    int rows;
    int width;
    int blocks;
    int row_stride;
    int tokens;
    int padded_tokens;
    int tiles_n;                // row tiles
    int tiles;                  // row tiles x token tiles
    int stages_per_tile;        // blocks / 4
    float *output;              // [tokens][rows]
    int32_t *block_dots;        // optional [tokens][rows][blocks]
    int *status;
};

// Work split.  The unit of work is one pipeline stage (4 blocks) of one 128 x 128
// tile; units are numbered tile-major and CTA c owns units
// [c * total / grid, (c + 1) * total / grid): equal shares whatever the tile count
// (304 tiles on 148 SMs would otherwise run as three waves, the last one 5 % full).
// A tile whose units fall to more than one CTA is "split": its pieces are added
// into zeroed output with atomics; other tiles are stored plainly.
__host__ __device__ inline long long mmq_unit_begin(long long total_units, int grid, int cta) {
    return total_units * cta / grid;
}

__host__ __device__ inline bool mmq_tile_is_split(long long total_units, int grid,
    int stages_per_tile, int tile) {
    const long long a = static_cast<long long>(tile) * stages_per_tile;
    const long long b = a + stages_per_tile;
    // first CTA whose range starts after a
    long long c = a * grid / total_units;
    for (long long k = c; k <= c + 2 && k <= grid; ++k) {
        const long long bound = total_units * k / grid;
        if (bound > a && bound < b) return true;
    }
    return false;
}

constexpr int kMmqScaleChunkBlocks = 16;   // activation-scale chunk: 16 blocks x 128 tokens
constexpr int kMmqScaleChunks = 4;
constexpr int kMmqScaleChunkBytes = kMmqScaleChunkBlocks * kMmqTileTokens * 4;

struct MmqShared {
    uint64_t smem_full[kMmqStages];
    uint64_t smem_empty[kMmqStages];
    uint64_t tmem_full[kMmqTmemBuffers];
    uint64_t tmem_empty[kMmqTmemBuffers];
    uint64_t scale_full[kMmqScaleChunks];
    uint64_t scale_empty[kMmqScaleChunks];
    uint32_t tmem_base;
    int abort_flag;
};

// Two floats as one 64-bit register pair.  mov.b64 lets ptxas put the halves in
// adjacent registers instead of assembling the pair with integer moves.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

// (float(a), float(b)) of two int32 accumulator words, packed.
__device__ __forceinline__ unsigned long long cvt2(uint32_t a, uint32_t b) {
    float lo, hi;
    asm("cvt.rn.f32.s32 %0, %1;" : "=f"(lo) : "r"(a));
    asm("cvt.rn.f32.s32 %0, %1;" : "=f"(hi) : "r"(b));
    return pack2(lo, hi);
}

__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
    unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// Ten warps (TMA, MMA, eight epilogue warps of 64 columns): up to 168 registers per thread.  A
// sixteen-warp epilogue would be 18 warps, allocated like 20 (groups of four): 96 per thread.
template <bool DOTS>
__global__ void __launch_bounds__(kMmqThreads, 1)
q8_mmq_kernel(const __grid_constant__ CUtensorMap weights_map,
    const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap scale_map,
    const __grid_constant__ MmqParams p) {
    extern __shared__ uint8_t mmq_smem_raw[];
    // [stages x (A 16 KB | B 16 KB)] [scale chunks: 4 x 8 KB] [barriers]
    // Swizzled tiles must start on a 1024-byte boundary: round the base up (the
    // launch reserves the slack).
    uint8_t *mmq_smem = mmq_smem_raw + ((1024u - (smem_u32(mmq_smem_raw) & 1023u)) & 1023u);
    uint8_t *stage_base = mmq_smem;
    uint8_t *scale_base = mmq_smem + kMmqStages * kMmqStageBytes;
    MmqShared *sh = reinterpret_cast<MmqShared *>(scale_base +
        kMmqScaleChunks * kMmqScaleChunkBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh->abort_flag;

    const long long total_units = static_cast<long long>(p.tiles) * p.stages_per_tile;
    const long long unit_begin = mmq_unit_begin(total_units, gridDim.x, blockIdx.x);
    const long long unit_end = mmq_unit_begin(total_units, gridDim.x, blockIdx.x + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMmqStages; ++s) {
            mbar_init(&sh->smem_full[s], 1);
            mbar_init(&sh->smem_empty[s], 1);
        }
        for (int b = 0; b < kMmqTmemBuffers; ++b) {
            mbar_init(&sh->tmem_full[b], 1);
            mbar_init(&sh->tmem_empty[b], kMmqEpilogueWarps);
        }
        for (int c = 0; c < kMmqScaleChunks; ++c) {
            mbar_init(&sh->scale_full[c], 1);
            mbar_init(&sh->scale_empty[c], kMmqEpilogueWarps);
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int armed = 0;          // stages armed so far (ring position)
            int chunks = 0;         // scale chunks armed so far
            bool failed = false;
            for (long long u = unit_begin; u < unit_end && !failed;) {
                const int tile = static_cast<int>(u / p.stages_per_tile);
                const int first_stage = static_cast<int>(u - static_cast<long long>(tile) *
                    p.stages_per_tile);
                const long long tile_end = static_cast<long long>(tile + 1) * p.stages_per_tile;
                const int count = static_cast<int>((tile_end < unit_end ? tile_end : unit_end) - u);
                const int row0 = (tile % p.tiles_n) * kMmqTileRows;
                const int token0 = (tile / p.tiles_n) * kMmqTileTokens;
                for (int i = 0; i < count; ++i) {
                    const int st = first_stage + i;
                    if ((i & 3) == 0) {
                        // activation scales of the next 16 blocks of this piece
                        const int c = chunks % kMmqScaleChunks;
                        const int use = chunks / kMmqScaleChunks;
                        if (use > 0 && !mmq_wait(&sh->scale_empty[c], (use - 1) & 1)) {
                            atomicExch(p.status, kStatusMmqLoadTimeout);
                            *abort_flag = 1;
                            failed = true;
                            break;
                        }
                        mbar_arrive_expect_tx(&sh->scale_full[c], kMmqScaleChunkBytes);
                        tma_load_2d(scale_base + c * kMmqScaleChunkBytes, &scale_map, token0,
                            st * kMmqStageBlocks, &sh->scale_full[c]);
                        ++chunks;
                    }
                    const int s = armed % kMmqStages;
                    const int use = armed / kMmqStages;
                    MMQ_STAMP(0, armed, 0);
                    if (use > 0 && !mmq_wait(&sh->smem_empty[s], (use - 1) & 1)) {
                        atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        failed = true;
                        break;
                    }
                    if (*abort_flag) {
                        failed = true;
                        break;
                    }
                    uint8_t *dst = stage_base + s * kMmqStageBytes;
                    mbar_arrive_expect_tx(&sh->smem_full[s], kMmqStageBytes);
                    tma_load_2d(dst, &weights_map, st * 128, row0, &sh->smem_full[s]);
                    tma_load_2d(dst + kMmqTileRows * 128, &act_map, st * 128, token0,
                        &sh->smem_full[s]);
                    MMQ_STAMP(0, armed, 1);
                    ++armed;
                }
                u += count;
            }
            if (failed || *abort_flag) {
                // let the loads that are still in flight land before the CTA ends
                const int lap = armed < kMmqStages ? armed : kMmqStages;
                for (int k = 0; k < lap; ++k) {
                    const int n = armed - 1 - k;
                    mbar_wait_bounded(&sh->smem_full[n % kMmqStages], (n / kMmqStages) & 1,
                        1u << 16);
                }
                const int clap = chunks < kMmqScaleChunks ? chunks : kMmqScaleChunks;
                for (int k = 0; k < clap; ++k) {
                    const int n = chunks - 1 - k;
                    mbar_wait_bounded(&sh->scale_full[n % kMmqScaleChunks],
                        (n / kMmqScaleChunks) & 1, 1u << 16);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = mmq_instr_desc(kMmqTileRows, kMmqTileTokens);
            bool failed = false;
            int consumed = 0;       // stages consumed (ring position)
            int issued = 0;         // MMAs issued (TMEM ring position)
            for (long long u = unit_begin; u < unit_end && !failed; ++u, ++consumed) {
                const int s = consumed % kMmqStages;
                MMQ_STAMP(1, consumed, 0);
                if (!mmq_wait(&sh->smem_full[s], (consumed / kMmqStages) & 1)) {
                    atomicExch(p.status, kStatusMmqLoadTimeout);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                MMQ_STAMP(1, consumed, 1);
                const uint8_t *tile = stage_base + s * kMmqStageBytes;
                const uint64_t desc_a = smem_desc_k_major_sw128(tile);
                const uint64_t desc_b = smem_desc_k_major_sw128(tile + kMmqTileRows * 128);
                for (int j = 0; j < kMmqStageBlocks; ++j, ++issued) {
                    const int buf = issued % kMmqTmemBuffers;
                    const int use = issued / kMmqTmemBuffers;
                    if (j == 0) MMQ_STAMP(1, consumed, 2);
                    if (use > 0) {
                        if (!mmq_wait(&sh->tmem_empty[buf], (use - 1) & 1)) {
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
                    // 32 K-bytes further inside the 128-byte swizzled row: +2 in
                    // units of 16 bytes on the descriptor's start address
                    mma_i8(tmem_base + buf * kMmqTileTokens, desc_a + 2 * j, desc_b + 2 * j,
                        idesc);
                    mma_commit(&sh->tmem_full[buf]);
                    if (j == 0) MMQ_STAMP(1, consumed, 3);
                }
                if (!failed) mma_commit(&sh->smem_empty[s]);
                MMQ_STAMP(1, consumed, 4);
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int ew = warp - 2;
        const int quadrant = warp & 3;              // TMEM lanes this warp may touch
        const int col0 = (ew >> 2) * kMmqWarpColumns;   // token columns of this warp
        constexpr int kPairs = kMmqWarpColumns / 2;
        unsigned long long acc[kPairs];             // fp32 accumulators, packed in pairs
        bool failed = false;
        int drained = 0;        // accumulators drained (TMEM ring position)
        int chunks = 0;         // scale chunks consumed
        for (long long u = unit_begin; u < unit_end && !failed;) {
            const int tile = static_cast<int>(u / p.stages_per_tile);
            const int first_stage = static_cast<int>(u - static_cast<long long>(tile) *
                p.stages_per_tile);
            const long long tile_end = static_cast<long long>(tile + 1) * p.stages_per_tile;
            const int count = static_cast<int>((tile_end < unit_end ? tile_end : unit_end) - u);
            const int row0 = (tile % p.tiles_n) * kMmqTileRows;
            const int token0 = (tile / p.tiles_n) * kMmqTileTokens;
            const int row = row0 + quadrant * 32 + lane;
            const bool row_ok = row < p.rows;
            const uint8_t *scale_plane = p.weights +
                static_cast<size_t>(row_ok ? row : 0) * p.row_stride + p.width;
#pragma unroll
            for (int i = 0; i < kPairs; ++i) acc[i] = 0ull;
            // The four fp16 weight scales of a stage are 8 aligned bytes of the row's
            // scale plane; they are fetched one stage ahead so that the L2 latency
            // hides behind a whole stage of drain work.
            uint2 dw_next = *reinterpret_cast<const uint2 *>(scale_plane +
                first_stage * kMmqStageBlocks * 2);

            for (int i = 0; i < count && !failed; ++i) {
                const int st = first_stage + i;
                const int chunk = (chunks + (i >> 2)) % kMmqScaleChunks;
                if ((i & 3) == 0) {
                    const int n = chunks + (i >> 2);
                    if (!mmq_wait(&sh->scale_full[chunk], (n / kMmqScaleChunks) & 1)) {
                        if (lane == 0) atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        failed = true;
                        break;
                    }
                }
                const uint2 dw4 = dw_next;
                if (i + 1 < count)
                    dw_next = *reinterpret_cast<const uint2 *>(scale_plane +
                        (st + 1) * kMmqStageBlocks * 2);
                const float *da_stage = reinterpret_cast<const float *>(scale_base +
                    chunk * kMmqScaleChunkBytes) + (i & 3) * kMmqStageBlocks * kMmqTileTokens;
#pragma unroll
                for (int j = 0; j < kMmqStageBlocks; ++j, ++drained) {
                    const int buf = drained % kMmqTmemBuffers;
                    const uint32_t parity = (drained / kMmqTmemBuffers) & 1;
                    const uint32_t taddr = tmem_base +
                        (static_cast<uint32_t>(quadrant * 32) << 16) + buf * kMmqTileTokens + col0;
                    if (warp == 2 && lane == 0) MMQ_STAMP(2, drained, 0);
                    if (!mmq_wait(&sh->tmem_full[buf], parity)) {
                        if (lane == 0) atomicExch(p.status, kStatusMmqMmaTimeout);
                        *abort_flag = 1;
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    if (warp == 2 && lane == 0) MMQ_STAMP(2, drained, 1);
                    // All of the warp's columns leave TMEM at once and the buffer is handed
                    // back before any arithmetic.  (Tried and dropped: draining in slabs of 32
                    // columns with the next slab in flight, and requesting the next
                    // accumulator's first slab before the last slab of this one is worked on -
                    // both were 5 % slower.  A clock64 trace (-DFORTAI_MMQ_TRACE) shows why: of
                    // the ~770 cycles a warp spends per block, the load and its wait are 37, the
                    // barrier wait ~130 and the arithmetic below ~520.)
                    constexpr int kSlabs = kMmqWarpColumns / 32;
                    uint32_t v[kSlabs][32];
#pragma unroll
                    for (int h = 0; h < kSlabs; ++h) tmem_load_32(taddr + 32 * h, v[h]);
                    tmem_load_wait();
                    if (warp == 2 && lane == 0) MMQ_STAMP(2, drained, 2);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
                    if (warp == 2 && lane == 0) MMQ_STAMP(2, drained, 3);

                    const uint32_t word = j < 2 ? dw4.x : dw4.y;
                    const float dw = half_bits_to_float(
                        static_cast<uint16_t>((j & 1) ? (word >> 16) : (word & 0xffffu)));
                    const unsigned long long dw2 = pack2(dw, dw);
                    // four activation scales per 16-byte load, read as two packed pairs
                    const ulonglong2 *da = reinterpret_cast<const ulonglong2 *>(da_stage +
                        j * kMmqTileTokens + col0);
#pragma unroll
                    for (int h = 0; h < kSlabs; ++h) {
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const ulonglong2 a = da[8 * h + q];
                            acc[16 * h + 2 * q] = fma2(cvt2(v[h][4 * q], v[h][4 * q + 1]),
                                mul2(dw2, a.x), acc[16 * h + 2 * q]);
                            acc[16 * h + 2 * q + 1] = fma2(cvt2(v[h][4 * q + 2], v[h][4 * q + 3]),
                                mul2(dw2, a.y), acc[16 * h + 2 * q + 1]);
                        }
                    }
                    if (warp == 2 && lane == 0) MMQ_STAMP(2, drained, 4);
                    if (DOTS && row_ok) {
                        const int kb = st * kMmqStageBlocks + j;
#pragma unroll
                        for (int e = 0; e < kMmqWarpColumns; ++e) {
                            const int t0 = token0 + col0 + e;
                            if (t0 < p.tokens)
                                p.block_dots[(static_cast<size_t>(t0) * p.rows + row) * p.blocks +
                                    kb] = static_cast<int>(v[e >> 5][e & 31]);
                        }
                    }
                }
                if (!failed && ((i & 3) == 3 || i == count - 1)) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->scale_empty[chunk]);
                }
            }
            chunks += (count + 3) >> 2;
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

// Before the product: the planar activation image, and zeros in the output of every
// split tile (their pieces arrive as atomic adds).
template <int ACT>
__global__ void __launch_bounds__(256)
mmq_prepare_kernel(const void *__restrict__ activation, int tokens, int padded_tokens, int width,
    int8_t *__restrict__ quants, float *__restrict__ scales, float *__restrict__ output, int rows,
    int tiles_n, int tiles, int stages_per_tile, int product_grid) {
    grid_dependents_may_launch();
    prepare_token_image<ACT>(activation, tokens, padded_tokens, width, quants, scales);
    if (!output) return;
    const long long total_units = static_cast<long long>(tiles) * stages_per_tile;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        if (!mmq_tile_is_split(total_units, product_grid, stages_per_tile, tile)) continue;
        const int row0 = (tile % tiles_n) * kMmqTileRows;
        const int token0 = (tile / tiles_n) * kMmqTileTokens;
        for (int i = threadIdx.x; i < kMmqTileRows * kMmqTileTokens; i += blockDim.x) {
            const int r = row0 + (i & (kMmqTileRows - 1));
            const int t = token0 + i / kMmqTileRows;
            if (r < rows && t < tokens) output[static_cast<size_t>(t) * rows + r] = 0.0f;
        }
    }
}

// ---- host side ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
    const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn mmq_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault,
                &result) == cudaSuccess && result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(entry);
    }
    return fn;
}

// fp32 matrix `rows` x `cols`, dense; boxes of 16 rows x 128 columns, no swizzle.
inline bool mmq_make_scale_map(CUtensorMap *map, const void *base, int rows, int cols) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * sizeof(float)};
    const cuuint32_t box[2] = {kMmqTileTokens, kMmqScaleChunkBlocks};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims,
               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

// int8 matrix, `rows` x `width` bytes, row pitch `pitch`; boxes of 128 rows x 128 bytes.
inline bool mmq_make_map(CUtensorMap *map, const void *base, int rows, int width, size_t pitch) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

inline cudaError_t mmq_reserve(void **aux, size_t *aux_bytes, int rows, int width, int tokens) {
    (void)rows;
    const size_t want = mmq_scratch_bytes(width, tokens);
    if (want <= *aux_bytes) return cudaSuccess;
    cudaError_t error = cudaFree(*aux);
    *aux = nullptr;
    *aux_bytes = 0;
    if (error != cudaSuccess) return error;
    error = cudaMalloc(aux, want);
    if (error == cudaSuccess) *aux_bytes = want;
    return error;
}

inline size_t mmq_smem_bytes() {
    return static_cast<size_t>(kMmqStages) * kMmqStageBytes +
        static_cast<size_t>(kMmqScaleChunks) * kMmqScaleChunkBytes + sizeof(MmqShared) + 64 +
        1024;
}

// activation: fp32 [tokens][width] (act == 1) or Q8_0 blocks (act == 0), device memory.
inline cudaError_t mmq_enqueue(cudaStream_t stream, int sm_count, int *status,
    MmqWeightsPlan *plan, const uint8_t *weights, int rows, int width, int row_stride,
    const void *activation, int act, int tokens, float *output, int32_t *block_dots, void **aux,
    size_t *aux_bytes, uint64_t *launches) {
    const int blocks = width / kBlockElems;
    const int padded = mmq_padded_tokens(tokens);
    cudaError_t error = mmq_reserve(aux, aux_bytes, rows, width, tokens);
    if (error != cudaSuccess) return error;
    int8_t *quants = static_cast<int8_t *>(*aux);
    float *scales = reinterpret_cast<float *>(quants + static_cast<size_t>(padded) * width);
    if (!plan->ready) {
        if (!mmq_make_map(&plan->weights_map, weights, rows, width, row_stride))
            return cudaErrorNotSupported;
        plan->ready = true;
    }
    CUtensorMap act_map, scale_map;
    if (!mmq_make_map(&act_map, quants, padded, width, width)) return cudaErrorNotSupported;
    if (!mmq_make_scale_map(&scale_map, scales, blocks, padded)) return cudaErrorNotSupported;

    MmqParams p = {};
    p.weights = weights;
    p.rows = rows;
    p.width = width;
    p.blocks = blocks;
    p.row_stride = row_stride;
    p.tokens = tokens;
    p.padded_tokens = padded;
    p.tiles_n = (rows + kMmqTileRows - 1) / kMmqTileRows;
    p.tiles = p.tiles_n * (padded / kMmqTileTokens);
    p.stages_per_tile = blocks / kMmqStageBlocks;
    p.output = output;
    p.block_dots = block_dots;
    p.status = status;
    const size_t smem = mmq_smem_bytes();
    const long long total_units = static_cast<long long>(p.tiles) * p.stages_per_tile;
    const int grid = static_cast<int>(std::min<long long>(sm_count, total_units));
    {
        const long long work = act == 1 ? static_cast<long long>(padded) * (width / 4) / 256
                                        : static_cast<long long>(padded) * blocks / 8;
        const int prep_grid = static_cast<int>(std::max<long long>(1,
            std::min<long long>(work + 1, static_cast<long long>(sm_count) * 8)));
        if (act == 1)
            mmq_prepare_kernel<1><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                quants, scales, output, rows, p.tiles_n, p.tiles, p.stages_per_tile, grid);
        else
            mmq_prepare_kernel<0><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                quants, scales, output, rows, p.tiles_n, p.tiles, p.stages_per_tile, grid);
        ++*launches;
        error = cudaGetLastError();
        if (error != cudaSuccess) return error;
    }
    // the product kernel may start (barriers, TMEM, descriptors) under the prepare kernel
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kMmqThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute overlap = {};
    overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    overlap.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &overlap;
    config.numAttrs = 1;
    if (block_dots) {
        error = cudaFuncSetAttribute(q8_mmq_kernel<true>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (error != cudaSuccess) return error;
        error = cudaLaunchKernelEx(&config, q8_mmq_kernel<true>, plan->weights_map, act_map,
            scale_map, p);
    } else {
        error = cudaFuncSetAttribute(q8_mmq_kernel<false>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (error != cudaSuccess) return error;
        error = cudaLaunchKernelEx(&config, q8_mmq_kernel<false>, plan->weights_map, act_map,
            scale_map, p);
    }
    if (error != cudaSuccess) return error;
    ++*launches;
    return cudaGetLastError();
}

#ifdef FORTAI_MMQ_TRACE
inline cudaError_t mmq_trace_read(long long *host) {
    return cudaMemcpyFromSymbol(host, g_mmq_trace, sizeof(g_mmq_trace));
}
#endif

}  // namespace fortai_b200
