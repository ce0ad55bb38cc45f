// Batched Q8_0 x Q8_0 product for multi-token prefill on the sm_100a tensor cores, with the
// activation scale folded into the tensor-core operand.
//
// out[t][r] = sum_b half(dw[r][b]) * half(da[t][b]) * (sum_i qw[r][b][i] * qa[t][b][i])
//
// The reference has no batched call (one token per forward,
// src/models/qwen35/fortai_qwen35_cpu.f90:591); parity is defined as `tokens` independent
// reference matvecs (src/fortai_gguf_runtime.f90:424-465).
//
// Why not kind::i8 with one scaling step per block.  Every Q8_0 block has its own pair of
// scales, so a block's dot has to be scaled before the next block is added to it.  Doing
// that on the CUDA cores costs, per accumulator element and block, a conversion (quarter
// rate), a multiply and an FMA, and - whichever way the tile is laid out - one of the two
// scales is the same for all lanes of a warp and has to be fetched through the load/store
// unit, whose return path moves 128 bytes per clock: 1024 cycles per block of 128 x 256
// elements against 128 cycles of int8 MMA (q8_mmq.cuh is that kernel; it is kept as the
// exact-int32-block-dot probe).
//
// Here the activation scale goes into the operand instead.  da * qa (binary16 scale x 7-bit
// quant) has at most 18 significant bits, so it is the exact sum of two binary16 numbers,
// hi = rn16(da * qa) and lo = da * qa - hi; the prepare kernel writes both once per call,
// scaled per token by a power of two so that neither overflows nor leaves the binary16
// range.  The int8 weights are widened to binary16 (exact) on their way through shared
// memory.  Four kind::f16 MMAs per block (K = 16 each: two over hi, two over lo) leave
// sum_i qw * (da * qa) in a fresh fp32 TMEM accumulator, and what is left for the CUDA cores
// is one packed FMA per two elements and block with the weight scale, which each thread
// owns (a thread is a weight row): no conversion, no multiply, no shared-memory traffic.
// The fp32 results differ from the int32 formulation only by the rounding of the tensor
// core's fp32 accumulation (about 1e-7 relative per block), far inside the 1e-5 * L2 bound;
// this path has no int32 block dots.
//
// Tile: 128 weight rows (MMA M, TMEM lanes) x TN tokens (MMA N, TMEM columns), TN = 256
// for long prompts (an MMA takes 128 cycles whatever N is, so N = 256 is the only shape at
// full rate), 128 or 64 for short ones.
//
//   warps 0, 3    TMA producers (even / odd blocks): per block the CTA's half of the
//                 activation tile (TN/2 x [32 hi | 32 lo] binary16, 128-byte swizzle); per
//                 four blocks the raw int8 weight tile (128 rows x 128 bytes)
//   warps 1, 2    MMA issue (one elected thread each, even / odd blocks), commits; warp 1
//                 also owns the TMEM allocation
//   warps 4..7    int8 -> binary16 of the weight tile into the swizzled K-major operand
//                 tile, each warp every fourth block
//   warps 8..23   the drain: warp w owns TMEM lanes 32*(w%4).. and a quarter of the token
//                 columns
//
// Registers: the first two warpgroups give registers back (setmaxnreg) to the sixteen
// drain warps.  The grid is persistent (one CTA per SM); work is split in units of one block of
// one tile so that every CTA gets the same number of units, and a tile that two CTAs share
// is completed with atomic adds onto zeroed output.  All waits on mbarriers are bounded; a
// wait that gives up records a status word, raises the CTA's abort flag, and every role
// falls through to the common exit, where the TMEM allocation is released.
#pragma once

#include <cuda.h>

#include "q8_mmq.cuh"

namespace fortai_b200 {

#ifndef FORTAI_PF_PRODUCER_REGS
#define FORTAI_PF_PRODUCER_REGS 48
#endif
#ifndef FORTAI_PF_CONVERTER_REGS
#define FORTAI_PF_CONVERTER_REGS 48
#endif
#ifndef FORTAI_PF_EPILOGUE_REGS
#define FORTAI_PF_EPILOGUE_REGS 96
#endif
#ifndef FORTAI_PF_SLAB
#define FORTAI_PF_SLAB 16
#endif

constexpr int kPfTileRows = 128;            // weight rows per CTA (TMEM lanes)
constexpr int kPfPairRows = 256;            // weight rows per CTA pair (MMA M with cta_group::2)
constexpr int kPfMaxStages = 8;
constexpr int kPfEpilogueWarps = 16;        // 4 TMEM lane quadrants x 4 column groups
constexpr int kPfFrontWarps = 8;            // producer, two MMA issuers, a spare, four converters
constexpr int kPfConverterWarps = 4;
constexpr int kPfThreads = (kPfFrontWarps + kPfEpilogueWarps) * 32;
constexpr int kPfProducerRegs = FORTAI_PF_PRODUCER_REGS;   // per thread of the first warpgroup after the hand-over
constexpr int kPfConverterRegs = FORTAI_PF_CONVERTER_REGS; // of the converter warpgroup
constexpr int kPfEpilogueRegs = FORTAI_PF_EPILOGUE_REGS;   // and of the drain warpgroups
constexpr int kPfSlab = FORTAI_PF_SLAB;                    // TMEM columns per tcgen05.ld
constexpr int kPfRawBlocks = 4;                            // blocks per raw weight load (128 bytes of every row)
constexpr int kPfRawBytes = kPfTileRows * kPfRawBlocks * kBlockElems;
constexpr int kPfRawBuffers = 2;
constexpr int kPfW16Bytes = kPfTileRows * 128;             // binary16, each row [w | w]: 128 bytes

// a CTA holds its 128 weight rows and its half of the pair's token tile
__host__ __device__ constexpr int pf_stage_bytes(int tn) {
    return kPfW16Bytes + (tn / 2) * 128;
}
__host__ __device__ constexpr int pf_tmem_buffers(int tn) { return tn >= 256 ? 2 : 4; }
// shared-memory ring: as deep as fits (a tensor-map load takes well over a thousand cycles to land)
__host__ __device__ constexpr int pf_stages(int tn) { return tn >= 256 ? 6 : 8; }

inline int pf_tile_tokens(int tokens) { return tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256; }

inline int pf_padded_tokens(int tokens) {
    const int tn = pf_tile_tokens(tokens);
    return (tokens + tn - 1) / tn * tn;
}

// Activation image in scratch:
//   [ tokens_padded x blocks x (32 hi | 32 lo) binary16 ][ tokens_padded float unscale ]
inline size_t pf_scratch_bytes(int width, int tokens) {
    const size_t padded = static_cast<size_t>(pf_padded_tokens(tokens));
    return padded * width * 4 + padded * sizeof(float);
}

inline bool pf_supported(int rows, int width, int tokens, int min_tokens) {
    const int threshold = min_tokens > 0 ? min_tokens : 65;
    return tokens >= threshold && width % kBlockElems == 0 && width <= 65536 && rows >= 1;
}

#ifdef FORTAI_PF_TRACE
// Debug builds only: clock64 stamps of CTA 0's roles (producer, MMA, converter, drain).
constexpr int kPfTraceEvents = 96;
__device__ long long g_pf_trace[4][kPfTraceEvents][6];
#define PF_STAMP(role, n, slot) \
    do { if (blockIdx.x == 0 && (n) < kPfTraceEvents) g_pf_trace[role][n][slot] = clock64(); } while (0)
#ifdef FORTAI_PF_TRACE_DRAIN
#define PF_STAMP_DRAIN(role, n, slot) PF_STAMP(role, n, slot)
#else
#define PF_STAMP_DRAIN(role, n, slot) do { } while (0)
#endif
#else
#define PF_STAMP(role, n, slot) do { } while (0)
#define PF_STAMP_DRAIN(role, n, slot) do { } while (0)
#endif

struct PfWeightsPlan {
    bool ready = false;
    CUtensorMap weights_map;    // raw int8 quant plane, boxes of 128 rows x 128 bytes
};

struct PfParams {
    const uint8_t *weights;     // row-planar weight rows (for the fp16 scale plane)
    const float *unscale;       // [padded_tokens] power of two that undoes the token's operand scaling
    int rows;
    int width;
    int blocks;
    int row_stride;
    int tokens;
    int padded_tokens;
    int tiles_n;                // row tiles
    int tiles;                  // row tiles x token tiles
    float *output;              // [tokens][rows]
    int *status;
};

struct PfShared {
    uint64_t full[kPfMaxStages];           // the stage's activation tile has landed
    uint64_t converted[kPfMaxStages];      // binary16 weight tile written
    uint64_t empty[kPfMaxStages];          // the stage's MMAs have finished reading
    uint64_t raw_full[kPfRawBuffers];   // four blocks of raw int8 weights have landed
    uint64_t raw_empty[kPfRawBuffers];  // and have been converted
    uint64_t tmem_full[4];
    uint64_t tmem_empty[4];
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

// The same for a CTA pair: issued by one thread of the leader CTA, executed by both tensor
// cores; each CTA contributes its 128 rows of A and its half of B from its own shared memory
// (the descriptors are offsets valid in both) and keeps its 128 rows of D in its own TMEM.
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
    uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive, once every MMA issued so far by this thread has finished, on the barrier at this
// offset in both CTAs of the pair.
__device__ __forceinline__ void pf_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
        " [%0], %1;"
        ::"r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_result)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

// All threads of both CTAs of the pair.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on the barrier at this shared-memory offset in CTA `rank` of the pair.
__device__ __forceinline__ void mbar_arrive_in_cta(uint32_t bar, uint32_t rank) {
    asm volatile(
        "{\n\t"
        ".reg .b32 remote;\n\t"
        "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t"
        "}"
        ::"r"(bar), "r"(rank) : "memory");
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

// Bounded wait on an mbarrier phase, by shared-memory address: one probe and one branch
// when the phase is already complete (the single-thread roles of this kernel are bound by
// their own instruction count).  Returns false after 2^20 probes.
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n\t"
        "PF_WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra PF_WAIT_DONE;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 p, n, 1048576;\n\t"
        "@p bra PF_WAIT_LOOP;\n\t"
        "setp.ne.u32 p, n, n;\n\t"
        "PF_WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ void pf_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(bar) : "memory");
}

template <int REGS>
__device__ __forceinline__ void regs_release() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void regs_claim() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

// 16 bytes from global memory, issued where it stands (the compiler may not sink it to its
// first use): the weight scales of the next eight blocks are requested a whole chunk ahead.
__device__ __forceinline__ uint4 ldg_early_16(const void *address) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(address));
    return v;
}

// ---- work split ---------------------------------------------------------------------------
// T tiles (256 weight rows x TN tokens, `blocks` units each) on P CTA pairs.  Pair p takes
// the whole tiles p, p + P, ... (floor(T / P) of them: no other pair touches these, their
// results are stored plainly) and then its share of the T mod P tiles that are left over, cut
// into P equal runs of units whatever the tile borders ("split" tiles: their pieces are added
// into zeroed output with atomics).  Every pair gets the same number of units to within one;
// only the left-over tiles pay for zeroing, atomics and a second epilogue.  (Equal shares of
// one long tile-major unit list split nearly every tile: 76 tiles on 74 pairs then cost 20 us
// more than 74 tiles.)
struct PfWalk {
    int tile, kb, count;        // current segment: blocks kb .. kb + count - 1 of `tile`
    int whole_left, pairs, blocks, rem_tile, rem_kb, rem_count;
    bool rem_entered;
};

__host__ __device__ inline int pf_whole_tiles(int tiles, int pairs) {
    return tiles / pairs * pairs;      // tiles below this index are never split
}

__device__ __forceinline__ void pf_walk_next_segment(PfWalk &w) {
    if (w.whole_left > 0) {
        --w.whole_left;
        w.tile += w.pairs;
        w.kb = 0;
        w.count = w.blocks;
        return;
    }
    if (!w.rem_entered) {
        w.rem_entered = true;
        w.tile = w.rem_tile;
        w.kb = w.rem_kb;
    } else {
        ++w.tile;
        w.kb = 0;
    }
    const int room = w.blocks - w.kb;
    w.count = w.rem_count < room ? w.rem_count : room;
    w.rem_count -= w.count;
}

// Positions `w` on the pair's first segment; returns the pair's number of units.
__device__ __forceinline__ int pf_walk_begin(PfWalk &w, int tiles, int blocks, int pairs, int pair) {
    const int whole = tiles / pairs;
    const int rest = tiles - whole * pairs;
    const long long rem_begin = static_cast<long long>(rest) * blocks * pair / pairs;
    const long long rem_end = static_cast<long long>(rest) * blocks * (pair + 1) / pairs;
    w.pairs = pairs;
    w.blocks = blocks;
    w.rem_tile = whole * pairs + static_cast<int>(rem_begin / blocks);
    w.rem_kb = static_cast<int>(rem_begin % blocks);
    w.rem_count = static_cast<int>(rem_end - rem_begin);
    const int total = whole * blocks + w.rem_count;
    w.whole_left = whole;
    w.rem_entered = false;
    w.tile = pair - pairs;
    w.kb = 0;
    w.count = 0;
    pf_walk_next_segment(w);
    return total;
}

template <int TN>
__global__ void __launch_bounds__(kPfThreads, 1)
q8_prefill_kernel(const __grid_constant__ CUtensorMap weights_map,
    const __grid_constant__ CUtensorMap act_map, const __grid_constant__ PfParams p) {
    constexpr int kStageBytes = pf_stage_bytes(TN);
    constexpr int kPfStages = pf_stages(TN);
    constexpr int kBufs = pf_tmem_buffers(TN);
    constexpr int kBufStride = 512 / kBufs;             // TMEM columns per accumulator buffer
    constexpr uint32_t kStageTx = (TN / 2) * 128;

    extern __shared__ uint8_t pf_smem_raw[];
    // [stages x (W16 16 KB | A TN/2*128)] [raw weights: 2 x 16 KB] [barriers]; swizzled tiles
    // start on 1024-byte boundaries (the launch reserves the slack).
    uint8_t *smem = pf_smem_raw + ((1024u - (smem_u32(pf_smem_raw) & 1023u)) & 1023u);
    uint8_t *raw_base = smem + kPfStages * kStageBytes;
    PfShared *sh = reinterpret_cast<PfShared *>(raw_base + kPfRawBuffers * kPfRawBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh->abort_flag;

    // The two CTAs of a cluster work on the same units: one Q8_0 block of one pair tile (256
    // weight rows x TN tokens), numbered tile-major.  CTA `rank` owns weight rows 128 * rank ..
    // of the tile and supplies tokens TN/2 * rank .. of the activation operand.
    const uint32_t rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1;
    const int pairs = gridDim.x >> 1;
    int unit_count;
    {
        PfWalk probe;
        unit_count = pf_walk_begin(probe, p.tiles, p.blocks, pairs, pair);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPfStages; ++s) {
            mbar_init(&sh->full[s], 1);
            mbar_init(&sh->converted[s], 2);   // one converter warp of each CTA
            mbar_init(&sh->empty[s], 1);
        }
        for (int b = 0; b < kPfRawBuffers; ++b) {
            mbar_init(&sh->raw_full[b], 1);
            mbar_init(&sh->raw_empty[b], kPfConverterWarps);
        }
        for (int b = 0; b < 4; ++b) {
            mbar_init(&sh->tmem_full[b], 1);
            mbar_init(&sh->tmem_empty[b], 2 * kPfEpilogueWarps);   // both CTAs' drain warps
        }
        sh->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();         // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    // Everything above may run under the prepare kernel.  What that kernel writes - the
    // activation image, the token scales, the zeroed split tiles - is touched by the TMA
    // producers' activation loads and by the drain only: those wait for it where they start.
    // The first weight load and its conversion do not (weights are nobody's output).

    if (warp < kPfFrontWarps) {
        if (warp < 4) regs_release<kPfProducerRegs>();
        else regs_release<kPfConverterRegs>();
        if (warp == 0 || warp == 3) {
            // ------------------------------ TMA producers -----------------------------
            // A tensor-map load holds the thread that issues it for about 500 cycles whatever
            // its size, about as long as a block's MMAs take: two threads issue, one the even
            // and one the odd blocks, and the weights come four blocks at a time (128 rows x
            // 128 bytes; issued by whichever thread owns the block that starts the four).
            if (lane == 0) {
                const int producer = warp == 0 ? 0 : 1;
                bool ok = true;
                int chunks = 0;         // raw weight loads armed so far
                bool image_ready = false;
                PfWalk walk;
                pf_walk_begin(walk, p.tiles, p.blocks, pairs, pair);
                int kb = walk.kb, left = walk.count;
                bool segment_first = true;
                const uint32_t empty_bar = smem_u32(&sh->empty[0]);
                const uint32_t raw_empty_bar = smem_u32(&sh->raw_empty[0]);
                int armed = 0;
                for (; armed < unit_count && ok; ++armed) {
                    const bool mine = (armed & 1) == producer;
                    const int tile = walk.tile;
                    const int row0 = (tile % p.tiles_n) * kPfPairRows + rank * kPfTileRows;
                    const int token0 = (tile / p.tiles_n) * TN + rank * (TN / 2);
                    if (segment_first || (kb & (kPfRawBlocks - 1)) == 0) {
                        if (mine) {
                            const int rb = chunks % kPfRawBuffers;
                            const int use = chunks / kPfRawBuffers;
                            if (use > 0) ok = pf_wait(raw_empty_bar + 8 * rb, (use - 1) & 1);
                            if (!ok) break;
                            mbar_arrive_expect_tx(&sh->raw_full[rb], kPfRawBytes);
                            tma_load_2d(raw_base + rb * kPfRawBytes, &weights_map,
                                (kb & ~(kPfRawBlocks - 1)) * kBlockElems, row0, &sh->raw_full[rb]);
                        }
                        ++chunks;
                    }
                    if (mine) {
                        const int s = armed % kPfStages;
                        const int use = armed / kPfStages;
                        if (producer == 0) PF_STAMP(0, armed >> 1, 0);
                        if (use > 0) ok = pf_wait(empty_bar + 8 * s, (use - 1) & 1);
                        if (!ok) break;
                        if (!image_ready) {
                            grid_dependency_wait();
                            image_ready = true;
                        }
                        mbar_arrive_expect_tx(&sh->full[s], kStageTx);
                        tma_load_2d(smem + s * kStageBytes + kPfW16Bytes, &act_map, kb * 64,
                            token0, &sh->full[s]);
                        if (producer == 0) PF_STAMP(0, armed >> 1, 1);
                    }
                    if (--left == 0) {
                        pf_walk_next_segment(walk);
                        kb = walk.kb;
                        left = walk.count;
                        segment_first = true;
                    } else {
                        ++kb;
                        segment_first = false;
                    }
                }
                if (!ok) {
                    atomicExch(p.status, kStatusMmqLoadTimeout);
                    *abort_flag = 1;
                    // let the loads that are still in flight land before the CTA ends
                    const int lap = armed < kPfStages ? armed : kPfStages;
                    for (int k = 0; k < lap; ++k) {
                        const int n = armed - 1 - k;
                        mbar_wait_bounded(&sh->full[n % kPfStages], (n / kPfStages) & 1, 1u << 16);
                    }
                    const int clap = chunks < kPfRawBuffers ? chunks : kPfRawBuffers;
                    for (int k = 0; k < clap; ++k) {
                        const int n = chunks - 1 - k;
                        mbar_wait_bounded(&sh->raw_full[n % kPfRawBuffers],
                            (n / kPfRawBuffers) & 1, 1u << 16);
                    }
                }
            }
        } else if (warp == 1 || warp == 2) {
            // ------------------------------ MMA issuers -------------------------------
            // Two threads, one for the even and one for the odd blocks (they use disjoint
            // stages and TMEM buffers): a single issuer needs about 850 cycles per block for
            // its two waits, the fence, four MMAs and two commits, more than the 512 cycles
            // the MMAs themselves take.  The stage ring is unrolled so that barrier addresses
            // and operand descriptors are loop constants.
            if (lane == 0 && rank == 0) {
                constexpr uint32_t idesc = pf_instr_desc(kPfPairRows, TN);
                static_assert(kPfStages % 2 == 0 && kBufs % 2 == 0 && kPfStages % kBufs == 0,
                    "two issuers share the stage ring and the TMEM ring evenly");
                const int issuer = warp - 1;
                const uint32_t full_bar = smem_u32(&sh->full[0]);
                const uint32_t converted_bar = smem_u32(&sh->converted[0]);
                const uint32_t empty_bar = smem_u32(&sh->empty[0]);
                const uint32_t tmem_full_bar = smem_u32(&sh->tmem_full[0]);
                const uint32_t tmem_empty_bar = smem_u32(&sh->tmem_empty[0]);
                // descriptors differ only in their low word (the start address in 16-byte
                // units); keeping that word and building each descriptor where it is used
                // keeps this thread inside its small register budget
                const uint64_t desc_w0 = smem_desc_k_major_sw128(smem);
                const uint32_t desc_hi = static_cast<uint32_t>(desc_w0 >> 32);
                const uint32_t w_lo0 = static_cast<uint32_t>(desc_w0);
                const uint32_t a_lo0 = static_cast<uint32_t>(
                    smem_desc_k_major_sw128(smem + kPfW16Bytes));
                bool ok = true;
                for (int n0 = 0; n0 < unit_count && ok; n0 += kPfStages) {
                    const uint32_t lap = static_cast<uint32_t>(n0 / kPfStages);
#pragma unroll
                    for (int j = 0; j < kPfStages / 2; ++j) {
                        const int s = 2 * j + issuer;
                        if (n0 + s >= unit_count || !ok) break;
                        if (issuer == 0) PF_STAMP(1, (n0 + s) >> 1, 0);
                        ok = pf_wait(full_bar + 8 * s, lap & 1) &&
                            pf_wait(converted_bar + 8 * s, lap & 1);
                        if (!ok) {
                            atomicExch(p.status, kStatusMmqLoadTimeout);
                            break;
                        }
                        if (issuer == 0) PF_STAMP(1, (n0 + s) >> 1, 2);
                        constexpr int kLapBufs = kPfStages / kBufs;     // uses of a buffer per lap
                        const int buf = s % kBufs;
                        const uint32_t use = lap * kLapBufs + s / kBufs;
                        if (use > 0) {
                            ok = pf_wait(tmem_empty_bar + 8 * buf, (use - 1) & 1);
                            if (!ok) {
                                atomicExch(p.status, kStatusMmqDrainTimeout);
                                break;
                            }
                        }
                        tc_fence_after();
                        if (issuer == 0) PF_STAMP(1, (n0 + s) >> 1, 3);
                        // stage s is s * kStageBytes further: the descriptor counts 16 bytes
                        const uint32_t w_lo = w_lo0 + s * (kStageBytes >> 4);
                        const uint32_t a_lo = a_lo0 + s * (kStageBytes >> 4);
                        const uint32_t d = tmem_base + buf * kBufStride;
                        // the 128-byte operand rows are [w | w] and [hi | lo]: four K = 16 steps
                        // of 32 bytes, +2 each in the descriptor's 16-byte units
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_f16_pair(d, pack_bits(w_lo + 2 * k, desc_hi),
                                pack_bits(a_lo + 2 * k, desc_hi), idesc, k > 0 ? 1u : 0u);
                        pf_commit_pair(tmem_full_bar + 8 * buf);
                        pf_commit_pair(empty_bar + 8 * s);
                        if (issuer == 0) PF_STAMP(1, (n0 + s) >> 1, 4);
                    }
                }
                if (!ok) *abort_flag = 1;
            }
        } else if (warp >= kPfFrontWarps - kPfConverterWarps) {
            // ------------------------------ weight converters -------------------------
            // int8 -> binary16 of one block's weight tile (128 rows x 32 quants).  Four warps,
            // each takes every fourth block whole: the waits, the proxy fence and the arrivals
            // of a block cost a warp about as much as the conversion itself, and a warp that
            // owns one block in four pays them once per four block times.  A thread converts
            // eight pieces of 16 raw bytes (half a row each) and writes every piece twice, as
            // the first and the second half of the row's 128 bytes ([w | w]: the tensor core
            // multiplies the same weights with hi and with lo), in the 128-byte swizzled
            // K-major layout.  The raw bytes sit in the same swizzle (four blocks per row).
            const int cw = warp - (kPfFrontWarps - kPfConverterWarps);     // 0..3
            const uint32_t raw_full_bar = smem_u32(&sh->raw_full[0]);
            const uint32_t empty_bar = smem_u32(&sh->empty[0]);
            const uint32_t full_bar = smem_u32(&sh->full[0]);
            const uint32_t converted_bar = smem_u32(&sh->converted[0]);
            PfWalk walk;
            pf_walk_begin(walk, p.tiles, p.blocks, pairs, pair);
            int kb = walk.kb, left = walk.count;
            bool segment_first = true;
            int chunks = 0;             // raw weight loads seen so far
            bool own_in_chunk = false;  // this warp has converted a block of the current load
            bool ok = true;
            for (int n = 0; n < unit_count && ok; ++n) {
                const bool mine = (n & (kPfConverterWarps - 1)) == cw;
                if (segment_first || (kb & (kPfRawBlocks - 1)) == 0) {
                    ++chunks;
                    own_in_chunk = false;
                }
                const int rb = (chunks - 1) % kPfRawBuffers;
                const uint32_t raw_parity = ((chunks - 1) / kPfRawBuffers) & 1;
                const int j = kb & (kPfRawBlocks - 1);
                const bool chunk_last = j == kPfRawBlocks - 1 || left == 1;
                if (mine) {
                    if (cw == 0) PF_STAMP(2, n >> 2, 0);
                    const int s = n % kPfStages;
                    const int use = n / kPfStages;
                    ok = pf_wait(raw_full_bar + 8 * rb, raw_parity);
                    // the stage's previous binary16 tile has been read by its MMAs
                    if (ok && use > 0) ok = pf_wait(empty_bar + 8 * s, (use - 1) & 1);
                    if (!ok) {
                        if (lane == 0) atomicExch(p.status, kStatusMmqLoadTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    if (cw == 0) PF_STAMP(2, n >> 2, 1);
                    uint8_t *stage = smem + s * kStageBytes;
                    const uint8_t *raw = raw_base + rb * kPfRawBytes;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint4 x[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int piece = lane + 32 * (4 * half + q);
                            const int r = piece >> 1;
                            const int c = piece & 1;        // which 16 of the block's 32 quants
                            x[q] = *reinterpret_cast<const uint4 *>(raw + r * 128 +
                                (((2 * j + c) ^ (r & 7)) << 4));
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int piece = lane + 32 * (4 * half + q);
                            const int r = piece >> 1;
                            const int c = piece & 1;
                            uint4 h0, h1;
                            widen4(x[q].x, h0.x, h0.y);
                            widen4(x[q].y, h0.z, h0.w);
                            widen4(x[q].z, h1.x, h1.y);
                            widen4(x[q].w, h1.z, h1.w);
                            // 128-byte swizzle: 16-byte chunk k of row r lives at chunk k ^ (r & 7)
                            uint8_t *row = stage + r * 128;
                            const int x7 = r & 7;
                            *reinterpret_cast<uint4 *>(row + (((2 * c) ^ x7) << 4)) = h0;
                            *reinterpret_cast<uint4 *>(row + (((2 * c + 1) ^ x7) << 4)) = h1;
                            *reinterpret_cast<uint4 *>(row + (((2 * c + 4) ^ x7) << 4)) = h0;
                            *reinterpret_cast<uint4 *>(row + (((2 * c + 5) ^ x7) << 4)) = h1;
                        }
                    }
                    // generic-proxy writes must be visible to the tensor core's async-proxy reads
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    // The leader CTA issues the MMAs for both; what it is told is "this CTA's
                    // operands of the stage are in place", so the peer's converter also waits
                    // for its own activation half before it arrives there.
                    if (rank != 0) ok = pf_wait(full_bar + 8 * s, use & 1);
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive_in_cta(converted_bar + 8 * s, 0);
                        // a warp owns at most one block of a raw load: hand the buffer back
                        mbar_arrive(&sh->raw_empty[rb]);
                    }
                    own_in_chunk = true;
                    if (cw == 0) PF_STAMP(2, n >> 2, 2);
                } else if (chunk_last && !own_in_chunk) {
                    // none of this load's blocks was this warp's: it still owes the buffer its
                    // arrival, and gives it only once the load has landed, so that arrivals of
                    // consecutive uses of the buffer cannot mix
                    ok = pf_wait(raw_full_bar + 8 * rb, raw_parity);
                    if (lane == 0) mbar_arrive(&sh->raw_empty[rb]);
                }
                if (chunk_last) own_in_chunk = true;    // nothing more is owed for this load
                if (--left == 0) {
                    pf_walk_next_segment(walk);
                    kb = walk.kb;
                    left = walk.count;
                    segment_first = true;
                } else {
                    ++kb;
                    segment_first = false;
                }
            }
        }
    } else {
        // ------------------------------ drain ------------------------------------------
        regs_claim<kPfEpilogueRegs>();
        grid_dependency_wait();     // token scales and zeroed split tiles
        const int ew = warp - kPfFrontWarps;
        const int et = threadIdx.x - kPfFrontWarps * 32;    // 0 .. 511
        const int quadrant = warp & 3;              // TMEM lanes this warp may touch
        constexpr int kCols = TN / 4;               // token columns of this warp
        constexpr int kSlab = kCols < kPfSlab ? kCols : kPfSlab;
        const int col0 = (ew >> 2) * kCols;
        constexpr int kPairs = kCols / 2;
        constexpr int kSlabs = kCols / kSlab;
        float acc[kCols];                           // fp32 accumulators
        bool failed = false;

        int drained = 0;        // blocks drained (TMEM ring position)
        PfWalk walk;
        pf_walk_begin(walk, p.tiles, p.blocks, pairs, pair);
        const int whole_tiles = pf_whole_tiles(p.tiles, pairs);
        for (int done = 0; done < unit_count && !failed;) {
            const int tile = walk.tile;
            const int first_block = walk.kb;
            const int count = walk.count;
            const int row0 = (tile % p.tiles_n) * kPfPairRows + rank * kPfTileRows;
            const int token0 = (tile / p.tiles_n) * TN;
            const int row = row0 + quadrant * 32 + lane;
            const bool row_ok = row < p.rows;
            const uint8_t *scale_plane = p.weights +
                static_cast<size_t>(row_ok ? row : 0) * p.row_stride + p.width;
#pragma unroll
            for (int i = 0; i < kCols; ++i) acc[i] = 0.0f;
            // the row's fp16 weight scales, eight blocks (16 aligned bytes) at a time and one
            // chunk ahead; the scale plane is padded to a multiple of 32 bytes per row
            uint4 dw_chunk = ldg_early_16(scale_plane + (first_block & ~7) * 2);
            uint4 dw_ahead = dw_chunk;

            for (int i = 0; i < count && !failed; ++i, ++drained) {
                const int kb = first_block + i;
                if ((kb & 7) == 0 || i == 0) {
                    if (i > 0) dw_chunk = dw_ahead;
                    const int next = (kb & ~7) + 8;
                    if (next < p.blocks) dw_ahead = ldg_early_16(scale_plane + next * 2);
                }
                const int buf = drained % kBufs;
                const uint32_t parity = (drained / kBufs) & 1;
                const uint32_t taddr = tmem_base +
                    (static_cast<uint32_t>(quadrant * 32) << 16) + buf * kBufStride + col0;
                if (et == 0) PF_STAMP(3, drained, 0);
                if (!pf_wait(smem_u32(&sh->tmem_full[buf]), parity)) {
                    if (lane == 0) atomicExch(p.status, kStatusMmqMmaTimeout);
                    *abort_flag = 1;
                    failed = true;
                    break;
                }
                tc_fence_after();
                if (et == 0) PF_STAMP_DRAIN(3, drained, 1);
                const int k8 = kb & 7;
                const uint32_t word = k8 < 2 ? dw_chunk.x : k8 < 4 ? dw_chunk.y
                    : k8 < 6 ? dw_chunk.z : dw_chunk.w;
                const float dw = half_bits_to_float(
                    static_cast<uint16_t>((k8 & 1) ? (word >> 16) : (word & 0xffffu)));
                // Slabs of kSlab columns through two register buffers.  Both buffers are
                // requested at once and each is requested again (two slabs further) as soon as
                // its math is done, so the accumulator buffer goes back to the MMA warp after
                // kSlabs - 2 slab maths instead of kSlabs - 1, and the last two overlap with
                // the next block's MMAs.
                auto slab_math = [&](const uint32_t (&vv)[kSlab], int h) {
                    // scalar FMAs: the packed form needs its operands in aligned register
                    // pairs, and pairing what tcgen05.ld delivers costs more than it saves
#pragma unroll
                    for (int q = 0; q < kSlab; ++q)
                        acc[kSlab * h + q] = fmaf(__uint_as_float(vv[q]), dw, acc[kSlab * h + q]);
                };
                auto release = [&]() {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_in_cta(smem_u32(&sh->tmem_empty[buf]), 0);
                    if (et == 0) PF_STAMP_DRAIN(3, drained, 2);
                };
                if (kSlabs == 1) {
                    uint32_t v0[kSlab];
                    tmem_load_slab(taddr, v0);
                    tmem_load_wait();
                    release();
                    slab_math(v0, 0);
                } else {
                    uint32_t v0[kSlab], v1[kSlab];
                    tmem_load_slab(taddr, v0);
                    tmem_load_slab(taddr + kSlab, v1);
#pragma unroll
                    for (int h = 0; h < kSlabs; h += 2) {
                        tmem_load_wait();
                        if (h + 2 >= kSlabs) release();
                        slab_math(v0, h);
                        if (h + 2 < kSlabs) tmem_load_slab(taddr + kSlab * (h + 2), v0);
                        slab_math(v1, h + 1);
                        if (h + 3 < kSlabs) tmem_load_slab(taddr + kSlab * (h + 3), v1);
                    }
                }
                if (et == 0) PF_STAMP(3, drained, 3);
            }
            if (!failed && row_ok) {
                const bool split = tile >= whole_tiles;
#pragma unroll
                for (int e = 0; e < kPairs; ++e) {
                    const int t = token0 + col0 + 2 * e;
                    const float lo = acc[2 * e], hi = acc[2 * e + 1];
                    // tokens beyond the batch are padding rows of the image (unscale 0)
                    const float2 un = *reinterpret_cast<const float2 *>(p.unscale + t);
                    float *dst = p.output + static_cast<size_t>(t) * p.rows + row;
                    if (split) {
                        if (t < p.tokens) atomicAdd(dst, lo * un.x);
                        if (t + 1 < p.tokens) atomicAdd(dst + p.rows, hi * un.y);
                    } else {
                        if (t < p.tokens) *dst = lo * un.x;
                        if (t + 1 < p.tokens) dst[p.rows] = hi * un.y;
                    }
                }
            }
            done += count;
            pf_walk_next_segment(walk);
        }
    }

    // neither CTA may leave while the peer's tensor core can still read its shared memory or
    // a peer thread can still arrive on its barriers
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- activation image -----------------------------------------------------------------
// One CTA per (padded) token.  Per Q8_0 block: the quantized activation exactly as the
// reference makes it (src/backend/cpu/fortai_q8_dot.c:153-198: same arithmetic and bytes as
// quantize_lane), then da * q split into hi + lo, both binary16, both multiplied by the
// token's power of two 2^(7 - E), E the exponent of the token's largest block scale, so that
// |hi| < 2^15 and lo keeps its bits down to 2^-24.  image[token][block] = [32 hi | 32 lo];
// unscale[token] = 2^(E - 7) (0 for padding rows).  Also zeroes the output of every split
// tile (their pieces arrive as atomic adds).
__device__ __forceinline__ void pf_split_store(float value, float up, __half &hi, __half &lo) {
    const float scaled = value * up;                        // exact: a power of two
    hi = __float2half_rn(scaled);
    lo = __float2half_rn(scaled - __half2float(hi));        // exact difference, fits binary16
}

// Split tiles take their pieces as atomic adds: zero them first.  All CTAs of the grid share
// the work (one CTA per tile took 17 us for a 256 x 256 tile, and the product kernel waits for
// this grid): four consecutive rows per thread and step.
__device__ __forceinline__ void pf_zero_split_tiles(float *__restrict__ output, int rows, int tokens,
    int tile_tokens, int tiles_n, int tiles, int product_grid) {
    if (!output) return;
    const int first_split = pf_whole_tiles(tiles, product_grid);
    const int per_tile = (kPfPairRows / 4) * tile_tokens;           // groups of four rows
    const long long total = static_cast<long long>(tiles - first_split) * per_tile;
    const bool vector = (rows & 3) == 0 && (reinterpret_cast<uintptr_t>(output) & 15) == 0;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int tile = first_split + static_cast<int>(i / per_tile);
        const int within = static_cast<int>(i % per_tile);
        const int r = (tile % tiles_n) * kPfPairRows + (within % (kPfPairRows / 4)) * 4;
        const int t = (tile / tiles_n) * tile_tokens + within / (kPfPairRows / 4);
        if (t >= tokens || r >= rows) continue;
        float *dst = output + static_cast<size_t>(t) * rows + r;
        if (vector) {                                  // rows % 4 == 0: r + 3 < rows
            *reinterpret_cast<float4 *>(dst) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        } else {
            for (int k = 0; k < 4 && r + k < rows; ++k) dst[k] = 0.0f;
        }
    }
}

// fp32 activations, the fast form: one CTA per token, blockDim.x * ITEMS >= width / 4.  A thread
// requests its ITEMS float4 at once and keeps them in registers through both steps (largest
// block scale of the token, then quantize + split), so the kernel costs one trip to memory
// instead of six in a row.
template <int ITEMS>
__global__ void __launch_bounds__(1024)
pf_prepare_f32_kernel(const float *__restrict__ activation, int tokens, int padded_tokens,
    int width, __half *__restrict__ image, float *__restrict__ unscale, float *__restrict__ output,
    int rows, int tile_tokens, int tiles_n, int tiles, int product_grid) {
    grid_dependents_may_launch();
    __shared__ float warp_max[32];
    const int lane = threadIdx.x & 31;
    const int quads = width >> 2;
    for (int token = blockIdx.x; token < padded_tokens; token += gridDim.x) {
        const bool real = token < tokens;
        const float4 *x4 = reinterpret_cast<const float4 *>(activation) +
            static_cast<size_t>(token) * quads;
        float4 v[ITEMS];
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int g = i * blockDim.x + threadIdx.x;
            v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (real && g < quads) v[i] = x4[g];
        }
        // eight lanes per block (trip counts are warp-uniform: the shuffles are safe)
        float amax[ITEMS], scale_max = 0.0f;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            float a = fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
            amax[i] = a;
            scale_max = fmaxf(scale_max, __half2float(__float2half_rn(__fdiv_rn(a, 127.0f))));
        }
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
            scale_max = fmaxf(scale_max, __shfl_xor_sync(0xffffffffu, scale_max, offset));
        __syncthreads();            // the previous token's maxima have been read by everyone
        if (lane == 0) warp_max[threadIdx.x >> 5] = scale_max;
        __syncthreads();
        float m = 0.0f;
        for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) m = fmaxf(m, warp_max[w]);
        // E = exponent of m; binary16 scales lie in [2^-24, 2^16), infinities clamp
        int e = m > 0.0f ? ((__float_as_int(m) >> 23) & 0xff) - 127 : 7;
        e = max(-30, min(e, 30));
        const float up = __int_as_float((127 + 7 - e) << 23);
        if (threadIdx.x == 0) unscale[token] = real ? __int_as_float((127 - 7 + e) << 23) : 0.0f;
        __half *row = image + static_cast<size_t>(token) * width * 2;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int g = i * blockDim.x + threadIdx.x;
            if (g >= quads) continue;
            const float da = __half2float(__float2half_rn(__fdiv_rn(amax[i], 127.0f)));
            const float inverse = amax[i] != 0.0f ? __fdiv_rn(127.0f, amax[i]) : 0.0f;
            const float q0 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v[i].x, inverse)))));
            const float q1 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v[i].y, inverse)))));
            const float q2 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v[i].z, inverse)))));
            const float q3 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v[i].w, inverse)))));
            __half h[4], l[4];
            pf_split_store(__fmul_rn(da, q0), up, h[0], l[0]);
            pf_split_store(__fmul_rn(da, q1), up, h[1], l[1]);
            pf_split_store(__fmul_rn(da, q2), up, h[2], l[2]);
            pf_split_store(__fmul_rn(da, q3), up, h[3], l[3]);
            // block g / 8, elements 4 * (g % 8) .. + 3
            __half *block = row + (g >> 3) * 64 + (g & 7) * 4;
            *reinterpret_cast<uint2 *>(block) = *reinterpret_cast<const uint2 *>(h);
            *reinterpret_cast<uint2 *>(block + 32) = *reinterpret_cast<const uint2 *>(l);
        }
    }
    pf_zero_split_tiles(output, rows, tokens, tile_tokens, tiles_n, tiles, product_grid);
}

// Any width, fp32 or Q8_0 input: two passes over the token.
template <int ACT>
__global__ void __launch_bounds__(256)
pf_prepare_kernel(const void *__restrict__ activation, int tokens, int padded_tokens, int width,
    __half *__restrict__ image, float *__restrict__ unscale, float *__restrict__ output, int rows,
    int tile_tokens, int tiles_n, int tiles, int product_grid) {
    grid_dependents_may_launch();
    __shared__ float warp_max[8];
    __shared__ float token_up;
    const int blocks = width / kBlockElems;
    const int lane = threadIdx.x & 31;
    for (int token = blockIdx.x; token < padded_tokens; token += gridDim.x) {
        const bool real = token < tokens;
        // pass 1: the largest block scale of the token
        float scale_max = 0.0f;
        if (real) {
            if (ACT == 1) {
                const float4 *x4 = static_cast<const float4 *>(activation) +
                    static_cast<size_t>(token) * (width >> 2);
                // eight lanes per block; warp-uniform trip count for the shuffles
                for (int base = 0; base < (width >> 2); base += blockDim.x) {
                    const int g = base + threadIdx.x;
                    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (g < (width >> 2)) v = x4[g];
                    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    scale_max = fmaxf(scale_max,
                        __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f))));
                }
            } else {
                const uint8_t *q8 = static_cast<const uint8_t *>(activation) +
                    static_cast<size_t>(token) * blocks * kBlockBytes;
                for (int b = threadIdx.x; b < blocks; b += blockDim.x)
                    scale_max = fmaxf(scale_max, fabsf(half_bits_to_float(
                        *reinterpret_cast<const uint16_t *>(q8 + static_cast<size_t>(b) * kBlockBytes))));
            }
        }
#pragma unroll
        for (int offset = 16; offset; offset >>= 1)
            scale_max = fmaxf(scale_max, __shfl_xor_sync(0xffffffffu, scale_max, offset));
        __syncthreads();            // the previous token's token_up has been read by everyone
        if (lane == 0) warp_max[threadIdx.x >> 5] = scale_max;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.0f;
            for (int w = 0; w < 8; ++w) m = fmaxf(m, warp_max[w]);
            // E = exponent of m; binary16 scales lie in [2^-24, 2^16), infinities clamp
            int e = m > 0.0f ? ((__float_as_int(m) >> 23) & 0xff) - 127 : 7;
            e = max(-30, min(e, 30));
            token_up = __int_as_float((127 + 7 - e) << 23);
            unscale[token] = real ? __int_as_float((127 - 7 + e) << 23) : 0.0f;
        }
        __syncthreads();
        const float up = token_up;
        // pass 2: quantize again (same arithmetic), split, store
        __half *row = image + static_cast<size_t>(token) * width * 2;
        if (ACT == 1) {
            const float4 *x4 = static_cast<const float4 *>(activation) +
                static_cast<size_t>(token) * (width >> 2);
            for (int base = 0; base < (width >> 2); base += blockDim.x) {
                const int g = base + threadIdx.x;
                const bool valid = g < (width >> 2);
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (valid && real) v = x4[g];
                float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                const float da = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
                const float inverse = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
                const float q0 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v.x, inverse)))));
                const float q1 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v.y, inverse)))));
                const float q2 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v.z, inverse)))));
                const float q3 = static_cast<float>(max(-128, min(127, __float2int_rn(__fmul_rn(v.w, inverse)))));
                if (valid) {
                    __half h[4], l[4];
                    pf_split_store(__fmul_rn(da, q0), up, h[0], l[0]);
                    pf_split_store(__fmul_rn(da, q1), up, h[1], l[1]);
                    pf_split_store(__fmul_rn(da, q2), up, h[2], l[2]);
                    pf_split_store(__fmul_rn(da, q3), up, h[3], l[3]);
                    // block g / 8, elements 4 * (g % 8) .. + 3
                    __half *block = row + (g >> 3) * 64 + (g & 7) * 4;
                    *reinterpret_cast<uint2 *>(block) = *reinterpret_cast<const uint2 *>(h);
                    *reinterpret_cast<uint2 *>(block + 32) = *reinterpret_cast<const uint2 *>(l);
                }
            }
        } else {
            const uint8_t *q8 = static_cast<const uint8_t *>(activation) +
                static_cast<size_t>(token) * blocks * kBlockBytes;
            for (int i = threadIdx.x; i < width; i += blockDim.x) {
                const int b = i >> 5, k = i & 31;
                float value = 0.0f;
                if (real) {
                    const uint8_t *block = q8 + static_cast<size_t>(b) * kBlockBytes;
                    const float da = half_bits_to_float(*reinterpret_cast<const uint16_t *>(block));
                    value = __fmul_rn(da, static_cast<float>(static_cast<int8_t>(block[2 + k])));
                }
                __half h, l;
                pf_split_store(value, up, h, l);
                row[b * 64 + k] = h;
                row[b * 64 + 32 + k] = l;
            }
        }
    }
    pf_zero_split_tiles(output, rows, tokens, tile_tokens, tiles_n, tiles, product_grid);
}

// ---- host side ----------------------------------------------------------------
// uint8 matrix `rows` x `width` bytes, row pitch `pitch`; boxes of 128 rows x 128 bytes
// (four blocks), 128-byte swizzle.
inline bool pf_make_raw_map(CUtensorMap *map, const void *base, int rows, int width, size_t pitch) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
    const cuuint32_t box[2] = {kPfRawBlocks * kBlockElems, kPfTileRows};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
        CUDA_SUCCESS;
}

// binary16 matrix `rows` x `2 * width`, dense; boxes of `box_rows` rows x 64 elements
// (one block: 32 hi, 32 lo), 128-byte swizzle.
inline bool pf_make_act_map(CUtensorMap *map, const void *base, int rows, int width, int box_rows) {
    EncodeTiledFn encode = mmq_encode_fn();
    if (!encode) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(width) * 2, static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(width) * 4};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
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
    return static_cast<size_t>(pf_stages(tn)) * pf_stage_bytes(tn) + kPfRawBuffers * kPfRawBytes +
        sizeof(PfShared) + 64 + 1024;
}

template <int TN>
inline cudaError_t pf_launch(const cudaLaunchConfig_t &config, const CUtensorMap &weights_map,
    const CUtensorMap &act_map, const PfParams &p) {
    static bool configured[16] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 16 && !configured[device]) {
        // The register hand-over inside the kernel (setmaxnreg) only works if the CTA was
        // given the pool it redistributes; a build that allocates fewer registers per
        // thread would wait for registers that never come, so refuse it here.
        cudaFuncAttributes attributes;
        cudaError_t error = cudaFuncGetAttributes(&attributes, q8_prefill_kernel<TN>);
        if (error != cudaSuccess) return error;
        if (attributes.numRegs * kPfThreads <
            128 * kPfProducerRegs + 128 * kPfConverterRegs + 32 * kPfEpilogueWarps * kPfEpilogueRegs)
            return cudaErrorLaunchOutOfResources;
        error = cudaFuncSetAttribute(q8_prefill_kernel<TN>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pf_smem_bytes(TN)));
        if (error != cudaSuccess) return error;
        configured[device] = true;
    }
    return cudaLaunchKernelEx(&config, q8_prefill_kernel<TN>, weights_map, act_map, p);
}

// activation: fp32 [tokens][width] (act == 1) or Q8_0 blocks (act == 0), device memory.
inline cudaError_t pf_enqueue(cudaStream_t stream, int sm_count, int *status, PfWeightsPlan *plan,
    const uint8_t *weights, int rows, int width, int row_stride, const void *activation, int act,
    int tokens, float *output, void **aux, size_t *aux_bytes, uint64_t *launches) {
    const int blocks = width / kBlockElems;
    const int tn = pf_tile_tokens(tokens);
    const int padded = pf_padded_tokens(tokens);
    cudaError_t error = pf_reserve(aux, aux_bytes, width, tokens);
    if (error != cudaSuccess) return error;
    __half *image = static_cast<__half *>(*aux);
    float *unscale = reinterpret_cast<float *>(image + static_cast<size_t>(padded) * width * 2);
    if (!plan->ready) {
        if (!pf_make_raw_map(&plan->weights_map, weights, rows, width, row_stride))
            return cudaErrorNotSupported;
        plan->ready = true;
    }
    CUtensorMap act_map;
    if (!pf_make_act_map(&act_map, image, padded, width, tn / 2)) return cudaErrorNotSupported;

    PfParams p = {};
    p.weights = weights;
    p.unscale = unscale;
    p.rows = rows;
    p.width = width;
    p.blocks = blocks;
    p.row_stride = row_stride;
    p.tokens = tokens;
    p.padded_tokens = padded;
    p.tiles_n = (rows + kPfPairRows - 1) / kPfPairRows;
    p.tiles = p.tiles_n * (padded / tn);
    p.output = output;
    p.status = status;
    const long long total_units = static_cast<long long>(p.tiles) * blocks;
    const int pairs = static_cast<int>(std::min<long long>(sm_count / 2, total_units));
    const int grid = 2 * pairs;
    {
        const int prep_grid = std::min(padded, sm_count * 8);
        const int quads = width / 4;
        const bool aligned = (reinterpret_cast<uintptr_t>(activation) & 15) == 0;
        if (act == 1 && aligned && quads <= 3 * 1024) {
            const int threads = std::min(1024, ((quads + 2) / 3 + 31) / 32 * 32);
            pf_prepare_f32_kernel<3><<<padded, threads, 0, stream>>>(
                static_cast<const float *>(activation), tokens, padded, width, image, unscale,
                output, rows, tn, p.tiles_n, p.tiles, pairs);
        } else if (act == 1 && aligned && quads <= 5 * 1024) {
            const int threads = std::min(1024, ((quads + 4) / 5 + 31) / 32 * 32);
            pf_prepare_f32_kernel<5><<<padded, threads, 0, stream>>>(
                static_cast<const float *>(activation), tokens, padded, width, image, unscale,
                output, rows, tn, p.tiles_n, p.tiles, pairs);
        } else if (act == 1)
            pf_prepare_kernel<1><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                image, unscale, output, rows, tn, p.tiles_n, p.tiles, pairs);
        else
            pf_prepare_kernel<0><<<prep_grid, 256, 0, stream>>>(activation, tokens, padded, width,
                image, unscale, output, rows, tn, p.tiles_n, p.tiles, pairs);
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
    cudaLaunchAttribute attributes[2] = {};
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    if (tn == 256) error = pf_launch<256>(config, plan->weights_map, act_map, p);
    else if (tn == 128) error = pf_launch<128>(config, plan->weights_map, act_map, p);
    else error = pf_launch<64>(config, plan->weights_map, act_map, p);
    if (error != cudaSuccess) return error;
    ++*launches;
    return cudaGetLastError();
}

}  // namespace fortai_b200
