// Q8_0 product for a few tokens at a time (2..64): batched decode, speculative decoding,
// the small end of prefill.  The reference has no such form (it runs one GEMV per token,
// backend/cuda/fortai_cuda_backend.cu:64-147); semantics are those of its matvec applied
// to every token: exact int32 block dots, fmaf((dw * da), float(dot), acc) per block.
//
// The bound is HBM: the weights must be streamed once, not once per token.  Per 32-byte
// block and token the work is one int8 dot plus one scale, and doing that with dp4a for
// eight or more tokens would make the kernel ALU-bound.  So the dots go to the tensor
// cores through warp-level mma.sync.m16n8k32 (int8 x int8 -> int32; one Q8_0 block is
// exactly K = 32), which leaves the CUDA cores one convert and one FMA per (row, token,
// block).  The tcgen05 kernel takes over above 64 tokens (measured on 9728 x 2560 at 64 tokens:
// 22.6 us here against 30.8 us there, whose four MMAs per block take the same 512 cycles for 64
// token columns as for 256).
//
// Mapping.  A warp step is a tile of 16 weight rows x CB bytes (CB = 512: 16 blocks).  The
// warp copies it global -> shared with 16-byte cp.async, one instruction per row, so every
// request is a contiguous 512-byte run of one row like the batch-1 kernel's (16 rows x 64
// bytes per request, the layout an mma fragment would ask for directly, left HBM at half
// speed).  Tiles live in a per-warp ring in shared memory, so bytes in flight do not cost
// registers and no block-level barrier is needed after the prologue.  ldmatrix.x4 turns a
// block of the tile into the A fragment; the activation image (token-major int8 with the
// 4-byte words of each block interleaved so that a lane's two k-slots are adjacent, plus
// one float scale per block and token) is staged once per CTA; every lane ends up with the
// complete block dots of (rows g, g+8) x (tokens 2t, 2t+1), so no cross-lane reduction is
// needed.
//
// Scheduling.  All (row group, step) pairs of a K range form one linear sequence that is
// cut into equal contiguous pieces, one per warp (the whole job is ~15 us, so an unequal
// share per warp would show).  A warp flushes its partial sums with fp32 atomic adds onto
// output that was zeroed beforehand whenever it leaves a row group; the last bit of an
// element can therefore differ between runs, as with the split tiles of the tcgen05
// kernel.  The int32 block dots (probe mode) are exact and deterministic.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "q8_common.cuh"

namespace fortai_b200 {

constexpr int kFewTokMaxTokens = 64;
constexpr int kFewTokMaxWarps = 16;

struct FewTokParams {
    const uint8_t *weights;
    int rows, width, blocks, row_stride;
    const int8_t *act_quants;    // [padded_tokens][width]
    const float *act_scales;     // [blocks][padded_tokens]
    int tokens, padded_tokens;
    int splits;                  // K ranges (grid is a multiple of this)
    int blocks_per_split;        // a multiple of the blocks of one step
    float *output;               // [tokens][rows], zeroed before the launch
    int32_t *block_dots;         // [tokens][rows][blocks] or null
};

inline bool fewtok_supported(int rows, int width, int tokens) {
    return tokens >= 2 && rows >= 1 && width % 64 == 0;
}

inline int fewtok_padded_tokens(int tokens) {
    return tokens <= 8 ? 8 : tokens <= 16 ? 16 : tokens <= 32 ? 32 : 64;
}

// Bytes between two tokens of the shared-memory image.  A half-warp reads 32 contiguous
// bytes of each of four tokens; they must fall into four different quarters of the
// 128-byte bank window.
__host__ __device__ inline int fewtok_token_stride(int range_bytes) {
    return range_bytes + (range_bytes % 128 == 0 ? 32 : 96);
}


inline size_t fewtok_image_bytes(int padded_tokens, int blocks_per_split) {
    const int range_bytes = blocks_per_split * kBlockElems;
    return static_cast<size_t>(padded_tokens) * fewtok_token_stride(range_bytes) +
        static_cast<size_t>(blocks_per_split) * padded_tokens * sizeof(float);
}

__device__ __forceinline__ void mma_s8_16x8x32(int (&d)[4], const uint32_t (&a)[4], uint32_t b0,
    uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_address) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address));
}

__device__ __forceinline__ void cp_async_16(uint32_t smem_address, const void *global) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_address), "l"(global)
                 : "memory");
}
__device__ __forceinline__ void cp_async_8(uint32_t smem_address, const void *global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_address), "l"(global)
                 : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t smem_address, const void *global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_address), "l"(global)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Activation image of a few tokens and the zeroing of the output the product kernel adds
// into.
template <int ACT>
__global__ void __launch_bounds__(256)
fewtok_prepare_kernel(const void *__restrict__ activation, int tokens, int padded_tokens, int width,
    int8_t *__restrict__ quants, float *__restrict__ scales, float4 *__restrict__ zero,
    long long zero_count) {
    grid_dependents_may_launch();
    prepare_token_image<ACT>(activation, tokens, padded_tokens, width, quants, scales);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < zero_count;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        zero[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
}

// NT: token tiles of 8.  CB: bytes of a row per step (512, 256 or 64).  ST: tiles in a
// warp's ring.  DOTS: write the int32 block dots instead of the scaled sums.
template <int NT, int CB, int ST, bool DOTS>
__global__ void __launch_bounds__(512)
q8_fewtok_kernel(const FewTokParams p) {
    constexpr int kFewTokStages = ST;
    extern __shared__ __align__(128) uint8_t fewtok_smem[];
    constexpr int kTokens = NT * 8;
    constexpr int kStepBlocks = CB / kBlockElems;
    constexpr int kRowPitch = CB + 16;               // 16-byte skew: ldmatrix reads 8 rows at once
    constexpr int kScaleBytes = CB / 16;             // binary16 scales of one row of a step
    constexpr int kScalePitch = kScaleBytes < 16 ? 16 : kScaleBytes;
    constexpr int kStageBytes = 16 * kRowPitch + 16 * kScalePitch;
    const int split = blockIdx.x % p.splits;
    const int cta_in_split = blockIdx.x / p.splits;
    const int ctas_per_split = gridDim.x / p.splits;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int range_blocks = p.blocks_per_split;
    const int range_bytes = range_blocks * kBlockElems;
    const int first_block = split * range_blocks;
    const int token_stride = fewtok_token_stride(range_bytes);
    uint8_t *image = fewtok_smem;
    float *image_scales = reinterpret_cast<float *>(fewtok_smem +
        static_cast<size_t>(kTokens) * token_stride);
    const size_t image_bytes = (static_cast<size_t>(kTokens) * token_stride +
        static_cast<size_t>(range_blocks) * kTokens * sizeof(float) + 127) / 128 * 128;
    uint8_t *ring = fewtok_smem + image_bytes + static_cast<size_t>(warp) * kFewTokStages * kStageBytes;
    const uint32_t ring_address = smem_u32(ring);

    // this warp's share of the (row group, step) sequence
    const int groups = (p.rows + 15) >> 4;
    const int steps = range_blocks / kStepBlocks;
    const long long total = static_cast<long long>(groups) * steps;
    const long long all_warps = static_cast<long long>(ctas_per_split) * warps;
    const long long my_warp = static_cast<long long>(cta_in_split) * warps + warp;
    const long long begin = total * my_warp / all_warps;
    const long long end = total * (my_warp + 1) / all_warps;

    int issue_group = static_cast<int>(begin / steps);
    int issue_step = static_cast<int>(begin - static_cast<long long>(issue_group) * steps);
    int group = issue_group, step = issue_step;
    long long issued = begin;
    int issue_stage = 0;

    // one tile: 16 rows x CB bytes, then the rows' scales; always closes a copy group
    auto issue = [&]() {
        if (issued < end) {
            const uint32_t stage = ring_address + issue_stage * kStageBytes;
            constexpr int kLanesPerRow = CB / 16;
            constexpr int kRowsPerCopy = 32 / kLanesPerRow;
            const int sub_row = lane / kLanesPerRow, piece = lane % kLanesPerRow;
            const size_t byte = static_cast<size_t>(first_block + issue_step * kStepBlocks) *
                kBlockElems + piece * 16;
#pragma unroll
            for (int r = 0; r < 16; r += kRowsPerCopy) {
                const int row = min(issue_group * 16 + r + sub_row, p.rows - 1);
                cp_async_16(stage + (r + sub_row) * kRowPitch + piece * 16,
                    p.weights + static_cast<size_t>(row) * p.row_stride + byte);
            }
            const size_t scale_byte = static_cast<size_t>(p.width) +
                static_cast<size_t>(first_block + issue_step * kStepBlocks) * 2;
            if (kScaleBytes == 32) {
                const int row = min(issue_group * 16 + (lane >> 1), p.rows - 1);
                cp_async_16(stage + 16 * kRowPitch + (lane >> 1) * kScalePitch + (lane & 1) * 16,
                    p.weights + static_cast<size_t>(row) * p.row_stride + scale_byte +
                        (lane & 1) * 16);
            } else if (lane < 16) {
                const int row = min(issue_group * 16 + lane, p.rows - 1);
                const uint8_t *src = p.weights + static_cast<size_t>(row) * p.row_stride + scale_byte;
                const uint32_t dst = stage + 16 * kRowPitch + lane * kScalePitch;
                if (kScaleBytes == 16) cp_async_16(dst, src);
                else if (kScaleBytes == 8) cp_async_8(dst, src);
                else cp_async_4(dst, src);
            }
            if (++issue_step == steps) {
                issue_step = 0;
                ++issue_group;
            }
            ++issued;
            issue_stage = issue_stage + 1 == kFewTokStages ? 0 : issue_stage + 1;
        }
        cp_async_commit();
    };
    // weight requests go out before the activation image is staged
#pragma unroll
    for (int u = 0; u < kFewTokStages - 1; ++u) issue();

    grid_dependency_wait();     // image and zeroed output come from the prepare kernel
    {   // stage this K range of the prepared activation image, one Q8_0 block per thread:
        // words (w0..w7) are stored as (w0 w4 w1 w5 w2 w6 w3 w7) so that the two k-slots an
        // mma lane owns, bytes [4t, 4t+4) and [16+4t, 16+4t+4), are one 8-byte load
        for (int i = threadIdx.x; i < kTokens * range_blocks; i += blockDim.x) {
            const int token = i / range_blocks, block = i - token * range_blocks;
            const int4 *src = reinterpret_cast<const int4 *>(p.act_quants +
                static_cast<size_t>(token) * p.width +
                static_cast<size_t>(first_block + block) * kBlockElems);
            const int4 lo = src[0], hi = src[1];
            int4 *dst = reinterpret_cast<int4 *>(image + static_cast<size_t>(token) * token_stride +
                block * kBlockElems);
            dst[0] = make_int4(lo.x, hi.x, lo.y, hi.y);
            dst[1] = make_int4(lo.z, hi.z, lo.w, hi.w);
        }
        const float *scales = p.act_scales + static_cast<size_t>(first_block) * p.padded_tokens;
        for (int i = threadIdx.x; i < range_blocks * kTokens; i += blockDim.x)
            image_scales[i] = scales[i];
    }
    __syncthreads();

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0.0f;

    // ldmatrix row address of this lane: matrices (rows 0-7, k 0-15), (rows 8-15, k 0-15),
    // (rows 0-7, k 16-31), (rows 8-15, k 16-31) = the a0..a3 of the mma
    const int matrix_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t matrix_offset = matrix_row * kRowPitch + (lane >> 4) * 16;
    int stage_index = 0;

    auto flush = [&]() {
        if (DOTS) return;
        const int row_lo = group * 16 + g, row_hi = row_lo + 8;
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = i < 2 ? row_lo : row_hi;
                const int token = 8 * j + 2 * t + (i & 1);
                if (row < p.rows && token < p.tokens)
                    atomicAdd(p.output + static_cast<size_t>(token) * p.rows + row, acc[j][i]);
                acc[j][i] = 0.0f;
            }
    };

    for (long long consumed = begin; consumed < end; ++consumed) {
        issue();                                    // keeps kFewTokStages - 1 tiles in flight
        cp_async_wait<kFewTokStages - 1>();
        __syncwarp();
        const uint8_t *stage = ring + stage_index * kStageBytes;
        const uint32_t stage_address = ring_address + stage_index * kStageBytes;
        // the binary16 scales of rows g and g + 8 for every block of the step
        constexpr int kScaleWords = kScaleBytes / 4;
        uint32_t words_lo[kScaleWords], words_hi[kScaleWords];
        {
            const uint8_t *lo = stage + 16 * kRowPitch + g * kScalePitch;
            const uint8_t *hi = stage + 16 * kRowPitch + (g + 8) * kScalePitch;
            if (kScaleWords >= 4) {
#pragma unroll
                for (int v = 0; v < kScaleWords / 4; ++v) {
                    const uint4 a = reinterpret_cast<const uint4 *>(lo)[v];
                    const uint4 b = reinterpret_cast<const uint4 *>(hi)[v];
                    words_lo[4 * v] = a.x, words_lo[4 * v + 1] = a.y;
                    words_lo[4 * v + 2] = a.z, words_lo[4 * v + 3] = a.w;
                    words_hi[4 * v] = b.x, words_hi[4 * v + 1] = b.y;
                    words_hi[4 * v + 2] = b.z, words_hi[4 * v + 3] = b.w;
                }
            } else {
#pragma unroll
                for (int v = 0; v < kScaleWords; ++v) {
                    words_lo[v] = reinterpret_cast<const uint32_t *>(lo)[v];
                    words_hi[v] = reinterpret_cast<const uint32_t *>(hi)[v];
                }
            }
        }
        const int range_block = step * kStepBlocks;
        const int row_lo = group * 16 + g, row_hi = row_lo + 8;
#pragma unroll
        for (int b = 0; b < kStepBlocks; ++b) {
            uint32_t a[4];
            ldmatrix_x4(a, stage_address + matrix_offset + b * kBlockElems);
            const float dw_lo = __half2float(__ushort_as_half(
                static_cast<uint16_t>(b & 1 ? words_lo[b >> 1] >> 16 : words_lo[b >> 1])));
            const float dw_hi = __half2float(__ushort_as_half(
                static_cast<uint16_t>(b & 1 ? words_hi[b >> 1] >> 16 : words_hi[b >> 1])));
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint2 x = *reinterpret_cast<const uint2 *>(image +
                    static_cast<size_t>(8 * j + g) * token_stride +
                    (range_block + b) * kBlockElems + t * 8);
                int dots[4];
                mma_s8_16x8x32(dots, a, x.x, x.y);
                if (DOTS) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = i < 2 ? row_lo : row_hi;
                        const int token = 8 * j + 2 * t + (i & 1);
                        if (row < p.rows && token < p.tokens)
                            p.block_dots[(static_cast<size_t>(token) * p.rows + row) * p.blocks +
                                first_block + range_block + b] = dots[i];
                    }
                } else {
                    const float2 da = *reinterpret_cast<const float2 *>(image_scales +
                        (range_block + b) * kTokens + 8 * j + 2 * t);
                    acc[j][0] = fmaf(dw_lo * da.x, static_cast<float>(dots[0]), acc[j][0]);
                    acc[j][1] = fmaf(dw_lo * da.y, static_cast<float>(dots[1]), acc[j][1]);
                    acc[j][2] = fmaf(dw_hi * da.x, static_cast<float>(dots[2]), acc[j][2]);
                    acc[j][3] = fmaf(dw_hi * da.y, static_cast<float>(dots[3]), acc[j][3]);
                }
            }
        }
        __syncwarp();                               // the tile may be overwritten from here on
        if (step + 1 == steps || consumed + 1 == end) flush();
        if (++step == steps) {
            step = 0;
            ++group;
        }
        stage_index = stage_index + 1 == kFewTokStages ? 0 : stage_index + 1;
    }
    cp_async_wait<0>();
}

struct FewTokPlan {
    int splits, blocks_per_split, step_bytes, stages, threads;
    size_t smem;
};

__host__ __device__ inline int fewtok_stage_bytes(int cb) {
    return 16 * (cb + 16) + 16 * (cb / 16 < 16 ? 16 : cb / 16);
}

// Step width: 256 bytes of a row where the width allows it and every warp still gets a
// step, else 64.  K ranges: as few as keep the activation image of one range
// within 96 KB.  Warps: up to 16 rings of two or three tiles beside the image (the consume
// phase is a chain of dependent shared-memory loads and MMAs, so it takes many warps to
// keep the SM busy).
inline bool fewtok_plan(int rows, int width, int padded_tokens, int sm_count, int split_option,
    int threads_option, int step_option, int stages_option, FewTokPlan *plan) {
    const int blocks = width / kBlockElems;
    const long long groups = (rows + 15) / 16;
    // 256-byte runs measured best on every shape tried (512 leaves room for fewer warps,
    // 64 makes more, smaller requests); 512 stays available as an option
    int cb = step_option > 0 ? step_option : (width % 256 == 0 && groups * (width / 256) >=
        static_cast<long long>(sm_count) * kFewTokMaxWarps ? 256 : 64);
    if (cb == 0 || width % cb != 0) return false;
    const int step_blocks = cb / kBlockElems;
    const size_t image_budget = 96 * 1024;
    int splits = split_option > 0 ? split_option : 1;
    for (;; ++splits) {
        if (splits > blocks / step_blocks) return false;
        if (blocks % (step_blocks * splits) != 0) continue;
        if (split_option > 0 || fewtok_image_bytes(padded_tokens, blocks / splits) <= image_budget)
            break;
    }
    plan->splits = splits;
    plan->blocks_per_split = blocks / splits;
    plan->step_bytes = cb;
    const size_t image = (fewtok_image_bytes(padded_tokens, plan->blocks_per_split) + 127) / 128 * 128;
    const size_t budget = 224 * 1024;
    const size_t stage = fewtok_stage_bytes(cb);
    if (image + 2 * stage > budget) return false;
    int stages = stages_option == 2 || stages_option == 3 ? stages_option
        : (image + 3 * stage * kFewTokMaxWarps <= budget ? 3 : 2);
    int warps = static_cast<int>(std::min<size_t>(kFewTokMaxWarps, (budget - image) / (stages * stage)));
    if (warps < 1) {
        stages = 2;
        warps = static_cast<int>(std::min<size_t>(kFewTokMaxWarps, (budget - image) / (2 * stage)));
    }
    if (threads_option > 0) warps = std::min(warps, threads_option / 32);
    warps = std::max(1, warps);
    plan->stages = stages;
    plan->threads = warps * 32;
    plan->smem = image + static_cast<size_t>(stages) * stage * warps;
    return true;
}

// Every CTA must be resident at once (the work is cut into equal shares up front), and no
// warp may be left without a step.
inline int fewtok_grid(const FewTokPlan &plan, int rows, int width, int sm_count, int ctas_per_sm) {
    const long long steps = static_cast<long long>((rows + 15) / 16) * (width / plan.step_bytes);
    long long ctas = static_cast<long long>(sm_count) * std::max(1, ctas_per_sm);
    ctas = std::min<long long>(ctas, std::max<long long>(1, steps / (plan.threads / 32)));
    ctas = std::max<long long>(plan.splits, ctas / plan.splits * plan.splits);
    return static_cast<int>(ctas);
}

}  // namespace fortai_b200
