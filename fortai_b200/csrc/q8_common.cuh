// Shared device helpers and the device-side weight layout of the Q8_0 backend.
//
// Host (GGUF) layout, as uploaded: rows x B blocks of 34 bytes, each block a
// binary16 scale followed by 32 int8 quants (reference:
// src/fortai_gguf_runtime.f90:312-318, 751-757).  Blocks are only 2-byte
// aligned, which is why the reference kernels fetch weights with 2-byte loads
// (backend/cuda/fortai_cuda_backend.cu:54-57).
//
// Device layout used here ("row-planar"): row r lives at r * row_stride bytes,
//     [ K int8 quants | B binary16 scales | pad to a multiple of 32 ]
// with row_stride = round_up(34 * B, 32).  The bytes per block are unchanged
// (34), every row and every block starts on a 32-byte boundary, quants can be fetched with
// 16- or 32-byte vector loads or 1-D bulk copies, a row stays one contiguous burst for
// the memory system, and both planes are addressable as 2-D tensor maps
// (pitch = row_stride) by the tensor-core prefill kernel.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fortai_b200 {

constexpr int kBlockElems = 32;
constexpr int kBlockBytes = 34;
constexpr int kSmCountB200 = 148;

// Codes written to the context's device status word by kernels whose bounded
// waits ran out.  Zero means no kernel gave up.
enum DeviceStatus : int {
    kStatusOk = 0,
    kStatusMmqLoadTimeout = 3,
    kStatusMmqMmaTimeout = 4,
    kStatusMmqDrainTimeout = 5,
    kStatusPeerFlagTimeout = 6,
    kStatusPositionOutOfRange = 7
};

__host__ __device__ inline size_t row_stride_bytes(int blocks) {
    return (static_cast<size_t>(blocks) * kBlockBytes + 31) & ~static_cast<size_t>(31);
}

__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

// 16-byte streaming load: read-only path, no L1 allocation (each weight byte is
// used exactly once per GEMV).
__device__ __forceinline__ int4 ldg_stream_16(const void *address) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(address));
    return v;
}

__device__ __forceinline__ uint16_t ldg_stream_u16(const void *address) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(address));
    return v;
}

__device__ __forceinline__ int dot16(const int4 &w, const int4 &a) {
    int d = __dp4a(w.x, a.x, 0);
    d = __dp4a(w.y, a.y, d);
    d = __dp4a(w.z, a.z, d);
    return __dp4a(w.w, a.w, d);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// silu(g) * u with the IEEE exponential and division (the reference CPU path
// approximates expf to ~2e-7 relative; its own test tolerance is 2e-5,
// test/test_fortai_smoke.f90:284-299).
__device__ __forceinline__ float silu_mul(float gate, float up) {
    return __fdiv_rn(gate, 1.0f + expf(-gate)) * up;
}

// silu(x) with the IEEE exponential and division.
__device__ __forceinline__ float silu_ieee(float x) {
    return __fdiv_rn(x, 1.0f + expf(-x));
}

// ---- Q8_0 quantization of 32 floats held one per lane ----------------------
// Bit-for-bit the arithmetic of the reference's AVX2 quantizer
// (src/backend/cpu/fortai_q8_dot.c:153-198): amax over the block, scale =
// amax / 127 (IEEE division) rounded to binary16 nearest-even, inverse =
// 127 / amax (0 for an all-zero block), quant = round-half-even(x * inverse)
// saturated to int8.  Returns the quant; *scale_bits gets the stored scale.
__device__ __forceinline__ int quantize_lane(float x, uint16_t *scale_bits) {
    float amax = fabsf(x);
#pragma unroll
    for (int offset = 16; offset; offset >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
    const float scale = __fdiv_rn(amax, 127.0f);
    const float inverse = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    *scale_bits = __half_as_ushort(__float2half_rn(scale));
    int q = __float2int_rn(__fmul_rn(x, inverse));
    return max(-128, min(127, q));
}

// ---- activation image of several tokens -----------------------------------------
// quants[token][width] int8 and scales[block][padded_tokens] float for `padded_tokens`
// rows (rows >= tokens are zero), from fp32 rows (ACT == 1: eight lanes per Q8_0 block,
// one 16-byte load and one 32-bit store per lane, same arithmetic and bytes as
// quantize_lane) or from GGUF Q8_0 rows (ACT == 0: one warp per block).  Called by all
// threads of a 256-thread CTA of a 1-D grid.
template <int ACT>
__device__ __forceinline__ void prepare_token_image(const void *__restrict__ activation, int tokens,
    int padded_tokens, int width, int8_t *__restrict__ quants, float *__restrict__ scales) {
    const int blocks = width / kBlockElems;
    if (ACT == 1) {
        const float4 *x4 = static_cast<const float4 *>(activation);
        uint32_t *q32 = reinterpret_cast<uint32_t *>(quants);
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
                q32[static_cast<size_t>(token) * groups + g] = static_cast<uint32_t>(q0 & 0xff) |
                    (static_cast<uint32_t>(q1 & 0xff) << 8) |
                    (static_cast<uint32_t>(q2 & 0xff) << 16) |
                    (static_cast<uint32_t>(q3 & 0xff) << 24);
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
                static_cast<int8_t>(q);
            if (lane == 0) scales[static_cast<size_t>(b) * padded_tokens + token] = scale;
        }
    }
}

// ---- programmatic dependent launch ---------------------------------------------
// A kernel launched with programmatic stream serialization may start while its
// predecessor in the stream still runs; it calls grid_dependency_wait() before it touches
// anything the predecessor writes, and the predecessor calls grid_dependents_may_launch()
// as early as it likes.  Both are no-ops for a plain launch.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_dependents_may_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- mbarrier / bulk-copy primitives (sm_90+; used without clusters) -------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Wait for the phase of the given parity to complete, giving up after `limit`
// probes (each probe itself blocks for a hardware-defined slice).  Returns false
// on give-up so that the caller can record a status and leave; no wait in this
// library spins without a bound.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
    uint32_t limit = 1u << 22) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// The same with non-suspending probes (mbarrier.test_wait): the waiter notices a completed
// phase within a few cycles instead of at the end of a suspension slice.  For the hot
// hand-offs of a pipeline whose stages take well under a microsecond; the bound is 2^26
// probes (tens of milliseconds).
__device__ __forceinline__ bool mbar_wait_spin_bounded(uint64_t *bar, uint32_t parity,
    uint32_t limit = 1u << 26) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// 1-D bulk asynchronous copy global -> shared, completion counted in bytes on an
// mbarrier.  Both addresses 16-byte aligned, size a multiple of 16.  Always the
// plain one-destination form: the copy lands in the issuing CTA's own shared memory.
__device__ __forceinline__ void bulk_copy_g2s(void *smem_dst, const void *gmem_src,
    uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

}  // namespace fortai_b200
