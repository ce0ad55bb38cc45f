// Bare tcgen05.mma loop: the tensor-core peak of this GPU, measured, as the denominator for
// the prefill kernel's utilisation figure (the data sheet gives 4.5 POPS int8 / 2.25 PFLOPS
// binary16 dense; what a B200 under its power cap sustains is lower and clock dependent).
//
// One CTA per SM; operands (one 128 x 32-byte A tile, one 256 x 32-byte B tile, 128-byte
// swizzle, pseudo-random values) sit in shared memory for the whole run; one thread issues
// MMAs of 128 x 256 x (32 bytes of K) into two TMEM buffers alternately, four per commit,
// and waits (bounded) for the commit before last.  Nothing is drained: this is the rate the
// tensor pipe runs at when nothing else limits it.
#pragma once

#include "q8_prefill.cuh"

namespace fortai_b200 {

struct PeakShared {
    uint64_t bar[2];
    uint32_t tmem_base;
};

// KIND 0: kind::i8 (K = 32), 1: kind::f16 (K = 16).
template <int KIND>
__global__ void __launch_bounds__(128, 1)
tensor_peak_kernel(int iterations, int *status) {
    extern __shared__ uint8_t peak_smem_raw[];
    uint8_t *smem = peak_smem_raw + ((1024u - (smem_u32(peak_smem_raw) & 1023u)) & 1023u);
    PeakShared *sh = reinterpret_cast<PeakShared *>(smem + 48 * 1024);
    const int warp = threadIdx.x >> 5;
    if (KIND == 0) {
        for (int i = threadIdx.x; i < 48 * 1024; i += blockDim.x)
            smem[i] = static_cast<uint8_t>(static_cast<int8_t>(
                static_cast<int>(((i * 2654435761u) >> 13) % 255u) - 127));
    } else {
        __half *values = reinterpret_cast<__half *>(smem);
        for (int i = threadIdx.x; i < 24 * 1024; i += blockDim.x)
            values[i] = __float2half(static_cast<float>(
                static_cast<int>(((i * 2654435761u) >> 13) % 255u) - 127));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x == 0) {
        mbar_init(&sh->bar[0], 1);
        mbar_init(&sh->bar[1], 1);
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(&sh->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;
    if (threadIdx.x == 0) {
        const uint32_t idesc = KIND == 0 ? mmq_instr_desc(128, 256) : pf_instr_desc(128, 256);
        const uint64_t desc_a = smem_desc_k_major_sw128(smem);
        const uint64_t desc_b = smem_desc_k_major_sw128(smem + 16 * 1024);
        bool ok = true;
        for (int it = 0; it < iterations && ok; ++it) {
            const int buf = it & 1;
            if (it >= 2) {
                ok = pf_wait(smem_u32(&sh->bar[buf]), ((it >> 1) - 1) & 1);
                tc_fence_after();
            }
            if (!ok) break;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (KIND == 0) {
                    // first of the four starts the accumulator afresh
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
                        ::"r"(tmem_base + buf * 256), "l"(desc_a + 2 * j), "l"(desc_b + 2 * j),
                        "r"(idesc), "r"(j > 0 ? 1u : 0u) : "memory");
                } else {
                    mma_f16(tmem_base + buf * 256, desc_a + 2 * j, desc_b + 2 * j, idesc,
                        j > 0 ? 1u : 0u);
                }
            }
            pf_commit(smem_u32(&sh->bar[buf]));
        }
        for (int it = iterations >= 2 ? iterations - 2 : 0; it < iterations && ok; ++it)
            ok = pf_wait(smem_u32(&sh->bar[it & 1]), (it >> 1) & 1);
        if (!ok) atomicExch(status, kStatusMmqMmaTimeout);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Operations (2 * M * N * K per MMA) of one launch of `iterations` commits on `grid` CTAs.
inline double tensor_peak_ops(int kind, int iterations, int grid) {
    return 2.0 * 128 * 256 * (kind == 0 ? 32 : 16) * 4.0 * iterations * grid;
}

inline cudaError_t tensor_peak_launch(cudaStream_t stream, int kind, int iterations, int grid,
    int *status) {
    // a whole SM's shared memory, so that exactly one CTA (and its 512 TMEM columns) is resident
    const int smem = 160 * 1024;
    cudaError_t error;
    if (kind == 0) {
        error = cudaFuncSetAttribute(tensor_peak_kernel<0>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (error != cudaSuccess) return error;
        tensor_peak_kernel<0><<<grid, 128, smem, stream>>>(iterations, status);
    } else {
        error = cudaFuncSetAttribute(tensor_peak_kernel<1>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (error != cudaSuccess) return error;
        tensor_peak_kernel<1><<<grid, 128, smem, stream>>>(iterations, status);
    }
    return cudaGetLastError();
}

}  // namespace fortai_b200
