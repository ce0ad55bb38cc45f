// placeholder replaced below
#pragma once
#include "q8_common.cuh"
namespace fortai_b200 {
struct MmqWeightsPlan { bool ready = false; };
inline bool mmq_supported(int, int, int, int) { return false; }
inline cudaError_t mmq_reserve(void **, size_t *, int, int, int) { return cudaSuccess; }
inline cudaError_t mmq_enqueue(cudaStream_t, int, int *, MmqWeightsPlan *, const uint8_t *, int, int,
    int, const void *, int, int, float *, int32_t *, void **, size_t *, uint64_t *) {
    return cudaErrorNotSupported;
}
}
