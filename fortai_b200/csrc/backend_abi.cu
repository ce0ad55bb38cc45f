// C ABI of the B200 Q8_0 backend: handles, validation, scratch, launch policy.
//
// Mirrors the behaviour of the reference backend's entry points
// (backend/cuda/fortai_cuda_backend.cu:789-1296, 1733-1736): same symbols, same
// argument checks, same return codes, same blocking/enqueue split.  The kernels
// behind them are in q8_gemv.cuh (batch 1) and q8_mmq.cuh (prefill).
#include "../../include/fortai_cuda_backend_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <new>

#include "q8_common.cuh"
#include "q8_gemv.cuh"
#include "q8_mmq.cuh"
#include "q8_prefill.cuh"
#include "tensor_peak.cuh"
#include "q8_fewtok.cuh"
#include "qwen35_layers.cuh"

using namespace fortai_b200;

struct fortai_cuda_q8_context {
    int device = 0;
    int sm_count = kSmCountB200;
    cudaStream_t stream = nullptr;
    bool owns_stream = true;
    cudaEvent_t start = nullptr;
    cudaEvent_t stop = nullptr;
    uint8_t *scratch_activation = nullptr;   // Q8_0 activation(s)
    size_t scratch_activation_bytes = 0;
    float *scratch_output = nullptr;         // fp32 intermediate / host-call output
    size_t scratch_output_bytes = 0;
    uint8_t *scratch_aux = nullptr;          // prefill: planar activation, partial tiles
    size_t scratch_aux_bytes = 0;
    uint8_t *scratch_planar = nullptr;       // batch 1: prepared activation image (long vectors)
    size_t scratch_planar_bytes = 0;
    int planar_min_width = 6144;             // vectors at least this long are prepared once
    int *position = nullptr;
    unsigned *cta_counter = nullptr;         // device word used by the fused all-gather tail
    unsigned allgather_sequence = 0;   // fused all-gather launches so far (wraps)
    unsigned host_sequence = 0;        // host-call completions so far (wraps)
    unsigned ffn_exchange_calls = 0;   // all-reduce FFN calls so far (slot parity)
    unsigned ll_calls = 0;             // pair all-gather calls so far (half of the pair arrays)
    unsigned ll_sequence = 0;          // their call number (never zero)
    int *status_host = nullptr;              // pinned + mapped: kernels write, host reads
    int *status_device = nullptr;
    unsigned *done_host = nullptr;           // pinned + mapped: completion word of host calls
    unsigned *done_device = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    uint64_t launches = 0;
    // options
    int host_flush_rows = 8;   // rows per store group into a page-locked host output
    int peer_flush_rows = 32;  // rows per store group into peers' vectors
    int peer_publish_per_cta = 0;   // fused exchanges: 0 = the last CTA raises a flag, 1 = per-CTA adds (capturable)
    int gemv_variant = 0;      // 0 = automatic choice, 1 = always the half-block kernel
    int gemv_ctas_per_sm = 0;  // 0 = occupancy-derived
    int gemv_rows_per_warp = 0;
    int gemv_depth = 1;        // rows in flight per warp in the pipelined kernel (1 or 2)
    int gemv_split = 0;        // slice kernel: 0 automatic, 1 off, 4 or 8 warps per row
    int gemv_balance = 0;      // 1 = trim the grid so that the last round of rows is full
    int peer_wait_clocks_millions = 2000;   // fused all-gather: wait for a peer's flag, in 1e6 SM clocks
    int mmq_min_tokens = 0;    // first token count of the tcgen05 kernel (0 = 65)
    int prefill_kind = 0;      // tcgen05 kernel: 0 = kind::f16, activation scale folded into the operand; 1 = kind::i8, scaled per block
    int fewtok_splits = 0;     // K ranges of the few-token kernel (0 = as few as fit)
    int fewtok_threads = 0;    // its CTA size (0 = 256)
    int fewtok_stages = 0;     // tiles per warp ring (0 = chosen from the shape, else 2 or 3)
    int fewtok_step = 0;       // bytes of a row per step (0 = chosen from the shape)
    int ffn_quantize_in_gemv = 4096;   // FFN inner sizes up to this skip the quantize kernel
    int gdn_conv_in_gemv = 1;      // recurrent layer: convolution in the projection's epilogue
    int gemv_even_rounds = 1;      // half-block kernel: equal rows per warp when rounds are few
    int gemv_early_trigger = 3;    // successor may be scheduled at once: 0 never, 1 always, 2 when the grid fills the machine, 3 after a residual epilogue
    int host_direct_output = 1;    // *_host_f32: store straight into page-locked output
    int host_spin_wait = 1;        // *_host_f32 with page-locked buffers: no copy engine, no events
    int peer_overlap = 1;          // fused all-gather GEMVs may start under their predecessor's tail
    int gemv_overlap = 1;      // GEMVs may start under the tail of the previous kernel
    int fewtok_overlap = 1;    // product kernel may start under the prepare kernel
    int fewtok_off = 0;        // 1 = small batches run one GEMV per token
    char error[256] = {};
};

struct fortai_cuda_q8_weights {
    fortai_cuda_q8_context *context = nullptr;
    int rows = 0;
    int width = 0;
    int blocks = 0;
    int row_stride = 0;
    uint8_t *data = nullptr;
    MmqWeightsPlan mmq;   // tensor maps for the prefill kernels, built lazily
    PfWeightsPlan prefill;
};

// Layer objects borrow their weight handles (the caller keeps them alive and destroys
// layers first, as the reference does: src/models/qwen35/fortai_qwen35_cpu.f90:519-530).
struct fortai_cuda_qwen35_recurrent {
    fortai_cuda_q8_context *context = nullptr;
    const fortai_cuda_q8_weights *qkv = nullptr, *gate = nullptr, *alpha = nullptr,
        *beta = nullptr, *out = nullptr;
    float *conv_weights = nullptr, *ssm_a = nullptr, *ssm_dt = nullptr, *ssm_norm = nullptr;
    float *conv_state = nullptr, *gdn_state = nullptr;
    float *projections = nullptr;   // qkv | gate | alpha | beta outputs, back to back
    float *gdn_output = nullptr;
    int conv_size = 0, conv_kernel = 0, state_size = 0, key_heads = 0, value_heads = 0,
        head_size = 0, inner_size = 0;
    float epsilon = 1.0e-6f;
};

struct fortai_cuda_qwen35_attention {
    fortai_cuda_q8_context *context = nullptr;
    const fortai_cuda_q8_weights *q = nullptr, *k = nullptr, *v = nullptr, *out = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr;
    __half *key_cache = nullptr, *value_cache = nullptr;
    float *projections = nullptr;   // query | key | value outputs, back to back
    float *attention = nullptr;
    int heads = 0, kv_heads = 0, head_size = 0, value_size = 0, max_context = 0,
        rope_dimension = 0;
    float rope_base = 1.0f, epsilon = 1.0e-6f;
};

namespace {

int fail(fortai_cuda_q8_context *context, const char *operation,
    cudaError_t error = cudaSuccess) {
    if (context) {
        if (error == cudaSuccess)
            std::snprintf(context->error, sizeof(context->error), "%s", operation);
        else
            std::snprintf(context->error, sizeof(context->error), "%s: %s", operation,
                cudaGetErrorString(error));
    }
    return FORTAI_CUDA_RUNTIME_ERROR;
}

const char *status_text(int code) {
    switch (code) {
    case kStatusMmqLoadTimeout: return "prefill kernel gave up waiting for an operand tile";
    case kStatusMmqMmaTimeout: return "prefill kernel gave up waiting for the tensor core";
    case kStatusMmqDrainTimeout: return "prefill kernel gave up waiting for an accumulator";
    case kStatusPeerFlagTimeout: return "gave up waiting for a peer flag";
    case kStatusPositionOutOfRange: return "attention position outside the layer's context";
    default: return "unknown device status";
    }
}

// After a synchronizing call: turn a device-side give-up into a runtime error.
int finish(fortai_cuda_q8_context *context, const char *operation, cudaError_t error) {
    if (error != cudaSuccess) return fail(context, operation, error);
    const int status = *static_cast<volatile int *>(context->status_host);
    if (status != kStatusOk) {
        *static_cast<volatile int *>(context->status_host) = kStatusOk;
        std::snprintf(context->error, sizeof(context->error), "%s: %s", operation,
            status_text(status));
        return FORTAI_CUDA_RUNTIME_ERROR;
    }
    return FORTAI_CUDA_OK;
}

cudaError_t grow(void **pointer, size_t *have, size_t want) {
    if (want <= *have) return cudaSuccess;
    cudaError_t error = cudaFree(*pointer);
    *pointer = nullptr;
    *have = 0;
    if (error != cudaSuccess) return error;
    error = cudaMalloc(pointer, want);
    if (error == cudaSuccess) *have = want;
    return error;
}

cudaError_t ensure_scratch(fortai_cuda_q8_context *c, size_t activation_bytes,
    size_t output_bytes, size_t aux_bytes = 0) {
    cudaError_t error = grow(reinterpret_cast<void **>(&c->scratch_activation),
        &c->scratch_activation_bytes, activation_bytes);
    if (error == cudaSuccess)
        error = grow(reinterpret_cast<void **>(&c->scratch_output), &c->scratch_output_bytes,
            output_bytes);
    if (error == cudaSuccess)
        error = grow(reinterpret_cast<void **>(&c->scratch_aux), &c->scratch_aux_bytes, aux_bytes);
    return error;
}

// ---------------------------------------------------------------------------
// GEMV launch policy
// ---------------------------------------------------------------------------
// A GEMV may start while its predecessor in the stream drains (programmatic stream
// serialization): the kernel waits by itself before it reads anything but weights.  Kept
// off for the multi-GPU epilogues, whose peers know nothing of this stream's order.
template <typename Kernel>
cudaError_t launch_gemv_kernel(fortai_cuda_q8_context *c, Kernel kernel, int grid, int threads,
    size_t smem, const GemvParams &params, int resident_limit) {
    GemvParams p = params;
    switch (c->gemv_early_trigger) {
    case 0: case 1: p.trigger_early = c->gemv_early_trigger; break;
    case 2: p.trigger_early = grid * 8 >= resident_limit * 7; break;
    default: p.trigger_early = params.residual != nullptr; break;   // last GEMV of a layer step
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(threads);
    config.dynamicSmemBytes = smem;
    config.stream = c->stream;
    cudaLaunchAttribute overlap = {};
    overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    overlap.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &overlap;
    // (p.overlap_ok: a "peer" launch whose only peer is this process's own host memory)
    config.numAttrs = c->gemv_overlap && ((p.peers == 0 && p.exchange == kExchangeOff) || p.overlap_ok) ? 1 : 0;
    const cudaError_t error = cudaLaunchKernelEx(&config, kernel, p);
    ++c->launches;
    return error != cudaSuccess ? error : cudaGetLastError();
}

// The small kernels between the GEMVs of a layer, launched the same way: each begins with
// grid_dependency_wait(), so only its launch latency overlaps the predecessor.
template <typename... Params, typename... Args>
cudaError_t launch_overlapped(fortai_cuda_q8_context *c, void (*kernel)(Params...), int grid,
    int threads, size_t smem, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(threads);
    config.dynamicSmemBytes = smem;
    config.stream = c->stream;
    cudaLaunchAttribute overlap = {};
    overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    overlap.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &overlap;
    config.numAttrs = c->gemv_overlap ? 1 : 0;
    const cudaError_t error = cudaLaunchKernelEx(&config, kernel, args...);
    ++c->launches;
    return error != cudaSuccess ? error : cudaGetLastError();
}

template <int U, int NR, int ACT, int EPI>
cudaError_t launch_direct_instance(fortai_cuda_q8_context *c, const GemvParams &p) {
    auto kernel = q8_gemv_direct_kernel<U, NR, ACT, EPI>;
    const size_t smem = activation_smem_bytes(p.width, p.blocks);
    static int per_sm_cache[64] = {};   // indexed by device
    cudaError_t error = cudaSuccess;
    if (smem > 48 * 1024) {
        error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
            static_cast<int>(smem));
        if (error != cudaSuccess) return error;
    }
    int per_sm = c->gemv_ctas_per_sm;
    if (per_sm <= 0) {
        int &cached = per_sm_cache[c->device & 63];
        if (cached == 0 || smem > 8 * 1024) {
            int blocks = 0;
            error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, kGemvThreads,
                smem);
            if (error != cudaSuccess) return error;
            if (smem <= 8 * 1024) cached = blocks;
            per_sm = blocks;
        } else {
            per_sm = cached;
        }
        if (per_sm < 1) per_sm = 1;
    }
    const int rows_per_cta = kGemvWarps * (EPI == kEpiSiluPair ? 1 : NR);
    const int needed = (p.total_rows + rows_per_cta - 1) / rows_per_cta;
    const int limit = c->sm_count * per_sm;
    int grid = std::max(1, std::min(needed, limit));
    if (c->gemv_even_rounds && needed > limit && needed < 4 * limit) {
        // a few rounds of rows per warp: size the grid so that every warp gets the same
        // number (5120 long rows on 592 CTAs are 1.08 rounds - most warps would wait for
        // the few that have a second row; 320 CTAs with two rows each finish sooner)
        const int rounds = (needed + limit - 1) / limit;
        grid = (needed + rounds - 1) / rounds;
    }
    return launch_gemv_kernel(c, kernel, grid, kGemvThreads, smem, p, limit);
}

template <int ACT, int EPI>
cudaError_t launch_direct(fortai_cuda_q8_context *c, const GemvParams &p) {
    const int nchunks = p.width / 16;
    const int per_lane = (nchunks + 31) / 32;
    int rows_per_warp = c->gemv_rows_per_warp;
    if (EPI == kEpiSiluPair || EPI == kEpiBlockDots) rows_per_warp = 1;
    else if (rows_per_warp <= 0) rows_per_warp = per_lane <= 4 ? 2 : 1;
    if (per_lane <= 2)
        return rows_per_warp == 2 ? launch_direct_instance<2, 2, ACT, EPI>(c, p)
                                  : launch_direct_instance<2, 1, ACT, EPI>(c, p);
    if (per_lane <= 4)
        return rows_per_warp == 2 ? launch_direct_instance<4, 2, ACT, EPI>(c, p)
                                  : launch_direct_instance<4, 1, ACT, EPI>(c, p);
    if (per_lane == 5 || per_lane == 10 || per_lane == 15 || per_lane == 19 || per_lane == 20)
        return rows_per_warp == 2 ? launch_direct_instance<5, 2, ACT, EPI>(c, p)
                                  : launch_direct_instance<5, 1, ACT, EPI>(c, p);
    return rows_per_warp == 2 ? launch_direct_instance<8, 2, ACT, EPI>(c, p)
                              : launch_direct_instance<8, 1, ACT, EPI>(c, p);
}

// Grid for a persistent warp-per-row kernel: at most `limit` CTAs, but prefer a
// slightly smaller count when that makes the last round of rows nearly full
// (151936 rows on 592 CTAs is 32.08 rounds - 2.8 % of the time almost every warp
// would idle; 576 CTAs make it 32.97).
int balanced_grid(int total_rows, int rows_per_cta, int limit) {
    const int needed = (total_rows + rows_per_cta - 1) / rows_per_cta;
    if (needed <= limit) return std::max(1, needed);
    int best = limit;
    double best_efficiency = 0.0;
    for (int grid = limit; grid >= limit - limit / 8 && grid >= 1; --grid) {
        const long long per_round = static_cast<long long>(grid) * rows_per_cta;
        const long long rounds = (total_rows + per_round - 1) / per_round;
        const double efficiency = static_cast<double>(total_rows) / (rounds * per_round) *
            (static_cast<double>(grid) / limit > 0.97 ? 1.0 : static_cast<double>(grid) / limit / 0.97);
        if (efficiency > best_efficiency + 1e-9) {
            best_efficiency = efficiency;
            best = grid;
        }
    }
    return best;
}

template <int CPL, int ACT, int EPI, int DEPTH>
cudaError_t launch_pipelined_depth(fortai_cuda_q8_context *c, const GemvParams &p) {
    auto kernel = q8_gemv_pipelined_kernel<CPL, ACT, EPI, DEPTH>;
    const size_t smem = pipelined_smem_bytes(p.width, p.blocks, CPL, EPI == kEpiSiluPair ? 2 : 1);
    cudaError_t error = cudaSuccess;
    if (smem > 48 * 1024) {
        error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
            static_cast<int>(smem));
        if (error != cudaSuccess) return error;
    }
    int per_sm = c->gemv_ctas_per_sm;
    if (per_sm <= 0) {
        // the occupancy query costs a microsecond or two per call: remember the last answer
        static size_t cached_smem[64] = {};
        static int cached_per_sm[64] = {};
        const int slot = c->device & 63;
        if (cached_per_sm[slot] > 0 && cached_smem[slot] == smem) {
            per_sm = cached_per_sm[slot];
        } else {
            error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kGemvThreads,
                smem);
            if (error != cudaSuccess) return error;
            if (per_sm < 1) per_sm = 1;
            cached_smem[slot] = smem;
            cached_per_sm[slot] = per_sm;
        }
    }
    const int limit = c->sm_count * per_sm;
    const int needed = (p.total_rows + kGemvWarps - 1) / kGemvWarps;
    const int grid = c->gemv_balance ? balanced_grid(p.total_rows, kGemvWarps, limit)
                                     : std::max(1, std::min(needed, limit));
    return launch_gemv_kernel(c, kernel, grid, kGemvThreads, smem, p, limit);
}

template <int CPL, int ACT, int EPI>
cudaError_t launch_pipelined_instance(fortai_cuda_q8_context *c, const GemvParams &p) {
    // the gate/up pair already has two rows per warp in flight
    if (EPI != kEpiSiluPair && EPI != kEpiStacked && c->gemv_depth == 2)
        return launch_pipelined_depth<CPL, ACT, EPI, 2>(c, p);
    return launch_pipelined_depth<CPL, ACT, EPI, 1>(c, p);
}

// The pipelined kernel needs width == 512 * CPL exactly and a single matrix (or the
// gate/up pair).  Returns false when the shape is not covered.
template <int ACT, int EPI>
bool launch_pipelined(fortai_cuda_q8_context *c, const GemvParams &p, cudaError_t *error) {
    if (p.width % 512 != 0) return false;
    // stacked matrices: plain epilogue with one row in flight; a convolution rides along
    // only there (a single matrix with a convolution has no caller)
    if (EPI == kEpiStacked && (p.segments < 2 || p.residual)) return false;
    if (EPI == kEpiPlain && (p.segments != 1 || p.conv_weights)) return false;
    if (EPI == kEpiPeers && p.segments != 1) return false;
    if (EPI == kEpiSiluPair && p.width / 512 > 5) return false;   // two rows double-buffered
    switch (p.width / 512) {
    case 1: *error = launch_pipelined_instance<1, ACT, EPI>(c, p); return true;
    case 2: *error = launch_pipelined_instance<2, ACT, EPI>(c, p); return true;
    case 3: *error = launch_pipelined_instance<3, ACT, EPI>(c, p); return true;
    case 4: *error = launch_pipelined_instance<4, ACT, EPI>(c, p); return true;
    case 5: *error = launch_pipelined_instance<5, ACT, EPI>(c, p); return true;
    case 8: *error = launch_pipelined_instance<8, ACT, EPI>(c, p); return true;
    case 10: *error = launch_pipelined_instance<10, ACT, EPI>(c, p); return true;
    default: return false;
    }
}

template <int G, int SPLIT, int ACT, int EPI>
cudaError_t launch_slice_instance(fortai_cuda_q8_context *c, const GemvParams &p) {
    auto kernel = q8_gemv_slice_kernel<G, SPLIT, ACT, EPI>;
    const size_t smem = slice_smem_bytes(p.width, p.blocks, G);
    cudaError_t error = cudaSuccess;
    if (smem > 48 * 1024) {
        error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
            static_cast<int>(smem));
        if (error != cudaSuccess) return error;
    }
    int per_sm = c->gemv_ctas_per_sm;
    if (per_sm <= 0) {
        static size_t cached_smem[64] = {};
        static int cached_per_sm[64] = {};
        const int slot = c->device & 63;
        if (cached_per_sm[slot] > 0 && cached_smem[slot] == smem) {
            per_sm = cached_per_sm[slot];
        } else {
            error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kGemvThreads,
                smem);
            if (error != cudaSuccess) return error;
            if (per_sm < 1) per_sm = 1;
            cached_smem[slot] = smem;
            cached_per_sm[slot] = per_sm;
        }
    }
    // the same number of rows for every CTA (as far as the row count allows)
    const int rows_per_round = kGemvWarps / SPLIT;
    const int needed = (p.total_rows + rows_per_round - 1) / rows_per_round;
    const int limit = c->sm_count * per_sm;
    const int rounds = (needed + limit - 1) / limit;
    const int grid = std::max(1, (needed + rounds - 1) / rounds);
    return launch_gemv_kernel(c, kernel, grid, kGemvThreads, smem, p, limit);
}

// Few long rows: K-slices of a row on 4 or 8 warps.  Chosen by itself for plain single-matrix
// products of at least 16 granules (8192 elements) whose rows are fewer than two rounds of a
// warp-per-row grid; "gemv_split" = 1 turns it off, 4 or 8 force it where the shape allows.
template <int ACT, int EPI>
bool launch_slice(fortai_cuda_q8_context *c, const GemvParams &p, cudaError_t *error) {
    if (p.segments != 1 || p.norm_weights || p.conv_weights || p.width % 512 != 0 ||
        c->gemv_split == 1 || (EPI == kEpiPeers && p.residual))
        return false;
    const int granules = p.width / 512;
    int split = c->gemv_split;
    if (split == 0) {
        if (granules < 16 || p.total_rows > 2 * c->sm_count * 4 * kGemvWarps) return false;
        // measured: 34 granules 17.1 us with 8 warps per row against 17.8 with 4; 19 granules
        // 7.7 us with 4 against 8.1 with 8
        split = granules >= 24 ? 8 : 4;
    }
    const int most = (granules + split - 1) / split;
    if (most > 9 || granules < split) return false;
    if (split == 4) {
        if (most <= 3) *error = launch_slice_instance<3, 4, ACT, EPI>(c, p);
        else if (most <= 5) *error = launch_slice_instance<5, 4, ACT, EPI>(c, p);
        else *error = launch_slice_instance<9, 4, ACT, EPI>(c, p);
    } else if (split == 8) {
        if (most <= 3) *error = launch_slice_instance<3, 8, ACT, EPI>(c, p);
        else if (most <= 5) *error = launch_slice_instance<5, 8, ACT, EPI>(c, p);
        else *error = launch_slice_instance<9, 8, ACT, EPI>(c, p);
    } else {
        return false;
    }
    return true;
}

// Kernel choice: the slice kernel for few long rows, the pipelined kernel where the width is
// one of its granule counts, else the half-block kernel ("gemv_variant" = 1: always that one).
template <int ACT>
cudaError_t launch_gemv_act(fortai_cuda_q8_context *c, const GemvParams &p, int epi) {
    // the fused norm, residual and convolution exist for the plain and gate/up epilogues only
    if ((p.norm_weights || p.residual || p.conv_weights) && epi != kEpiPlain &&
        epi != kEpiSiluPair)
        return cudaErrorNotSupported;
    if (c->gemv_variant == 0) {
        cudaError_t error = cudaSuccess;
        bool done = false;
        if (epi == kEpiPlain && launch_slice<ACT, kEpiPlain>(c, p, &error)) return error;
        if (epi == kEpiPeers && launch_slice<ACT, kEpiPeers>(c, p, &error)) return error;
        if (epi == kEpiPlain && p.segments > 1)
            done = launch_pipelined<ACT, kEpiStacked>(c, p, &error);
        if (!done && epi == kEpiPlain) done = launch_pipelined<ACT, kEpiPlain>(c, p, &error);
        else if (epi == kEpiSiluPair) done = launch_pipelined<ACT, kEpiSiluPair>(c, p, &error);
        else if (epi == kEpiPeers) done = launch_pipelined<ACT, kEpiPeers>(c, p, &error);
        if (done) return error;
    }
    switch (epi) {
    case kEpiPlain: return launch_direct<ACT, kEpiPlain>(c, p);
    case kEpiSiluPair: return launch_direct<ACT, kEpiSiluPair>(c, p);
    case kEpiPeers: return launch_direct<ACT, kEpiPeers>(c, p);
    default: return launch_direct<kActQ8, kEpiBlockDots>(c, p);
    }
}

// Launch with the activation exactly as given (no preparation pass, no allocation).
cudaError_t launch_gemv_raw(fortai_cuda_q8_context *c, const GemvParams &p, int act, int epi) {
    // fp32 and prepared activations are read with 16-byte loads, Q8_0 ones with 2-byte loads
    const uintptr_t address = reinterpret_cast<uintptr_t>(p.activation);
    if ((act != kActQ8 && (address & 15)) || (act == kActQ8 && (address & 1)))
        return cudaErrorMisalignedAddress;
    if (act == kActF32) return launch_gemv_act<kActF32>(c, p, epi);
    if (act == kActPlanar) return launch_gemv_act<kActPlanar>(c, p, epi);
    return launch_gemv_act<kActQ8>(c, p, epi);
}

cudaError_t launch_planar_prepare(fortai_cuda_q8_context *c, const void *activation, int act,
    int width, int blocks, uint8_t *image) {
    const int grid = std::max(1, std::min((blocks + 7) / 8, c->sm_count * 4));
    if (act == kActF32)
        return launch_overlapped(c, q8_planar_prepare_kernel<kActF32>, grid, 256, 0, activation,
            width, blocks, image);
    return launch_overlapped(c, q8_planar_prepare_kernel<kActQ8>, grid, 256, 0, activation, width,
        blocks, image);
}

// Long activation vectors are quantized / unpacked once into the context's prepared image
// instead of in every CTA's prologue (K = 17408 is 68 KB of fp32 per CTA otherwise).
cudaError_t launch_gemv(fortai_cuda_q8_context *c, const GemvParams &p, int act, int epi) {
    // (a fused norm is computed in the GEMV prologue, not by the preparation pass)
    if (act == kActPlanar || epi == kEpiBlockDots || p.width < c->planar_min_width ||
        p.norm_weights)
        return launch_gemv_raw(c, p, act, epi);
    const uintptr_t address = reinterpret_cast<uintptr_t>(p.activation);
    if ((act == kActF32 && (address & 3)) || (act == kActQ8 && (address & 1)))
        return cudaErrorMisalignedAddress;
    cudaError_t error = grow(reinterpret_cast<void **>(&c->scratch_planar),
        &c->scratch_planar_bytes, activation_smem_bytes(p.width, p.blocks));
    if (error == cudaSuccess)
        error = launch_planar_prepare(c, p.activation, act, p.width, p.blocks, c->scratch_planar);
    if (error != cudaSuccess) return error;
    GemvParams prepared = p;
    prepared.activation = c->scratch_planar;
    return launch_gemv_raw(c, prepared, kActPlanar, epi);
}

// The device-side alias of a host pointer when that memory is page-locked and mapped into
// the device's address space (16-byte aligned), else null.  Never fails: unknown pointers
// are pageable memory.
float *mapped_host_pointer(const void *host) {
    cudaPointerAttributes attributes = {};
    if (cudaPointerGetAttributes(&attributes, host) != cudaSuccess) {
        cudaGetLastError();                       // not an error for the caller
        return nullptr;
    }
    if (attributes.type != cudaMemoryTypeHost || !attributes.devicePointer) return nullptr;
    if (reinterpret_cast<uintptr_t>(attributes.devicePointer) % 16 != 0) return nullptr;
    return static_cast<float *>(attributes.devicePointer);
}

GemvParams single_params(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w,
    const void *activation, float *output) {
    GemvParams p = {};
    p.weights[0] = w->data;
    p.outputs[0] = output;
    p.rows[0] = w->rows;
    p.segments = 1;
    p.total_rows = w->rows;
    p.width = w->width;
    p.blocks = w->blocks;
    p.row_stride = w->row_stride;
    p.activation = activation;
    p.status = c->status_device;
    return p;
}

cudaError_t launch_quantize(fortai_cuda_q8_context *c, const float *input, uint8_t *output,
    size_t blocks) {
    const long long want = static_cast<long long>((blocks + 7) / 8);
    const int grid = static_cast<int>(std::max<long long>(1,
        std::min<long long>(want, static_cast<long long>(c->sm_count) * 16)));
    return launch_overlapped(c, q8_quantize_kernel, grid, 256, 0, input, output,
        static_cast<long long>(blocks));
}

bool owned(const fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w) {
    return c && w && w->context == c && w->data;
}

int create_context(int device, bool borrow, cudaStream_t stream, fortai_cuda_q8_context **out) {
    if (!out || device < 0) return FORTAI_CUDA_INVALID;
    *out = nullptr;
    auto *c = new (std::nothrow) fortai_cuda_q8_context;
    if (!c) return FORTAI_CUDA_RUNTIME_ERROR;
    c->device = device;
    c->owns_stream = !borrow;
    c->stream = stream;
    bool ok = cudaSetDevice(device) == cudaSuccess;
    if (ok && !borrow)
        ok = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreate(&c->start) == cudaSuccess &&
        cudaEventCreate(&c->stop) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&c->position), sizeof(int)) == cudaSuccess &&
        cudaMemsetAsync(c->position, 0, sizeof(int), c->stream) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&c->cta_counter), sizeof(unsigned)) ==
        cudaSuccess && cudaMemsetAsync(c->cta_counter, 0, sizeof(unsigned), c->stream) ==
        cudaSuccess;
    ok = ok && cudaHostAlloc(reinterpret_cast<void **>(&c->status_host), sizeof(int),
        cudaHostAllocMapped) == cudaSuccess;
    if (ok) {
        *c->status_host = kStatusOk;
        ok = cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->status_device),
            c->status_host, 0) == cudaSuccess;
    }
    ok = ok && cudaHostAlloc(reinterpret_cast<void **>(&c->done_host), sizeof(unsigned),
        cudaHostAllocMapped) == cudaSuccess;
    if (ok) {
        *c->done_host = 0;
        ok = cudaHostGetDevicePointer(reinterpret_cast<void **>(&c->done_device), c->done_host,
            0) == cudaSuccess;
    }
    int sms = 0;
    if (ok && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess
        && sms > 0)
        c->sm_count = sms;
    ok = ok && cudaStreamSynchronize(c->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        fortai_cuda_q8_context_destroy(c);
        return FORTAI_CUDA_RUNTIME_ERROR;
    }
    *out = c;
    return FORTAI_CUDA_OK;
}

int upload_weights(fortai_cuda_q8_context *context, const void *host_weights,
    size_t weight_bytes, int rows, int width, int first_block, int block_count,
    fortai_cuda_q8_weights **weights) {
    if (!context || !host_weights || !weights || rows <= 0 || width <= 0 ||
        width % kBlockElems != 0) return FORTAI_CUDA_INVALID;
    *weights = nullptr;
    const int src_blocks = width / kBlockElems;
    if (first_block < 0 || block_count <= 0 || first_block + block_count > src_blocks)
        return FORTAI_CUDA_INVALID;
    const size_t expected = static_cast<size_t>(rows) * src_blocks * kBlockBytes;
    if (weight_bytes < expected) return FORTAI_CUDA_INVALID;
    auto *w = new (std::nothrow) fortai_cuda_q8_weights;
    if (!w) return FORTAI_CUDA_RUNTIME_ERROR;
    w->context = context;
    w->rows = rows;
    w->width = block_count * kBlockElems;
    w->blocks = block_count;
    w->row_stride = static_cast<int>(row_stride_bytes(block_count));
    cudaSetDevice(context->device);
    uint8_t *staging = nullptr;
    const size_t device_bytes = static_cast<size_t>(rows) * w->row_stride;
    // 32 spare bytes: the prefill kernel fetches a row's fp16 scales in aligned 16-byte
    // pieces, and the last piece of the last row may reach past the row's padding
    cudaError_t error = cudaMalloc(reinterpret_cast<void **>(&w->data), device_bytes + 32);
    if (error == cudaSuccess) error = cudaMalloc(reinterpret_cast<void **>(&staging), expected);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(staging, host_weights, expected, cudaMemcpyHostToDevice,
            context->stream);
    if (error == cudaSuccess && device_bytes != static_cast<size_t>(rows) * block_count * kBlockBytes)
        error = cudaMemsetAsync(w->data, 0, device_bytes, context->stream);
    if (error == cudaSuccess) {
        const long long total = static_cast<long long>(rows) * block_count;
        const int grid = static_cast<int>(std::max<long long>(1,
            std::min<long long>((total + 255) / 256, 148LL * 32)));
        q8_repack_kernel<<<grid, 256, 0, context->stream>>>(staging, w->data, rows, src_blocks,
            first_block, block_count, w->row_stride);
        ++context->launches;
        error = cudaGetLastError();
    }
    if (error == cudaSuccess) error = cudaStreamSynchronize(context->stream);
    cudaFree(staging);
    if (error != cudaSuccess) {
        cudaFree(w->data);
        delete w;
        return fail(context, "weight upload", error);
    }
    *weights = w;
    return FORTAI_CUDA_OK;
}

struct HostRequest {
    const fortai_cuda_q8_weights *weights;
    float *output;
    size_t output_bytes;
};

// reference: matvec_host_many, backend.cu:249-315
int matvec_host_many(fortai_cuda_q8_context *c, const HostRequest *requests, int count,
    const void *host_activation, size_t activation_bytes, float *elapsed_ms,
    float *combined_output) {
    if (!c || !requests || count <= 0 || count > kMaxSegments || !host_activation || !elapsed_ms)
        return FORTAI_CUDA_INVALID;
    const fortai_cuda_q8_weights *first = requests[0].weights;
    if (!first || !first->data) return FORTAI_CUDA_INVALID;
    const size_t expected_activation = static_cast<size_t>(first->blocks) * kBlockBytes;
    // the reference returns the outputs back to back only when it fuses the
    // launch, i.e. for fewer than 128 blocks per row
    if (combined_output && first->blocks >= 128) return FORTAI_CUDA_INVALID;
    size_t total_rows = 0;
    for (int i = 0; i < count; ++i) {
        const fortai_cuda_q8_weights *w = requests[i].weights;
        if (!owned(c, w) || w->blocks != first->blocks || !requests[i].output)
            return FORTAI_CUDA_INVALID;
        if (activation_bytes < expected_activation ||
            requests[i].output_bytes < static_cast<size_t>(w->rows) * sizeof(float))
            return FORTAI_CUDA_INVALID;
        total_rows += static_cast<size_t>(w->rows);
    }
    cudaSetDevice(c->device);
    cudaError_t error = ensure_scratch(c, expected_activation, total_rows * sizeof(float));
    // a single product into page-locked, device-mapped memory: the kernel stores there itself
    float *mapped_output = nullptr;
    if (error == cudaSuccess && count == 1 && !combined_output && c->host_direct_output &&
        first->width % 512 == 0)
        mapped_output = mapped_host_pointer(requests[0].output);
    if (error == cudaSuccess) error = cudaEventRecord(c->start, c->stream);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(c->scratch_activation, host_activation, expected_activation,
            cudaMemcpyHostToDevice, c->stream);
    if (error == cudaSuccess && mapped_output) {
        GemvParams p = single_params(c, first, c->scratch_activation, c->scratch_output);
        p.peers = 1;
        p.peer_outputs[0] = mapped_output;
            p.peer_flush = c->host_flush_rows;
        error = launch_gemv(c, p, kActQ8, kEpiPeers);
    } else if (error == cudaSuccess) {
        GemvParams p = {};
        size_t offset = 0;
        for (int i = 0; i < count; ++i) {
            p.weights[i] = requests[i].weights->data;
            p.outputs[i] = c->scratch_output + offset;
            p.rows[i] = requests[i].weights->rows;
            offset += static_cast<size_t>(requests[i].weights->rows);
        }
        p.segments = count;
        p.total_rows = static_cast<int>(total_rows);
        p.width = first->width;
        p.blocks = first->blocks;
        p.row_stride = first->row_stride;
        p.activation = c->scratch_activation;
        p.status = c->status_device;
        error = launch_gemv(c, p, kActQ8, kEpiPlain);
    }
    if (error == cudaSuccess && !mapped_output) {
        if (combined_output) {
            error = cudaMemcpyAsync(combined_output, c->scratch_output,
                total_rows * sizeof(float), cudaMemcpyDeviceToHost, c->stream);
        } else {
            size_t offset = 0;
            for (int i = 0; i < count && error == cudaSuccess; ++i) {
                const size_t rows = static_cast<size_t>(requests[i].weights->rows);
                error = cudaMemcpyAsync(requests[i].output, c->scratch_output + offset,
                    rows * sizeof(float), cudaMemcpyDeviceToHost, c->stream);
                offset += rows;
            }
        }
    }
    if (error == cudaSuccess) error = cudaEventRecord(c->stop, c->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(c->stop);
    if (error == cudaSuccess) error = cudaEventElapsedTime(elapsed_ms, c->start, c->stop);
    return finish(c, "grouped host matvec", error);
}

bool ffn_shapes_ok(const fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *gate,
    const fortai_cuda_q8_weights *up, const fortai_cuda_q8_weights *down) {
    return owned(c, gate) && owned(c, up) && owned(c, down) && gate->blocks == up->blocks &&
        gate->rows == up->rows && gate->rows == down->blocks * kBlockElems;
}

// quantize(x) is folded into the gate/up kernel when x is fp32; then
// h = silu(gate.x) * (up.x) -> scratch_output, Q8(h) -> scratch_activation, down.
// The caller's glue around a projection chain, fused into its first and last GEMV:
// the input is RMS-normalised with `norm_weights` in the first prologue, and the last
// epilogue adds `residual` (which may be the output vector itself).  All null = plain.
struct Glue {
    const float *norm_weights = nullptr;
    float epsilon = 0.0f;
    const float *residual = nullptr;
};

// A column-sharded down projection whose ranks exchange their partial output vectors inside
// the GEMV: rank r's partial travels as (value, call number) pairs into slot r of every rank's
// pair array, and the kernel's tail adds the slots in rank order into the output.
struct FfnExchange {
    float *pairs[kMaxPeers] = {};      // every rank's pair array, at the half this call uses
    int peers = 0;
    int rank = 0;
    float *output = nullptr;           // this rank's sum
};

void attach_exchange(fortai_cuda_q8_context *c, GemvParams *d, const FfnExchange &x, int hidden) {
    for (int i = 0; i < x.peers; ++i) d->peer_outputs[i] = x.pairs[i];
    d->outputs[0] = nullptr;
    d->peers = x.peers;
    d->peer_flush = c->peer_flush_rows;
    d->first_row = x.rank * hidden;
    d->my_rank = x.rank;
    if (++c->ll_sequence == 0) ++c->ll_sequence;
    d->ll_sequence = c->ll_sequence;
    d->ll_output = x.output;
    d->ll_total = hidden;
    d->ll_reduce = x.peers;
    d->flag_wait_clocks = static_cast<long long>(c->peer_wait_clocks_millions) * 1000000LL;
    d->overlap_ok = c->peer_overlap;
}

cudaError_t enqueue_ffn(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *gate,
    const fortai_cuda_q8_weights *up, const fortai_cuda_q8_weights *down, const void *activation,
    int act, float *output, const Glue &glue = Glue(), const FfnExchange *exchange = nullptr) {
    const int down_epi = exchange ? kEpiPeers : kEpiPlain;
    GemvParams p = single_params(c, gate, activation, c->scratch_output);
    p.weights[1] = up->data;
    p.rows[1] = up->rows;
    p.segments = 2;
    p.norm_weights = glue.norm_weights;
    p.norm_epsilon = glue.epsilon;
    // size the prepared-image scratch for both halves before anything is enqueued, so that
    // it is never reallocated between the two GEMVs
    const int widest = std::max(gate->width, down->width);
    cudaError_t error = cudaSuccess;
    if (widest >= c->planar_min_width)
        error = grow(reinterpret_cast<void **>(&c->scratch_planar), &c->scratch_planar_bytes,
            activation_smem_bytes(widest, widest / kBlockElems));
    if (error == cudaSuccess) error = launch_gemv(c, p, act, kEpiSiluPair);
    if (error != cudaSuccess) return error;
    if (down->width >= c->planar_min_width) {
        // long hidden vector: quantize it once, straight into the prepared image
        error = grow(reinterpret_cast<void **>(&c->scratch_planar), &c->scratch_planar_bytes,
            activation_smem_bytes(down->width, down->blocks));
        if (error == cudaSuccess)
            error = launch_planar_prepare(c, c->scratch_output, kActF32, down->width,
                down->blocks, c->scratch_planar);
        if (error == cudaSuccess) {
            GemvParams d = single_params(c, down, c->scratch_planar, output);
            d.residual = glue.residual;
            if (exchange) attach_exchange(c, &d, *exchange, down->rows);
            error = launch_gemv_raw(c, d, kActPlanar, down_epi);
        }
        return error;
    }
    if (down->width <= c->ffn_quantize_in_gemv) {
        // short hidden vectors: the down projection quantizes them in its own prologue (same
        // bytes, one launch less; from about 4096 elements on every CTA redoing the work
        // costs more than the separate kernel)
        GemvParams d = single_params(c, down, c->scratch_output, output);
        d.residual = glue.residual;
        if (exchange) attach_exchange(c, &d, *exchange, down->rows);
        return launch_gemv_raw(c, d, kActF32, down_epi);
    }
    error = launch_quantize(c, c->scratch_output, c->scratch_activation,
        static_cast<size_t>(down->blocks));
    if (error == cudaSuccess) {
        GemvParams d = single_params(c, down, c->scratch_activation, output);
        d.residual = glue.residual;
        if (exchange) attach_exchange(c, &d, *exchange, down->rows);
        error = launch_gemv(c, d, kActQ8, down_epi);
    }
    return error;
}


}  // namespace

// ===========================================================================
// Part 1: reference interface
// ===========================================================================
extern "C" int fortai_cuda_q8_context_create(int device, fortai_cuda_q8_context **context) {
    return create_context(device, false, nullptr, context);
}

extern "C" int fortai_cuda_q8_context_create_on_stream(int device, void *stream,
    fortai_cuda_q8_context **context) {
    return create_context(device, true, static_cast<cudaStream_t>(stream), context);
}

extern "C" int fortai_cuda_q8_context_destroy(fortai_cuda_q8_context *context) {
    if (!context) return FORTAI_CUDA_OK;
    cudaSetDevice(context->device);
    if (context->graph_exec) cudaGraphExecDestroy(context->graph_exec);
    if (context->graph) cudaGraphDestroy(context->graph);
    cudaFree(context->position);
    cudaFree(context->cta_counter);
    cudaFree(context->scratch_activation);
    cudaFree(context->scratch_output);
    cudaFree(context->scratch_aux);
    cudaFree(context->scratch_planar);
    if (context->status_host) cudaFreeHost(context->status_host);
    if (context->done_host) cudaFreeHost(context->done_host);
    if (context->start) cudaEventDestroy(context->start);
    if (context->stop) cudaEventDestroy(context->stop);
    if (context->owns_stream && context->stream) cudaStreamDestroy(context->stream);
    delete context;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_context_set_position(fortai_cuda_q8_context *context,
    int position) {
    if (!context || !context->position || position < 0) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaMemcpyAsync(context->position, &position, sizeof(position),
        cudaMemcpyHostToDevice, context->stream);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "set device position", error);
}

extern "C" int fortai_cuda_q8_context_capture_begin(fortai_cuda_q8_context *context) {
    if (!context || context->graph || context->graph_exec) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaStreamBeginCapture(context->stream,
        cudaStreamCaptureModeGlobal);
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(context, "begin CUDA graph capture", error);
}

extern "C" int fortai_cuda_q8_context_capture_end(fortai_cuda_q8_context *context) {
    if (!context) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = cudaStreamEndCapture(context->stream, &context->graph);
    if (error == cudaSuccess)
        error = cudaGraphInstantiate(&context->graph_exec, context->graph, nullptr, nullptr, 0);
    if (error != cudaSuccess) {
        if (context->graph_exec) cudaGraphExecDestroy(context->graph_exec);
        if (context->graph) cudaGraphDestroy(context->graph);
        context->graph_exec = nullptr;
        context->graph = nullptr;
        return fail(context, "end CUDA graph capture", error);
    }
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_context_graph_launch(fortai_cuda_q8_context *context) {
    if (!context || !context->graph_exec) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaGraphLaunch(context->graph_exec, context->stream);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "launch CUDA graph", error);
}

extern "C" int fortai_cuda_q8_weights_upload(fortai_cuda_q8_context *context,
    const void *host_weights, size_t weight_bytes, int rows, int width,
    fortai_cuda_q8_weights **weights) {
    if (width <= 0 || width % kBlockElems != 0) return FORTAI_CUDA_INVALID;
    return upload_weights(context, host_weights, weight_bytes, rows, width, 0,
        width / kBlockElems, weights);
}

extern "C" int fortai_cuda_q8_weights_upload_columns(fortai_cuda_q8_context *context,
    const void *host_weights, size_t weight_bytes, int rows, int width, int first_block,
    int block_count, fortai_cuda_q8_weights **weights) {
    return upload_weights(context, host_weights, weight_bytes, rows, width, first_block,
        block_count, weights);
}

extern "C" int fortai_cuda_q8_weights_destroy(fortai_cuda_q8_weights *weights) {
    if (!weights) return FORTAI_CUDA_OK;
    if (weights->context) cudaSetDevice(weights->context->device);
    cudaFree(weights->data);
    delete weights;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_weights_shape(const fortai_cuda_q8_weights *weights, int *rows,
    int *width) {
    if (!weights || !rows || !width) return FORTAI_CUDA_INVALID;
    *rows = weights->rows;
    *width = weights->width;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_device_buffer_create(fortai_cuda_q8_context *context, size_t bytes,
    void **device_buffer) {
    if (!context || !device_buffer || bytes == 0) return FORTAI_CUDA_INVALID;
    *device_buffer = nullptr;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaMalloc(device_buffer, bytes);
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(context, "device buffer allocation", error);
}

extern "C" int fortai_cuda_q8_device_buffer_destroy(fortai_cuda_q8_context *context,
    void *device_buffer) {
    if (!context || !device_buffer) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaFree(device_buffer);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device buffer free", error);
}

extern "C" int fortai_cuda_q8_device_buffer_upload(fortai_cuda_q8_context *context,
    void *device_buffer, const void *host_data, size_t bytes) {
    if (!context || !device_buffer || !host_data || bytes == 0) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = cudaMemcpyAsync(device_buffer, host_data, bytes, cudaMemcpyHostToDevice,
        context->stream);
    if (error == cudaSuccess) error = cudaStreamSynchronize(context->stream);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device upload", error);
}

extern "C" int fortai_cuda_q8_device_buffer_upload_ptr(fortai_cuda_q8_context *context,
    void *device_buffer, const void *host_data, size_t bytes) {
    if (!context || !device_buffer || !host_data || bytes == 0) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaMemcpyAsync(device_buffer, host_data, bytes,
        cudaMemcpyHostToDevice, context->stream);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "async device upload", error);
}

extern "C" int fortai_cuda_q8_device_buffer_download(fortai_cuda_q8_context *context,
    void *host_data, const void *device_buffer, size_t bytes) {
    if (!context || !device_buffer || !host_data || bytes == 0) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = cudaMemcpyAsync(host_data, device_buffer, bytes, cudaMemcpyDeviceToHost,
        context->stream);
    if (error == cudaSuccess) error = cudaStreamSynchronize(context->stream);
    return finish(context, "device download", error);
}

extern "C" int fortai_cuda_q8_matvec_resident(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    float *kernel_ms) {
    if (!owned(context, weights) || !device_activation || !device_output || !kernel_ms)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess) {
        const GemvParams p = single_params(context, weights, device_activation,
            static_cast<float *>(device_output));
        error = launch_gemv(context, p, kActQ8, kEpiPlain);
    }
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    if (error == cudaSuccess)
        error = cudaEventElapsedTime(kernel_ms, context->start, context->stop);
    return finish(context, "resident matvec", error);
}

// The resident matvec without its event pair and wait: pre-quantized device activation in,
// enqueue only (what the reference's micro-benchmark times back to back).
extern "C" int fortai_cuda_q8_matvec_device_q8(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !device_output ||
        output_elements < static_cast<size_t>(weights->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const GemvParams p = single_params(context, weights, device_activation,
        static_cast<float *>(device_output));
    const cudaError_t error = launch_gemv(context, p, kActQ8, kEpiPlain);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device Q8 matvec", error);
}

extern "C" int fortai_cuda_q8_matvec_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !device_output ||
        activation_elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(weights->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const GemvParams p = single_params(context, weights, device_activation,
        static_cast<float *>(device_output));
    const cudaError_t error = launch_gemv(context, p, kActF32, kEpiPlain);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device F32 matvec", error);
}

extern "C" int fortai_cuda_qwen35_embedding_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, int64_t token_id, void *device_output,
    size_t output_elements) {
    if (!owned(context, weights) || !device_output || token_id < 0 ||
        token_id >= weights->rows || output_elements < static_cast<size_t>(weights->width))
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    q8_dequantize_row_kernel<<<(weights->width + 255) / 256, 256, 0, context->stream>>>(
        weights->data, token_id, weights->width, weights->row_stride,
        static_cast<float *>(device_output));
    ++context->launches;
    const cudaError_t error = cudaGetLastError();
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device Q8 embedding", error);
}

extern "C" int fortai_cuda_qwen35_copy_device(fortai_cuda_q8_context *context,
    const void *device_input, void *device_output, size_t bytes) {
    if (!context || !device_input || !device_output || bytes == 0) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = cudaMemcpyAsync(device_output, device_input, bytes,
        cudaMemcpyDeviceToDevice, context->stream);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device copy", error);
}

namespace {

__global__ void add_kernel(const float *left, const float *right, float *output, int elements) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < elements) output[i] = left[i] + right[i];
}

// One CTA; squares are accumulated in double as in the reference
// (qwen_rms_norm_float, backend.cu:518-537).
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float *input, const float *weights, float *output, int elements,
    float epsilon) {
    __shared__ double partial[8];
    double sum = 0.0;
    for (int i = threadIdx.x; i < elements; i += blockDim.x) {
        const double v = static_cast<double>(input[i]);
        sum += v * v;
    }
    for (int offset = 16; offset; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = sum;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < 8; ++w) total += partial[w];
    const float inverse = 1.0f / sqrtf(static_cast<float>(total /
        static_cast<double>(elements)) + epsilon);
    for (int i = threadIdx.x; i < elements; i += blockDim.x)
        output[i] = input[i] * inverse * weights[i];
}

}  // namespace

extern "C" int fortai_cuda_qwen35_add_device(fortai_cuda_q8_context *context,
    const void *device_left, const void *device_right, void *device_output, size_t elements) {
    if (!context || !device_left || !device_right || !device_output || elements == 0 ||
        elements > static_cast<size_t>(INT32_MAX)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    add_kernel<<<(static_cast<int>(elements) + 255) / 256, 256, 0, context->stream>>>(
        static_cast<const float *>(device_left), static_cast<const float *>(device_right),
        static_cast<float *>(device_output), static_cast<int>(elements));
    ++context->launches;
    const cudaError_t error = cudaGetLastError();
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device add", error);
}

extern "C" int fortai_cuda_qwen35_rms_norm_device(fortai_cuda_q8_context *context,
    const void *device_input, const void *device_weights, void *device_output, size_t elements,
    float epsilon) {
    if (!context || !device_input || !device_weights || !device_output || elements == 0 ||
        elements > static_cast<size_t>(INT32_MAX) || epsilon <= 0.0f)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    rms_norm_kernel<<<1, 256, 0, context->stream>>>(static_cast<const float *>(device_input),
        static_cast<const float *>(device_weights), static_cast<float *>(device_output),
        static_cast<int>(elements), epsilon);
    ++context->launches;
    const cudaError_t error = cudaGetLastError();
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device RMS norm", error);
}

extern "C" int fortai_cuda_q8_matvec_host(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *host_activation, size_t activation_bytes,
    float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!owned(context, weights) || !host_activation || !host_output || !elapsed_ms ||
        activation_bytes < static_cast<size_t>(weights->blocks) * kBlockBytes ||
        output_bytes < static_cast<size_t>(weights->rows) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    const HostRequest request = {weights, host_output, output_bytes};
    return matvec_host_many(context, &request, 1, host_activation, activation_bytes, elapsed_ms,
        nullptr);
}

extern "C" int fortai_cuda_q8_matvec_host_pair(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const void *host_activation, size_t activation_bytes, float *first_output,
    size_t first_output_bytes, float *second_output, size_t second_output_bytes,
    float *elapsed_ms) {
    const HostRequest requests[] = {
        {first_weights, first_output, first_output_bytes},
        {second_weights, second_output, second_output_bytes}};
    return matvec_host_many(context, requests, 2, host_activation, activation_bytes, elapsed_ms,
        nullptr);
}

extern "C" int fortai_cuda_q8_matvec_host_triplet(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const fortai_cuda_q8_weights *third_weights, const void *host_activation,
    size_t activation_bytes, float *first_output, size_t first_output_bytes,
    float *second_output, size_t second_output_bytes, float *third_output,
    size_t third_output_bytes, float *elapsed_ms) {
    const HostRequest requests[] = {
        {first_weights, first_output, first_output_bytes},
        {second_weights, second_output, second_output_bytes},
        {third_weights, third_output, third_output_bytes}};
    return matvec_host_many(context, requests, 3, host_activation, activation_bytes, elapsed_ms,
        nullptr);
}

extern "C" int fortai_cuda_q8_matvec_host_triplet_contiguous(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const fortai_cuda_q8_weights *third_weights, const void *host_activation,
    size_t activation_bytes, float *host_output, size_t host_output_bytes, float *elapsed_ms) {
    if (!first_weights || !second_weights || !third_weights || !host_output)
        return FORTAI_CUDA_INVALID;
    const size_t first_bytes = static_cast<size_t>(first_weights->rows) * sizeof(float);
    const size_t second_bytes = static_cast<size_t>(second_weights->rows) * sizeof(float);
    const size_t third_bytes = static_cast<size_t>(third_weights->rows) * sizeof(float);
    if (host_output_bytes < first_bytes + second_bytes + third_bytes) return FORTAI_CUDA_INVALID;
    const HostRequest requests[] = {
        {first_weights, host_output, first_bytes},
        {second_weights, host_output + first_weights->rows, second_bytes},
        {third_weights, host_output + first_weights->rows + second_weights->rows, third_bytes}};
    return matvec_host_many(context, requests, 3, host_activation, activation_bytes, elapsed_ms,
        host_output);
}

extern "C" int fortai_cuda_q8_ffn_host(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *host_activation,
    size_t activation_bytes, float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!context || !gate_weights || !up_weights || !down_weights || !host_activation ||
        !host_output || !elapsed_ms) return FORTAI_CUDA_INVALID;
    if (!ffn_shapes_ok(context, gate_weights, up_weights, down_weights))
        return FORTAI_CUDA_INVALID;
    const size_t expected_activation = static_cast<size_t>(gate_weights->blocks) * kBlockBytes;
    const size_t down_activation = static_cast<size_t>(down_weights->blocks) * kBlockBytes;
    const size_t inner_bytes = static_cast<size_t>(gate_weights->rows) * sizeof(float);
    const size_t expected_output = static_cast<size_t>(down_weights->rows) * sizeof(float);
    if (activation_bytes < expected_activation || output_bytes < expected_output)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    // activation scratch: x's blocks, later overwritten by h's; output scratch:
    // h (inner floats) followed by the result (hidden floats)
    cudaError_t error = ensure_scratch(context, std::max(expected_activation, down_activation),
        inner_bytes + expected_output);
    if (error == cudaSuccess) error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(context->scratch_activation, host_activation,
            expected_activation, cudaMemcpyHostToDevice, context->stream);
    float *result = context->scratch_output + gate_weights->rows;
    if (error == cudaSuccess)
        error = enqueue_ffn(context, gate_weights, up_weights, down_weights,
            context->scratch_activation, kActQ8, result);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(host_output, result, expected_output, cudaMemcpyDeviceToHost,
            context->stream);
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    if (error == cudaSuccess)
        error = cudaEventElapsedTime(elapsed_ms, context->start, context->stop);
    return finish(context, "Qwen FFN host", error);
}

extern "C" int fortai_cuda_q8_ffn_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements) {
    if (!context || !gate_weights || !up_weights || !down_weights || !device_activation ||
        !device_output) return FORTAI_CUDA_INVALID;
    if (!ffn_shapes_ok(context, gate_weights, up_weights, down_weights) ||
        activation_elements != static_cast<size_t>(gate_weights->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(down_weights->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = ensure_scratch(context,
        static_cast<size_t>(down_weights->blocks) * kBlockBytes,
        static_cast<size_t>(gate_weights->rows) * sizeof(float));
    if (error == cudaSuccess)
        error = enqueue_ffn(context, gate_weights, up_weights, down_weights, device_activation,
            kActF32, static_cast<float *>(device_output));
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "Qwen FFN device", error);
}

extern "C" int fortai_cuda_q8_ffn_device_allreduce(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *const *peer_pairs, int peer_count, int my_rank,
    void *device_output, size_t output_elements) {
    if (!context || !gate_weights || !up_weights || !down_weights || !device_activation ||
        !device_output || !peer_pairs || peer_count <= 0 || peer_count > kMaxPeers ||
        my_rank < 0 || my_rank >= peer_count)
        return FORTAI_CUDA_INVALID;
    if (!ffn_shapes_ok(context, gate_weights, up_weights, down_weights) ||
        activation_elements != static_cast<size_t>(gate_weights->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(down_weights->rows)) return FORTAI_CUDA_INVALID;
    for (int i = 0; i < peer_count; ++i)
        if (!peer_pairs[i] || reinterpret_cast<uintptr_t>(peer_pairs[i]) % 8 != 0)
            return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(context->stream, &capture) == cudaSuccess &&
        capture != cudaStreamCaptureStatusNone) {
        fail(context, "all-reduce FFN cannot be captured into a CUDA graph "
                      "(its call number is a launch argument)");
        return FORTAI_CUDA_INVALID;
    }
    const int hidden = down_weights->rows;
    // two halves of the pair arrays, used alternately: a rank that runs ahead stores call
    // n+1's partial while a peer may still be adding call n's; it cannot reach call n+2 before
    // that peer has sent its own partial of call n+1, which it does after adding call n
    const size_t half = static_cast<size_t>(context->ffn_exchange_calls++ & 1u) * peer_count *
        hidden;
    FfnExchange exchange;
    for (int i = 0; i < peer_count; ++i)
        exchange.pairs[i] = reinterpret_cast<float *>(static_cast<uint2 *>(peer_pairs[i]) + half);
    exchange.peers = peer_count;
    exchange.rank = my_rank;
    exchange.output = static_cast<float *>(device_output);
    cudaError_t error = ensure_scratch(context,
        static_cast<size_t>(down_weights->blocks) * kBlockBytes,
        static_cast<size_t>(gate_weights->rows) * sizeof(float));
    if (error == cudaSuccess)
        error = enqueue_ffn(context, gate_weights, up_weights, down_weights, device_activation,
            kActF32, nullptr, Glue(), &exchange);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "all-reduce FFN", error);
}

// ---------------------------------------------------------------------------
// Qwen3.5 gated-delta-net ("recurrent") layer
// reference: backend/cuda/fortai_cuda_backend.cu:1298-1567
// ---------------------------------------------------------------------------
namespace {

cudaError_t device_copy_of(fortai_cuda_q8_context *c, float **destination, const void *source,
    size_t bytes) {
    cudaError_t error = cudaMalloc(reinterpret_cast<void **>(destination), bytes);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(*destination, source, bytes, cudaMemcpyHostToDevice, c->stream);
    return error;
}

void free_recurrent(fortai_cuda_qwen35_recurrent *layer) {
    cudaFree(layer->conv_weights);
    cudaFree(layer->ssm_a);
    cudaFree(layer->ssm_dt);
    cudaFree(layer->ssm_norm);
    cudaFree(layer->conv_state);
    cudaFree(layer->gdn_state);
    cudaFree(layer->projections);
    cudaFree(layer->gdn_output);
}

cudaError_t clear_recurrent_state(fortai_cuda_qwen35_recurrent *layer) {
    fortai_cuda_q8_context *c = layer->context;
    cudaError_t error = cudaMemsetAsync(layer->conv_state, 0,
        static_cast<size_t>(layer->conv_kernel - 1) * layer->conv_size * sizeof(float), c->stream);
    if (error == cudaSuccess)
        error = cudaMemsetAsync(layer->gdn_state, 0, static_cast<size_t>(layer->value_heads) *
            layer->head_size * layer->head_size * sizeof(float), c->stream);
    if (error == cudaSuccess) error = cudaStreamSynchronize(c->stream);
    return error;
}

// qkv, gate, alpha and beta share one activation: one fused launch, then the
// convolution, the normalisations, the state update and the output projection
// (whose prologue quantizes the fp32 layer output, so no scratch is touched).
cudaError_t enqueue_recurrent(fortai_cuda_qwen35_recurrent *layer, const void *activation,
    int act, float *output, const Glue &glue = Glue()) {
    fortai_cuda_q8_context *c = layer->context;
    float *qkv = layer->projections;
    float *gate = qkv + layer->conv_size;
    float *alpha = gate + layer->inner_size;
    float *beta = alpha + layer->value_heads;
    GemvParams p = single_params(c, layer->qkv, activation, qkv);
    const fortai_cuda_q8_weights *mats[4] = {layer->qkv, layer->gate, layer->alpha, layer->beta};
    float *outs[4] = {qkv, gate, alpha, beta};
    p.total_rows = 0;
    for (int i = 0; i < 4; ++i) {
        p.weights[i] = mats[i]->data;
        p.outputs[i] = outs[i];
        p.rows[i] = mats[i]->rows;
        p.total_rows += mats[i]->rows;
    }
    p.segments = 4;
    p.norm_weights = glue.norm_weights;
    p.norm_epsilon = glue.epsilon;
    // the convolution + SiLU over the qkv channels rides in this launch's epilogue
    const bool conv_in_gemv = c->gdn_conv_in_gemv != 0;
    if (conv_in_gemv) {
        p.conv_weights = layer->conv_weights;
        p.conv_state = layer->conv_state;
        p.conv_rows = layer->conv_size;
        p.conv_kernel = layer->conv_kernel;
    }
    cudaError_t error = launch_gemv(c, p, act, kEpiPlain);
    if (error != cudaSuccess) return error;
    if (!conv_in_gemv)
        error = launch_overlapped(c, gdn_conv_silu_kernel, (layer->conv_size + 255) / 256, 256, 0,
            qkv, layer->conv_weights, layer->conv_state, layer->conv_size, layer->conv_kernel);
    if (error == cudaSuccess)
        // one CTA per value head; enough warps that each walks one or two pairs of rows
        error = launch_overlapped(c, gdn_step_kernel, layer->value_heads,
            std::max(64, std::min(1024, layer->head_size * 8)),
            3 * layer->head_size * sizeof(float), qkv, gate, alpha, beta, layer->ssm_a, layer->ssm_dt,
            layer->ssm_norm, layer->gdn_state, layer->gdn_output, layer->state_size,
            layer->key_heads, layer->value_heads, layer->head_size, layer->epsilon);
    if (error != cudaSuccess) return error;
    GemvParams o = single_params(c, layer->out, layer->gdn_output, output);
    o.residual = glue.residual;
    return launch_gemv(c, o, kActF32, kEpiPlain);
}

}  // namespace

extern "C" int fortai_cuda_qwen35_recurrent_create(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *qkv_weights, const fortai_cuda_q8_weights *gate_weights,
    const fortai_cuda_q8_weights *alpha_weights, const fortai_cuda_q8_weights *beta_weights,
    const fortai_cuda_q8_weights *output_weights, const void *conv_weights,
    size_t conv_weight_bytes, int conv_size, int conv_kernel, const void *ssm_a,
    size_t ssm_a_bytes, const void *ssm_dt, size_t ssm_dt_bytes, const void *ssm_norm,
    size_t ssm_norm_bytes, int state_size, int key_heads, int value_heads, int head_size,
    int inner_size, float norm_epsilon, fortai_cuda_qwen35_recurrent **layer) {
    if (!context || !layer || !qkv_weights || !gate_weights || !alpha_weights || !beta_weights ||
        !output_weights || !conv_weights || !ssm_a || !ssm_dt || !ssm_norm || conv_size <= 0 ||
        conv_kernel < 2 || state_size <= 0 || key_heads <= 0 || value_heads <= 0 ||
        head_size <= 0 || inner_size <= 0 || value_heads % key_heads != 0 ||
        value_heads * head_size != inner_size) return FORTAI_CUDA_INVALID;
    *layer = nullptr;
    if (!owned(context, qkv_weights) || !owned(context, gate_weights) ||
        !owned(context, alpha_weights) || !owned(context, beta_weights) ||
        !owned(context, output_weights)) return FORTAI_CUDA_INVALID;
    // shapes this layer relies on: all four input projections read the same vector, the
    // projection outputs are what the later kernels index, and the output projection
    // consumes the inner vector
    if (gate_weights->width != qkv_weights->width || alpha_weights->width != qkv_weights->width ||
        beta_weights->width != qkv_weights->width || qkv_weights->rows != conv_size ||
        gate_weights->rows != inner_size || alpha_weights->rows != value_heads ||
        beta_weights->rows != value_heads || output_weights->width != inner_size ||
        conv_size < 2 * state_size * key_heads + inner_size) return FORTAI_CUDA_INVALID;
    if (conv_weight_bytes < static_cast<size_t>(conv_size) * conv_kernel * sizeof(float) ||
        ssm_a_bytes < static_cast<size_t>(value_heads) * sizeof(float) ||
        ssm_dt_bytes < static_cast<size_t>(value_heads) * sizeof(float) ||
        ssm_norm_bytes < static_cast<size_t>(head_size) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    auto *created = new (std::nothrow) fortai_cuda_qwen35_recurrent;
    if (!created) return FORTAI_CUDA_RUNTIME_ERROR;
    created->context = context;
    created->qkv = qkv_weights;
    created->gate = gate_weights;
    created->alpha = alpha_weights;
    created->beta = beta_weights;
    created->out = output_weights;
    created->conv_size = conv_size;
    created->conv_kernel = conv_kernel;
    created->state_size = state_size;
    created->key_heads = key_heads;
    created->value_heads = value_heads;
    created->head_size = head_size;
    created->inner_size = inner_size;
    created->epsilon = norm_epsilon;
    cudaSetDevice(context->device);
    cudaError_t error = device_copy_of(context, &created->conv_weights, conv_weights,
        static_cast<size_t>(conv_size) * conv_kernel * sizeof(float));
    if (error == cudaSuccess)
        error = device_copy_of(context, &created->ssm_a, ssm_a, value_heads * sizeof(float));
    if (error == cudaSuccess)
        error = device_copy_of(context, &created->ssm_dt, ssm_dt, value_heads * sizeof(float));
    if (error == cudaSuccess)
        error = device_copy_of(context, &created->ssm_norm, ssm_norm, head_size * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->conv_state),
            static_cast<size_t>(conv_kernel - 1) * conv_size * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->gdn_state),
            static_cast<size_t>(value_heads) * head_size * head_size * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->projections),
            (static_cast<size_t>(conv_size) + inner_size + 2 * value_heads) * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->gdn_output),
            static_cast<size_t>(inner_size) * sizeof(float));
    if (error == cudaSuccess) error = clear_recurrent_state(created);
    if (error != cudaSuccess) {
        free_recurrent(created);
        delete created;
        return fail(context, "Qwen recurrent create", error);
    }
    *layer = created;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_qwen35_recurrent_destroy(fortai_cuda_qwen35_recurrent *layer) {
    if (!layer) return FORTAI_CUDA_OK;
    if (layer->context) {
        cudaSetDevice(layer->context->device);
        free_recurrent(layer);
    }
    delete layer;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_qwen35_recurrent_reset(fortai_cuda_qwen35_recurrent *layer) {
    if (!layer || !layer->context) return FORTAI_CUDA_INVALID;
    cudaSetDevice(layer->context->device);
    const cudaError_t error = clear_recurrent_state(layer);
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(layer->context, "Qwen recurrent reset", error);
}

extern "C" int fortai_cuda_qwen35_recurrent_run(fortai_cuda_qwen35_recurrent *layer,
    const void *host_activation, size_t activation_bytes, float *host_output,
    size_t output_bytes, float *elapsed_ms) {
    if (!layer || !layer->context || !host_activation || !host_output || !elapsed_ms)
        return FORTAI_CUDA_INVALID;
    fortai_cuda_q8_context *c = layer->context;
    const size_t expected_activation = static_cast<size_t>(layer->qkv->blocks) * kBlockBytes;
    const size_t expected_output = static_cast<size_t>(layer->out->rows) * sizeof(float);
    if (activation_bytes < expected_activation || output_bytes < expected_output)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(c->device);
    cudaError_t error = ensure_scratch(c, expected_activation, expected_output);
    if (error == cudaSuccess) error = cudaEventRecord(c->start, c->stream);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(c->scratch_activation, host_activation, expected_activation,
            cudaMemcpyHostToDevice, c->stream);
    if (error == cudaSuccess)
        error = enqueue_recurrent(layer, c->scratch_activation, kActQ8, c->scratch_output);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(host_output, c->scratch_output, expected_output,
            cudaMemcpyDeviceToHost, c->stream);
    if (error == cudaSuccess) error = cudaEventRecord(c->stop, c->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(c->stop);
    if (error == cudaSuccess) error = cudaEventElapsedTime(elapsed_ms, c->start, c->stop);
    return finish(c, "Qwen recurrent run", error);
}

extern "C" int fortai_cuda_qwen35_recurrent_run_device(fortai_cuda_qwen35_recurrent *layer,
    const void *device_activation, size_t activation_elements, void *device_output,
    size_t output_elements) {
    if (!layer || !layer->context || !device_activation || !device_output)
        return FORTAI_CUDA_INVALID;
    if (activation_elements != static_cast<size_t>(layer->qkv->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(layer->out->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(layer->context->device);
    const cudaError_t error = enqueue_recurrent(layer, device_activation, kActF32,
        static_cast<float *>(device_output));
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(layer->context, "Qwen recurrent device run", error);
}

// ---------------------------------------------------------------------------
// Qwen3.5 gated attention layer
// reference: backend/cuda/fortai_cuda_backend.cu:1569-1731
// ---------------------------------------------------------------------------
namespace {

void free_attention(fortai_cuda_qwen35_attention *layer) {
    cudaFree(layer->q_norm);
    cudaFree(layer->k_norm);
    cudaFree(layer->key_cache);
    cudaFree(layer->value_cache);
    cudaFree(layer->projections);
    cudaFree(layer->attention);
}

cudaError_t clear_attention_state(fortai_cuda_qwen35_attention *layer) {
    fortai_cuda_q8_context *c = layer->context;
    cudaError_t error = cudaMemsetAsync(layer->key_cache, 0, static_cast<size_t>(layer->max_context) *
        layer->kv_heads * layer->head_size * sizeof(__half), c->stream);
    if (error == cudaSuccess)
        error = cudaMemsetAsync(layer->value_cache, 0, static_cast<size_t>(layer->max_context) *
            layer->kv_heads * layer->value_size * sizeof(__half), c->stream);
    if (error == cudaSuccess) error = cudaStreamSynchronize(c->stream);
    return error;
}

}  // namespace

extern "C" int fortai_cuda_qwen35_attention_create(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *query_weights, const fortai_cuda_q8_weights *key_weights,
    const fortai_cuda_q8_weights *value_weights, const fortai_cuda_q8_weights *output_weights,
    const void *query_norm, size_t query_norm_bytes, const void *key_norm,
    size_t key_norm_bytes, int heads, int key_value_heads, int head_size, int value_size,
    int max_context, int rope_dimension, float rope_base, float norm_epsilon,
    fortai_cuda_qwen35_attention **layer) {
    if (!context || !layer || !query_weights || !key_weights || !value_weights ||
        !output_weights || !query_norm || !key_norm || heads <= 0 || key_value_heads <= 0 ||
        head_size <= 0 || value_size <= 0 || max_context <= 0 || heads % key_value_heads != 0 ||
        rope_dimension < 0 ||
        (rope_dimension > 0 && (rope_dimension > head_size || rope_dimension % 2 != 0)) ||
        rope_base <= 0.0f || norm_epsilon <= 0.0f) return FORTAI_CUDA_INVALID;
    if (!owned(context, query_weights) || !owned(context, key_weights) ||
        !owned(context, value_weights) || !owned(context, output_weights) ||
        query_weights->rows != heads * 2 * head_size ||
        key_weights->rows != key_value_heads * head_size ||
        value_weights->rows != key_value_heads * value_size ||
        output_weights->blocks * kBlockElems != heads * value_size ||
        // the output gate of a head is the second half of its query slot
        value_size > head_size ||
        query_norm_bytes < static_cast<size_t>(head_size) * sizeof(float) ||
        key_norm_bytes < static_cast<size_t>(head_size) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    *layer = nullptr;
    auto *created = new (std::nothrow) fortai_cuda_qwen35_attention;
    if (!created) return FORTAI_CUDA_RUNTIME_ERROR;
    created->context = context;
    created->q = query_weights;
    created->k = key_weights;
    created->v = value_weights;
    created->out = output_weights;
    created->heads = heads;
    created->kv_heads = key_value_heads;
    created->head_size = head_size;
    created->value_size = value_size;
    created->max_context = max_context;
    created->rope_dimension = rope_dimension;
    created->rope_base = rope_base;
    created->epsilon = norm_epsilon;
    cudaSetDevice(context->device);
    const size_t projection_floats = static_cast<size_t>(heads) * 2 * head_size +
        static_cast<size_t>(key_value_heads) * (head_size + value_size);
    cudaError_t error = device_copy_of(context, &created->q_norm, query_norm,
        head_size * sizeof(float));
    if (error == cudaSuccess)
        error = device_copy_of(context, &created->k_norm, key_norm, head_size * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->key_cache),
            static_cast<size_t>(max_context) * key_value_heads * head_size * sizeof(__half));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->value_cache),
            static_cast<size_t>(max_context) * key_value_heads * value_size * sizeof(__half));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->projections),
            projection_floats * sizeof(float));
    if (error == cudaSuccess)
        error = cudaMalloc(reinterpret_cast<void **>(&created->attention),
            static_cast<size_t>(heads) * value_size * sizeof(float));
    if (error == cudaSuccess) error = clear_attention_state(created);
    if (error != cudaSuccess) {
        free_attention(created);
        delete created;
        return fail(context, "Qwen attention create", error);
    }
    *layer = created;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_qwen35_attention_destroy(fortai_cuda_qwen35_attention *layer) {
    if (!layer) return FORTAI_CUDA_OK;
    if (layer->context) {
        cudaSetDevice(layer->context->device);
        free_attention(layer);
    }
    delete layer;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_qwen35_attention_reset(fortai_cuda_qwen35_attention *layer) {
    if (!layer || !layer->context) return FORTAI_CUDA_INVALID;
    cudaSetDevice(layer->context->device);
    const cudaError_t error = clear_attention_state(layer);
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(layer->context, "Qwen attention reset", error);
}

// The position used by the kernels is the context's device-side position word
// (fortai_cuda_q8_context_set_position), as in the reference; `position` only bounds it.
namespace {

int attention_run(fortai_cuda_qwen35_attention *layer, const void *device_activation,
    size_t activation_elements, int position, void *device_output, size_t output_elements,
    const Glue &glue) {
    if (!layer || !layer->context || !device_activation || !device_output || position < 0 ||
        position >= layer->max_context) return FORTAI_CUDA_INVALID;
    fortai_cuda_q8_context *c = layer->context;
    if (activation_elements != static_cast<size_t>(layer->q->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(layer->out->rows) ||
        layer->q->blocks != layer->k->blocks || layer->q->blocks != layer->v->blocks)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(c->device);
    float *query = layer->projections;
    float *key = query + static_cast<size_t>(layer->heads) * 2 * layer->head_size;
    float *value = key + static_cast<size_t>(layer->kv_heads) * layer->head_size;
    GemvParams p = single_params(c, layer->q, device_activation, query);
    p.weights[1] = layer->k->data;
    p.outputs[1] = key;
    p.rows[1] = layer->k->rows;
    p.weights[2] = layer->v->data;
    p.outputs[2] = value;
    p.rows[2] = layer->v->rows;
    p.segments = 3;
    p.total_rows = layer->q->rows + layer->k->rows + layer->v->rows;
    p.norm_weights = glue.norm_weights;
    p.norm_epsilon = glue.epsilon;
    cudaError_t error = launch_gemv(c, p, kActF32, kEpiPlain);
    if (error == cudaSuccess) {
        error = launch_overlapped(c, attention_prepare_kernel, layer->heads + layer->kv_heads, 256,
            0, query, key, value, layer->q_norm, layer->k_norm, layer->key_cache,
            layer->value_cache, layer->heads, layer->kv_heads, layer->head_size, layer->value_size,
            c->position, layer->rope_dimension, layer->rope_base, layer->epsilon,
            layer->max_context, c->status_device);
        // scores of every position, then one row of partial value sums per warp
        const size_t shared = (static_cast<size_t>(layer->max_context + 3) / 4 * 4 +
            8 * static_cast<size_t>(layer->value_size)) * sizeof(float);
        if (error == cudaSuccess && shared > 48 * 1024)
            error = cudaFuncSetAttribute(attention_apply_kernel,
                cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
        if (error == cudaSuccess)
            error = launch_overlapped(c, attention_apply_kernel, layer->heads, 256, shared, query,
                layer->key_cache, layer->value_cache, layer->attention, layer->heads,
                layer->kv_heads, layer->head_size, layer->value_size,
                (layer->max_context + 3) / 4 * 4, c->position, layer->max_context,
                c->status_device);
    }
    if (error == cudaSuccess) {
        GemvParams o = single_params(c, layer->out, layer->attention,
            static_cast<float *>(device_output));
        o.residual = glue.residual;
        error = launch_gemv(c, o, kActF32, kEpiPlain);
    }
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(c, "Qwen attention device run", error);
}

}  // namespace

extern "C" int fortai_cuda_qwen35_attention_run_device(fortai_cuda_qwen35_attention *layer,
    const void *device_activation, size_t activation_elements, int position,
    void *device_output, size_t output_elements) {
    return attention_run(layer, device_activation, activation_elements, position, device_output,
        output_elements, Glue());
}

extern "C" const char *fortai_cuda_q8_last_error(const fortai_cuda_q8_context *context) {
    return context ? context->error : "invalid CUDA Q8 context";
}

// ===========================================================================
// Part 2: extensions
// ===========================================================================
extern "C" void *fortai_cuda_q8_context_stream(const fortai_cuda_q8_context *context) {
    return context ? static_cast<void *>(context->stream) : nullptr;
}

extern "C" uint64_t fortai_cuda_q8_context_launch_count(const fortai_cuda_q8_context *context) {
    return context ? context->launches : 0;
}

extern "C" int fortai_cuda_q8_context_synchronize(fortai_cuda_q8_context *context) {
    if (!context) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    return finish(context, "synchronize", cudaStreamSynchronize(context->stream));
}

extern "C" int fortai_cuda_q8_context_set_option(fortai_cuda_q8_context *context,
    const char *name, int value) {
    if (!context || !name || value < 0) return FORTAI_CUDA_INVALID;
    if (!std::strcmp(name, "gemv_variant") && value <= 1) context->gemv_variant = value;
    else if (!std::strcmp(name, "host_flush_rows") && value >= 1 && value <= 32 &&
             (value & (value - 1)) == 0)
        context->host_flush_rows = static_cast<int>(value);
    else if (!std::strcmp(name, "peer_publish_per_cta") && value <= 1)
        context->peer_publish_per_cta = value;
    else if (!std::strcmp(name, "peer_flush_rows") && value >= 1 && value <= 32 &&
             (value & (value - 1)) == 0)
        context->peer_flush_rows = static_cast<int>(value);
    else if (!std::strcmp(name, "gemv_ctas_per_sm") && value <= 32)
        context->gemv_ctas_per_sm = value;
    else if (!std::strcmp(name, "gemv_rows_per_warp") && value <= 2)
        context->gemv_rows_per_warp = value;
    else if (!std::strcmp(name, "gemv_balance") && value <= 1) context->gemv_balance = value;
    else if (!std::strcmp(name, "planar_min_width")) context->planar_min_width = value;
    else if (!std::strcmp(name, "gemv_split") && (value <= 1 || value == 4 || value == 8))
        context->gemv_split = value;
    else if (!std::strcmp(name, "gemv_depth") && value >= 1 && value <= 2)
        context->gemv_depth = value;
    else if (!std::strcmp(name, "mmq_min_tokens")) context->mmq_min_tokens = value;
    else if (!std::strcmp(name, "peer_wait_clocks_millions"))
        context->peer_wait_clocks_millions = value > 0 ? value : 2000;
    else if (!std::strcmp(name, "prefill_kind")) context->prefill_kind = value;
    else if (!std::strcmp(name, "host_spin_wait")) context->host_spin_wait = value;
    else if (!std::strcmp(name, "peer_overlap")) context->peer_overlap = value;
    else if (!std::strcmp(name, "fewtok_splits") && value >= 0) context->fewtok_splits = value;
    else if (!std::strcmp(name, "fewtok_threads") && value >= 0 && value <= 512 &&
             value % 32 == 0) context->fewtok_threads = value;
    else if (!std::strcmp(name, "fewtok_step") &&
             (value == 0 || value == 64 || value == 256 || value == 512))
        context->fewtok_step = value;
    else if (!std::strcmp(name, "fewtok_stages") && (value == 0 || value == 2 || value == 3))
        context->fewtok_stages = value;
    else if (!std::strcmp(name, "ffn_quantize_in_gemv") && value >= 0)
        context->ffn_quantize_in_gemv = value;
    else if (!std::strcmp(name, "gdn_conv_in_gemv")) context->gdn_conv_in_gemv = value != 0;
    else if (!std::strcmp(name, "gemv_even_rounds")) context->gemv_even_rounds = value != 0;
    else if (!std::strcmp(name, "gemv_early_trigger") && value <= 3)
        context->gemv_early_trigger = value;
    else if (!std::strcmp(name, "host_direct_output")) context->host_direct_output = value != 0;
    else if (!std::strcmp(name, "gemv_overlap")) context->gemv_overlap = value != 0;
    else if (!std::strcmp(name, "fewtok_overlap")) context->fewtok_overlap = value != 0;
    else if (!std::strcmp(name, "fewtok_off")) context->fewtok_off = value != 0;
    else return FORTAI_CUDA_INVALID;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_quantize_device(fortai_cuda_q8_context *context,
    const void *device_input, size_t elements, void *device_output, size_t output_bytes) {
    if (!context || !device_input || !device_output || elements == 0 ||
        elements % kBlockElems != 0 || output_bytes < elements / kBlockElems * kBlockBytes)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = launch_quantize(context, static_cast<const float *>(device_input),
        static_cast<uint8_t *>(device_output), elements / kBlockElems);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device Q8 quantize", error);
}

extern "C" int fortai_cuda_q8_block_dots_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !device_output ||
        output_elements < static_cast<size_t>(weights->rows) * weights->blocks)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const GemvParams p = single_params(context, weights, device_activation,
        static_cast<float *>(device_output));
    const cudaError_t error = launch_gemv(context, p, kActQ8, kEpiBlockDots);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "block dots", error);
}

extern "C" int fortai_cuda_q8_matvec_host_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!owned(context, weights) || !host_activation || !host_output || !elapsed_ms ||
        activation_elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        output_bytes < static_cast<size_t>(weights->rows) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const size_t in_bytes = activation_elements * sizeof(float);
    const size_t out_bytes = static_cast<size_t>(weights->rows) * sizeof(float);
    // the fp32 activation is parked in the activation scratch (4 bytes per element)
    cudaError_t error = ensure_scratch(context, in_bytes, out_bytes);
    // Page-locked, device-mapped output (cudaHostAlloc / cudaHostRegister memory): the GEMV
    // stores its results there itself, a CTA's block of rows at a time in full lines, while
    // it is still streaming weights; the separate device-to-host copy (607 KB and a second
    // trip through the copy engine for the lm_head) disappears.  Pageable memory keeps the
    // copy.
    float *mapped_output = nullptr;
    if (error == cudaSuccess && context->host_direct_output && weights->width % 512 == 0)
        mapped_output = mapped_host_pointer(host_output);
    // Both buffers page-locked and mapped: the call needs neither the copy engine nor events.
    // A one-CTA kernel pulls the activation over PCIe into scratch (the GEMV, launched as its
    // programmatic dependent, streams its first weights meanwhile); the GEMV stores the
    // results into the output itself; its last CTA then writes this call's sequence number
    // into a mapped word of the context, on which the host spins.  That takes the two event
    // records, the DMA set-up and the driver's blocking wait out of a ~60 us call.  elapsed_ms
    // is then host time from here to completion (it still covers both transfers).
    const float *mapped_input = mapped_output && context->host_spin_wait && in_bytes % 16 == 0
        ? mapped_host_pointer(host_activation) : nullptr;
    if (error == cudaSuccess && mapped_input) {
        const auto begin = std::chrono::steady_clock::now();
        // one 16-byte request per thread, all in flight at once: the transfer then costs one
        // round trip over the link (three in a row took about 8 us for 10 KB)
        const int pieces = static_cast<int>(in_bytes / 16);
        const int fetch_threads = std::min(1024, (pieces + 31) / 32 * 32);
        q8_fetch_kernel<<<(pieces + fetch_threads - 1) / fetch_threads, fetch_threads, 0,
            context->stream>>>(reinterpret_cast<const float4 *>(mapped_input),
            reinterpret_cast<float4 *>(context->scratch_activation), pieces);
        ++context->launches;
        error = cudaGetLastError();
        unsigned sequence = 0;
        if (error == cudaSuccess) {
            GemvParams p = single_params(context, weights, context->scratch_activation,
                context->scratch_output);
            p.peers = 1;
            p.peer_outputs[0] = mapped_output;
            p.peer_flush = context->host_flush_rows;
            p.first_row = 0;
            // the fused all-gather tail with one rank whose flag word is host memory
            p.peer_flags[0] = context->done_device;
            p.my_flags = context->done_device;
            p.cta_counter = context->cta_counter;
            p.my_rank = 0;
            sequence = p.sequence = ++context->host_sequence;
            p.exchange = kExchangeLastCta;   // a host word: plain stores only
            p.flag_wait_clocks = static_cast<long long>(context->peer_wait_clocks_millions) *
                1000000LL;
            p.overlap_ok = 1;
            error = launch_gemv(context, p, kActF32, kEpiPeers);
        }
        if (error == cudaSuccess) {
            volatile unsigned *done = context->done_host;
            bool seen = false;
            // about two seconds of polling, then the driver's own wait
            for (long long spin = 0; spin < (1ll << 31); ++spin) {
                if (static_cast<int>(*done - sequence) >= 0) {
                    seen = true;
                    break;
                }
                if ((spin & 0xfffff) == 0xfffff &&
                    std::chrono::steady_clock::now() - begin > std::chrono::seconds(2)) break;
            }
            if (!seen) error = cudaStreamSynchronize(context->stream);
        }
        *elapsed_ms = std::chrono::duration<float, std::milli>(
            std::chrono::steady_clock::now() - begin).count();
        return finish(context, "host F32 matvec", error);
    }
    if (error == cudaSuccess) error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(context->scratch_activation, host_activation, in_bytes,
            cudaMemcpyHostToDevice, context->stream);
    if (error == cudaSuccess) {
        GemvParams p = single_params(context, weights, context->scratch_activation,
            context->scratch_output);
        if (mapped_output) {
            p.peers = 1;
            p.peer_outputs[0] = mapped_output;
            p.peer_flush = context->host_flush_rows;
            p.first_row = 0;
            error = launch_gemv(context, p, kActF32, kEpiPeers);
        } else {
            error = launch_gemv(context, p, kActF32, kEpiPlain);
        }
    }
    if (error == cudaSuccess && !mapped_output)
        error = cudaMemcpyAsync(host_output, context->scratch_output, out_bytes,
            cudaMemcpyDeviceToHost, context->stream);
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    if (error == cudaSuccess)
        error = cudaEventElapsedTime(elapsed_ms, context->start, context->stop);
    return finish(context, "host F32 matvec", error);
}

extern "C" int fortai_cuda_q8_matvec_device_f32_peers(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_outputs, int peer_count, size_t first_row,
    size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !peer_outputs || peer_count <= 0 ||
        peer_count > kMaxPeers ||
        activation_elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        first_row + static_cast<size_t>(weights->rows) > output_elements ||
        output_elements > static_cast<size_t>(INT32_MAX)) return FORTAI_CUDA_INVALID;
    for (int i = 0; i < peer_count; ++i)
        if (!peer_outputs[i]) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    GemvParams p = single_params(context, weights, device_activation, nullptr);
    for (int i = 0; i < peer_count; ++i) p.peer_outputs[i] = static_cast<float *>(peer_outputs[i]);
    p.peers = peer_count;
    p.peer_flush = context->peer_flush_rows;
    p.first_row = static_cast<int>(first_row);
    // the kernel stores nothing anywhere before its own dependency wait, which ends only when
    // everything earlier in this stream has completed: it may start under its predecessor
    p.overlap_ok = context->peer_overlap;
    const cudaError_t error = launch_gemv(context, p, kActF32, kEpiPeers);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "peer-output matvec", error);
}

extern "C" int fortai_cuda_q8_matvec_device_f32_allgather(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_outputs, void *const *peer_flags,
    int peer_count, int my_rank, size_t first_row, size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !peer_outputs || !peer_flags ||
        peer_count <= 0 || peer_count > kMaxPeers || my_rank < 0 || my_rank >= peer_count ||
        activation_elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        first_row + static_cast<size_t>(weights->rows) > output_elements ||
        output_elements > static_cast<size_t>(INT32_MAX)) return FORTAI_CUDA_INVALID;
    for (int i = 0; i < peer_count; ++i)
        if (!peer_outputs[i] || !peer_flags[i]) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    // With the last-CTA protocol the call's number is a kernel argument taken from a host
    // counter: a captured launch would replay the same number, and from the second replay on
    // the tail would find the peers' flags "already raised" and return without waiting.
    // Refuse capture there.  (The per-CTA protocol takes the number from the flag words.)
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (!context->peer_publish_per_cta &&
        cudaStreamIsCapturing(context->stream, &capture) == cudaSuccess &&
        capture != cudaStreamCaptureStatusNone) {
        fail(context, "all-gather matvec with peer_publish_per_cta = 0 cannot be captured into "
                      "a CUDA graph (its flag sequence number is a launch argument)");
        return FORTAI_CUDA_INVALID;
    }
    GemvParams p = single_params(context, weights, device_activation, nullptr);
    for (int i = 0; i < peer_count; ++i) {
        p.peer_outputs[i] = static_cast<float *>(peer_outputs[i]);
        p.peer_flags[i] = static_cast<unsigned *>(peer_flags[i]);
    }
    p.peers = peer_count;
    p.peer_flush = context->peer_flush_rows;
    p.first_row = static_cast<int>(first_row);
    p.my_flags = static_cast<unsigned *>(peer_flags[my_rank]);
    p.cta_counter = context->cta_counter;
    p.my_rank = my_rank;
    p.sequence = ++context->allgather_sequence;
    p.exchange = context->peer_publish_per_cta ? kExchangeCounters : kExchangeLastCta;
    p.flag_wait_clocks = static_cast<long long>(context->peer_wait_clocks_millions) * 1000000LL;
    // A following call of this kind may be launched while this one still waits for its peers'
    // flags: the kernel touches neither the peers' vectors nor the shared CTA counter before
    // its own dependency wait, which ends only when this launch has completed, so what
    // overlaps is the successor's launch latency and its first weight requests (option
    // "peer_overlap", default on).
    p.overlap_ok = context->peer_overlap;
    const cudaError_t error = launch_gemv(context, p, kActF32, kEpiPeers);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "all-gather matvec", error);
}

extern "C" int fortai_cuda_q8_matvec_device_f32_allgather_ll(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_pairs, int peer_count, int my_rank,
    size_t first_row, void *device_output, size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !peer_pairs || !device_output ||
        peer_count <= 0 || peer_count > kMaxPeers || my_rank < 0 || my_rank >= peer_count ||
        activation_elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        first_row + static_cast<size_t>(weights->rows) > output_elements ||
        output_elements > static_cast<size_t>(INT32_MAX)) return FORTAI_CUDA_INVALID;
    for (int i = 0; i < peer_count; ++i)
        if (!peer_pairs[i] || reinterpret_cast<uintptr_t>(peer_pairs[i]) % 8 != 0)
            return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    // the call's number and the half of the pair arrays it uses are launch arguments taken
    // from host counters: a captured launch would replay them
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(context->stream, &capture) == cudaSuccess &&
        capture != cudaStreamCaptureStatusNone) {
        fail(context, "all-gather matvec (pairs) cannot be captured into a CUDA graph "
                      "(its call number is a launch argument)");
        return FORTAI_CUDA_INVALID;
    }
    GemvParams p = single_params(context, weights, device_activation, nullptr);
    // two halves used alternately: a rank that runs ahead writes call n+1's pairs while a
    // peer may still collect call n's; it cannot reach call n+2 before that peer has sent its
    // own pairs of call n+1, which it does after collecting call n
    const size_t half = static_cast<size_t>(context->ll_calls++ & 1u) * output_elements;
    for (int i = 0; i < peer_count; ++i)
        p.peer_outputs[i] = reinterpret_cast<float *>(static_cast<uint2 *>(peer_pairs[i]) + half);
    p.peers = peer_count;
    p.peer_flush = context->peer_flush_rows;
    p.first_row = static_cast<int>(first_row);
    p.my_rank = my_rank;
    if (++context->ll_sequence == 0) ++context->ll_sequence;   // zero is "nothing has arrived"
    p.ll_sequence = context->ll_sequence;
    p.ll_output = static_cast<float *>(device_output);
    p.ll_total = static_cast<int>(output_elements);
    p.flag_wait_clocks = static_cast<long long>(context->peer_wait_clocks_millions) * 1000000LL;
    p.overlap_ok = context->peer_overlap;
    const cudaError_t error = launch_gemv(context, p, kActF32, kEpiPeers);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "all-gather matvec (pairs)", error);
}

// ---------------------------------------------------------------------------
// batched (prefill) product
// ---------------------------------------------------------------------------
namespace {

// One GEMV launch per token: the fallback for widths the batched kernels do not take.
cudaError_t enqueue_matmul_streaming(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w,
    const void *activation, int act, int tokens, float *output, int32_t *block_dots) {
    cudaError_t error = cudaSuccess;
    const size_t act_stride = act == kActF32 ? static_cast<size_t>(w->width) * sizeof(float)
                                             : static_cast<size_t>(w->blocks) * kBlockBytes;
    for (int t = 0; t < tokens && error == cudaSuccess; ++t) {
        float *out = block_dots
            ? reinterpret_cast<float *>(block_dots + static_cast<size_t>(t) * w->rows * w->blocks)
            : output + static_cast<size_t>(t) * w->rows;
        const GemvParams p = single_params(c, w,
            static_cast<const uint8_t *>(activation) + t * act_stride, out);
        error = launch_gemv(c, p, act, block_dots ? kEpiBlockDots : kEpiPlain);
    }
    return error;
}

template <int NT, int CB, int ST, bool DOTS>
cudaError_t launch_fewtok_instance(fortai_cuda_q8_context *c, const FewTokParams &p,
    const FewTokPlan &plan) {
    cudaError_t error = cudaSuccess;
    if (plan.smem > 48 * 1024)
        error = cudaFuncSetAttribute(q8_fewtok_kernel<NT, CB, ST, DOTS>,
            cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(plan.smem));
    int per_sm = 0;
    if (error == cudaSuccess)
        error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm,
            q8_fewtok_kernel<NT, CB, ST, DOTS>, plan.threads, plan.smem);
    if (error != cudaSuccess) return error;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const int grid = fewtok_grid(plan, p.rows, p.width, c->sm_count, per_sm);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(plan.threads);
    config.dynamicSmemBytes = plan.smem;
    config.stream = c->stream;
    cudaLaunchAttribute overlap = {};
    overlap.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    overlap.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &overlap;
    config.numAttrs = c->fewtok_overlap ? 1 : 0;
    error = cudaLaunchKernelEx(&config, q8_fewtok_kernel<NT, CB, ST, DOTS>, p);
    ++c->launches;
    return error != cudaSuccess ? error : cudaGetLastError();
}

template <int NT, int CB>
cudaError_t launch_fewtok_stages(fortai_cuda_q8_context *c, const FewTokParams &p,
    const FewTokPlan &plan, bool dots) {
    if (dots) return launch_fewtok_instance<NT, CB, 2, true>(c, p, plan);
    return plan.stages == 3 ? launch_fewtok_instance<NT, CB, 3, false>(c, p, plan)
                            : launch_fewtok_instance<NT, CB, 2, false>(c, p, plan);
}

template <int NT>
cudaError_t launch_fewtok(fortai_cuda_q8_context *c, const FewTokParams &p, const FewTokPlan &plan,
    bool dots) {
    switch (plan.step_bytes) {
    case 512: return launch_fewtok_stages<NT, 512>(c, p, plan, dots);
    case 256: return launch_fewtok_stages<NT, 256>(c, p, plan, dots);
    default: return launch_fewtok_stages<NT, 64>(c, p, plan, dots);
    }
}

// 2..64 tokens: activation image, zeroed output, one pass over the weights.
cudaError_t enqueue_fewtok(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w,
    const void *activation, int act, int tokens, float *output, int32_t *block_dots) {
    const int padded = fewtok_padded_tokens(tokens);
    FewTokPlan plan;
    if (!fewtok_plan(w->rows, w->width, padded, c->sm_count, c->fewtok_splits,
            c->fewtok_threads, c->fewtok_step, block_dots ? 2 : c->fewtok_stages, &plan))
        return cudaErrorNotSupported;
    cudaError_t error = mmq_reserve(reinterpret_cast<void **>(&c->scratch_aux),
        &c->scratch_aux_bytes, w->rows, w->width, tokens);
    if (error != cudaSuccess) return error;
    int8_t *quants = reinterpret_cast<int8_t *>(c->scratch_aux);
    float *scales = reinterpret_cast<float *>(quants + static_cast<size_t>(padded) * w->width);
    const long long prep_warps = static_cast<long long>(padded) * w->blocks;
    const int prep_grid = static_cast<int>(std::max<long long>(1,
        std::min<long long>((prep_warps + 7) / 8, static_cast<long long>(c->sm_count) * 16)));
    // the output (cudaMalloc'ed or a 16-byte aligned slice) is zeroed 16 bytes at a time by
    // the prepare kernel; an unaligned or odd-sized one by a memset node
    const size_t out_bytes = output ? static_cast<size_t>(tokens) * w->rows * sizeof(float) : 0;
    const bool zero_in_kernel = output && reinterpret_cast<uintptr_t>(output) % 16 == 0 &&
        out_bytes % 16 == 0;
    float4 *zero = zero_in_kernel ? reinterpret_cast<float4 *>(output) : nullptr;
    const long long zero_count = zero_in_kernel ? static_cast<long long>(out_bytes / 16) : 0;
    if (output && !zero_in_kernel) {
        error = cudaMemsetAsync(output, 0, out_bytes, c->stream);
        if (error != cudaSuccess) return error;
    }
    if (act == kActF32)
        fewtok_prepare_kernel<1><<<prep_grid, 256, 0, c->stream>>>(activation, tokens, padded,
            w->width, quants, scales, zero, zero_count);
    else
        fewtok_prepare_kernel<0><<<prep_grid, 256, 0, c->stream>>>(activation, tokens, padded,
            w->width, quants, scales, zero, zero_count);
    ++c->launches;
    error = cudaGetLastError();
    if (error != cudaSuccess) return error;
    FewTokParams p = {};
    p.weights = w->data;
    p.rows = w->rows;
    p.width = w->width;
    p.blocks = w->blocks;
    p.row_stride = static_cast<int>(w->row_stride);
    p.act_quants = quants;
    p.act_scales = scales;
    p.tokens = tokens;
    p.padded_tokens = padded;
    p.splits = plan.splits;
    p.blocks_per_split = plan.blocks_per_split;
    p.output = output;
    p.block_dots = block_dots;
    const bool dots = block_dots != nullptr;
    if (padded == 8) return launch_fewtok<1>(c, p, plan, dots);
    if (padded == 16) return launch_fewtok<2>(c, p, plan, dots);
    if (padded == 32) return launch_fewtok<4>(c, p, plan, dots);
    return launch_fewtok<8>(c, p, plan, dots);
}

// Batched product, any token count: the tcgen05 kernel above 64 tokens, the few-token
// kernel below that (in groups of up to 64 where the tcgen05 kernel does not take the
// width), one GEMV per token as the last resort.  Exactly one of output / block_dots.
cudaError_t enqueue_matmul(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w,
    const void *activation, int act, int tokens, float *output, int32_t *block_dots) {
    // the exact int32 block dots come from the kind::i8 kernel (or the few-token kernel)
    if (c->prefill_kind == 0 && !block_dots &&
        pf_supported(w->rows, w->width, tokens, c->mmq_min_tokens))
        return pf_enqueue(c->stream, c->sm_count, c->status_device,
            &const_cast<fortai_cuda_q8_weights *>(w)->prefill, w->data, w->rows, w->width,
            w->row_stride, activation, act, tokens, output,
            reinterpret_cast<void **>(&c->scratch_aux), &c->scratch_aux_bytes, &c->launches);
    if (mmq_supported(w->rows, w->width, tokens, c->mmq_min_tokens))
        return mmq_enqueue(c->stream, c->sm_count, c->status_device,
            &const_cast<fortai_cuda_q8_weights *>(w)->mmq, w->data, w->rows, w->width,
            w->row_stride, activation, act, tokens, output, block_dots,
            reinterpret_cast<void **>(&c->scratch_aux), &c->scratch_aux_bytes, &c->launches);
    if (c->fewtok_off || !fewtok_supported(w->rows, w->width, tokens))
        return enqueue_matmul_streaming(c, w, activation, act, tokens, output, block_dots);
    const size_t act_stride = act == kActF32 ? static_cast<size_t>(w->width) * sizeof(float)
                                             : static_cast<size_t>(w->blocks) * kBlockBytes;
    cudaError_t error = cudaSuccess;
    for (int first = 0; first < tokens && error == cudaSuccess; first += kFewTokMaxTokens) {
        const int count = std::min(kFewTokMaxTokens, tokens - first);
        const void *act_at = static_cast<const uint8_t *>(activation) + first * act_stride;
        float *out_at = output ? output + static_cast<size_t>(first) * w->rows : nullptr;
        int32_t *dots_at = block_dots
            ? block_dots + static_cast<size_t>(first) * w->rows * w->blocks : nullptr;
        if (count >= 2)
            error = enqueue_fewtok(c, w, act_at, act, count, out_at, dots_at);
        else
            error = enqueue_matmul_streaming(c, w, act_at, act, count, out_at, dots_at);
    }
    return error;
}

// scratch the batched kernels need, grown outside a timed region
cudaError_t reserve_matmul(fortai_cuda_q8_context *c, const fortai_cuda_q8_weights *w, int tokens) {
    if (c->prefill_kind == 0 && pf_supported(w->rows, w->width, tokens, c->mmq_min_tokens))
        return pf_reserve(reinterpret_cast<void **>(&c->scratch_aux), &c->scratch_aux_bytes,
            w->width, tokens);
    return mmq_reserve(reinterpret_cast<void **>(&c->scratch_aux), &c->scratch_aux_bytes, w->rows,
        w->width, tokens);
}

}  // namespace

extern "C" int fortai_cuda_q8_matmul_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !device_output || tokens <= 0 ||
        output_elements < static_cast<size_t>(tokens) * weights->rows)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = enqueue_matmul(context, weights, device_activation, kActF32, tokens,
        static_cast<float *>(device_output), nullptr);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "device F32 matmul", error);
}

extern "C" int fortai_cuda_q8_matmul_resident(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, float *kernel_ms) {
    if (!owned(context, weights) || !device_activation || !device_output || tokens <= 0 ||
        !kernel_ms) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    cudaError_t error = reserve_matmul(context, weights, tokens);   // before the timed region
    if (error == cudaSuccess) error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess)
        error = enqueue_matmul(context, weights, device_activation, kActQ8, tokens,
            static_cast<float *>(device_output), nullptr);
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    if (error == cudaSuccess)
        error = cudaEventElapsedTime(kernel_ms, context->start, context->stop);
    return finish(context, "resident matmul", error);
}

extern "C" int fortai_cuda_q8_matmul_host_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const float *host_activation, int tokens,
    float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!owned(context, weights) || !host_activation || !host_output || tokens <= 0 ||
        !elapsed_ms ||
        output_bytes < static_cast<size_t>(tokens) * weights->rows * sizeof(float))
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const size_t in_bytes = static_cast<size_t>(tokens) * weights->width * sizeof(float);
    const size_t out_bytes = static_cast<size_t>(tokens) * weights->rows * sizeof(float);
    cudaError_t error = ensure_scratch(context, in_bytes, out_bytes);
    if (error == cudaSuccess) error = reserve_matmul(context, weights, tokens);
    if (error == cudaSuccess) error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(context->scratch_activation, host_activation, in_bytes,
            cudaMemcpyHostToDevice, context->stream);
    if (error == cudaSuccess)
        error = enqueue_matmul(context, weights, context->scratch_activation, kActF32, tokens,
            context->scratch_output, nullptr);
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(host_output, context->scratch_output, out_bytes,
            cudaMemcpyDeviceToHost, context->stream);
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    if (error == cudaSuccess)
        error = cudaEventElapsedTime(elapsed_ms, context->start, context->stop);
    return finish(context, "host F32 matmul", error);
}

extern "C" int fortai_cuda_q8_matmul_block_dots_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements) {
    if (!owned(context, weights) || !device_activation || !device_output || tokens <= 0 ||
        output_elements < static_cast<size_t>(tokens) * weights->rows * weights->blocks)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const cudaError_t error = enqueue_matmul(context, weights, device_activation, kActQ8, tokens,
        nullptr, static_cast<int32_t *>(device_output));
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "matmul block dots", error);
}

// Measured tensor-core peak: `iterations` commits of four 128 x 256 MMAs on every SM, timed
// with the context's events.  kind 0 = kind::i8, 1 = kind::f16.  Blocks.
extern "C" int fortai_cuda_tensor_peak(fortai_cuda_q8_context *context, int kind, int iterations,
    float *tera_ops_per_second, float *elapsed_ms) {
    if (!context || (kind != 0 && kind != 1) || iterations < 2 || iterations > (1 << 24) ||
        !tera_ops_per_second) return FORTAI_CUDA_INVALID;
    *tera_ops_per_second = 0.0f;
    if (elapsed_ms) *elapsed_ms = 0.0f;
    cudaSetDevice(context->device);
    // once untimed: the first launch pays for module loading and the attribute call
    cudaError_t error = tensor_peak_launch(context->stream, kind, 64, context->sm_count,
        context->status_device);
    if (error == cudaSuccess) error = cudaEventRecord(context->start, context->stream);
    if (error == cudaSuccess)
        error = tensor_peak_launch(context->stream, kind, iterations, context->sm_count,
            context->status_device);
    context->launches += 2;
    if (error == cudaSuccess) error = cudaEventRecord(context->stop, context->stream);
    if (error == cudaSuccess) error = cudaEventSynchronize(context->stop);
    float ms = 0.0f;
    if (error == cudaSuccess) error = cudaEventElapsedTime(&ms, context->start, context->stop);
    if (error == cudaSuccess && ms > 0.0f) {
        *tera_ops_per_second = static_cast<float>(
            tensor_peak_ops(kind, iterations, context->sm_count) / (ms * 1.0e-3) / 1.0e12);
        if (elapsed_ms) *elapsed_ms = ms;
    }
    return finish(context, "tensor peak probe", error);
}

// h[i] = silu(gate[i]) * up[i], in place over gate
__global__ void __launch_bounds__(256)
silu_product_kernel(float *__restrict__ gate, const float *__restrict__ up, long long count) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        gate[i] = silu_mul(gate[i], up[i]);
}

extern "C" int fortai_cuda_q8_ffn_batch_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements) {
    if (!owned(context, gate_weights) || !owned(context, up_weights) ||
        !owned(context, down_weights) || !device_activation || !device_output || tokens <= 0)
        return FORTAI_CUDA_INVALID;
    // the shape rules of the single-token FFN
    if (gate_weights->rows != up_weights->rows || gate_weights->blocks != up_weights->blocks ||
        gate_weights->rows != down_weights->blocks * kBlockElems ||
        output_elements < static_cast<size_t>(tokens) * down_weights->rows)
        return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const size_t inner = static_cast<size_t>(tokens) * gate_weights->rows;
    cudaError_t error = ensure_scratch(context, 0, 2 * inner * sizeof(float));
    float *gate = context->scratch_output, *up = gate + inner;
    if (error == cudaSuccess)
        error = enqueue_matmul(context, gate_weights, device_activation, kActF32, tokens, gate,
            nullptr);
    if (error == cudaSuccess)
        error = enqueue_matmul(context, up_weights, device_activation, kActF32, tokens, up, nullptr);
    if (error == cudaSuccess) {
        const int grid = static_cast<int>(std::min<size_t>((inner + 255) / 256,
            static_cast<size_t>(context->sm_count) * 8));
        silu_product_kernel<<<grid, 256, 0, context->stream>>>(gate, up,
            static_cast<long long>(inner));
        ++context->launches;
        error = cudaGetLastError();
    }
    if (error == cudaSuccess)
        error = enqueue_matmul(context, down_weights, gate, kActF32, tokens,
            static_cast<float *>(device_output), nullptr);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "batched FFN", error);
}

// ---------------------------------------------------------------------------
// Residual-stream steps: the caller's copy / RMS norm / add folded into the GEMVs
// ---------------------------------------------------------------------------
// The reference's caller surrounds every layer object and FFN with copy -> rms_norm ->
// ... -> add (src/models/qwen35/fortai_qwen35_cpu.f90:713-747): four extra kernels and
// two copies per layer half on a step that is latency-bound.  These entry points take
// the residual stream x itself: the first GEMV normalises it in its prologue, the last
// one adds it back in its epilogue, in place.
namespace {

bool glue_arguments_ok(const void *x, const void *norm_weights, float epsilon) {
    return x && norm_weights && epsilon > 0.0f &&
        reinterpret_cast<uintptr_t>(norm_weights) % 16 == 0;
}

}  // namespace

extern "C" int fortai_cuda_qwen35_recurrent_step_device(fortai_cuda_qwen35_recurrent *layer,
    void *device_x, size_t elements, const void *device_norm_weights, float epsilon) {
    if (!layer || !layer->context || !glue_arguments_ok(device_x, device_norm_weights, epsilon))
        return FORTAI_CUDA_INVALID;
    if (elements != static_cast<size_t>(layer->qkv->blocks) * kBlockElems ||
        elements != static_cast<size_t>(layer->out->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(layer->context->device);
    Glue glue;
    glue.norm_weights = static_cast<const float *>(device_norm_weights);
    glue.epsilon = epsilon;
    glue.residual = static_cast<const float *>(device_x);
    const cudaError_t error = enqueue_recurrent(layer, device_x, kActF32,
        static_cast<float *>(device_x), glue);
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(layer->context, "Qwen recurrent step", error);
}

extern "C" int fortai_cuda_qwen35_attention_step_device(fortai_cuda_qwen35_attention *layer,
    void *device_x, size_t elements, int position, const void *device_norm_weights,
    float epsilon) {
    if (!layer || !layer->context || !glue_arguments_ok(device_x, device_norm_weights, epsilon))
        return FORTAI_CUDA_INVALID;
    if (elements != static_cast<size_t>(layer->out->rows)) return FORTAI_CUDA_INVALID;
    Glue glue;
    glue.norm_weights = static_cast<const float *>(device_norm_weights);
    glue.epsilon = epsilon;
    glue.residual = static_cast<const float *>(device_x);
    return attention_run(layer, device_x, elements, position, device_x, elements, glue);
}

extern "C" int fortai_cuda_q8_ffn_step_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, void *device_x, size_t elements,
    const void *device_norm_weights, float epsilon) {
    if (!owned(context, gate_weights) || !owned(context, up_weights) ||
        !owned(context, down_weights) || !glue_arguments_ok(device_x, device_norm_weights, epsilon))
        return FORTAI_CUDA_INVALID;
    if (gate_weights->rows != up_weights->rows || gate_weights->blocks != up_weights->blocks ||
        gate_weights->rows != down_weights->blocks * kBlockElems ||
        elements != static_cast<size_t>(gate_weights->blocks) * kBlockElems ||
        elements != static_cast<size_t>(down_weights->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    const size_t inner = static_cast<size_t>(gate_weights->rows);
    cudaError_t error = ensure_scratch(context, inner / kBlockElems * kBlockBytes,
        inner * sizeof(float));
    Glue glue;
    glue.norm_weights = static_cast<const float *>(device_norm_weights);
    glue.epsilon = epsilon;
    glue.residual = static_cast<const float *>(device_x);
    if (error == cudaSuccess)
        error = enqueue_ffn(context, gate_weights, up_weights, down_weights, device_x, kActF32,
            static_cast<float *>(device_x), glue);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "FFN step", error);
}

extern "C" int fortai_cuda_q8_matvec_norm_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_x, size_t elements,
    const void *device_norm_weights, float epsilon, void *device_output,
    size_t output_elements) {
    if (!owned(context, weights) || !device_output ||
        !glue_arguments_ok(device_x, device_norm_weights, epsilon)) return FORTAI_CUDA_INVALID;
    if (elements != static_cast<size_t>(weights->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(weights->rows)) return FORTAI_CUDA_INVALID;
    cudaSetDevice(context->device);
    GemvParams p = single_params(context, weights, device_x, static_cast<float *>(device_output));
    p.norm_weights = static_cast<const float *>(device_norm_weights);
    p.norm_epsilon = epsilon;
    const cudaError_t error = launch_gemv(context, p, kActF32, kEpiPlain);
    return error == cudaSuccess ? FORTAI_CUDA_OK : fail(context, "normalised matvec", error);
}

// ---------------------------------------------------------------------------
// FFN without any allocation
// ---------------------------------------------------------------------------
// Some hosts cannot let this library allocate once they are running: a serving
// process that has already handed every free byte of HBM to its weight and cache
// pools (a later cudaMalloc fails or fragments the pool), and a decode loop that
// cannot afford the device-wide synchronisation that cudaFree/cudaMalloc imply
// when a scratch buffer grows in the middle of a step.  For them the FFN's two
// intermediates - the fp32 hidden vector silu(gate.x) * (up.x) and its Q8_0
// image - live in a fixed array that is part of the library image.  Every GPU
// that loads the library holds these kStaticFfnBytes until the process exits.
namespace {

constexpr int kStaticFfnMaxInner = 32768;   // largest supported FFN inner size (gate/up rows)
constexpr size_t kStaticFfnHiddenBytes = static_cast<size_t>(kStaticFfnMaxInner) * sizeof(float);
// the prepared Q8_0 image of the hidden vector: int8 quants + one float scale per block
constexpr size_t kStaticFfnQ8Bytes =
    (static_cast<size_t>(kStaticFfnMaxInner) + kStaticFfnMaxInner / kBlockElems * 4 + 255) / 256 * 256;
constexpr size_t kStaticFfnBytes = kStaticFfnHiddenBytes + kStaticFfnQ8Bytes;

static __device__ __align__(256) unsigned char g_static_ffn_scratch[kStaticFfnBytes];

constexpr int kStaticFfnMaxDevices = 64;
unsigned char *g_static_ffn_address[kStaticFfnMaxDevices] = {};

// In host code the array's name is only a handle for the runtime, not a device
// address; the address on the current device comes from cudaGetSymbolAddress.
// Looked up once per device, with that device current.
cudaError_t static_ffn_address(int device, unsigned char **address) {
    if (device < 0 || device >= kStaticFfnMaxDevices) return cudaErrorInvalidDevice;
    if (!g_static_ffn_address[device]) {
        void *pointer = nullptr;
        const cudaError_t error = cudaGetSymbolAddress(&pointer, g_static_ffn_scratch);
        if (error != cudaSuccess) return error;
        g_static_ffn_address[device] = static_cast<unsigned char *>(pointer);
    }
    *address = g_static_ffn_address[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int fortai_cuda_q8_ffn_device_noalloc(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements) {
    if (!context || !gate_weights || !up_weights || !down_weights || !device_activation ||
        !device_output) return FORTAI_CUDA_INVALID;
    if (!ffn_shapes_ok(context, gate_weights, up_weights, down_weights) ||
        activation_elements != static_cast<size_t>(gate_weights->blocks) * kBlockElems ||
        output_elements < static_cast<size_t>(down_weights->rows)) return FORTAI_CUDA_INVALID;
    if (gate_weights->rows > kStaticFfnMaxInner) {
        std::snprintf(context->error, sizeof(context->error),
            "allocation-free FFN supports an inner size of at most %d, got %d",
            kStaticFfnMaxInner, gate_weights->rows);
        return FORTAI_CUDA_INVALID;
    }
    cudaSetDevice(context->device);
    unsigned char *scratch = nullptr;
    cudaError_t error = static_ffn_address(context->device, &scratch);
    if (error != cudaSuccess) return fail(context, "allocation-free FFN scratch lookup", error);
    float *hidden = reinterpret_cast<float *>(scratch);
    uint8_t *hidden_q8 = scratch + kStaticFfnHiddenBytes;
    // Both intermediates are fully rewritten by every call (each of the `inner`
    // floats, each of the inner/32 blocks), so nothing has to be cleared first.
    GemvParams p = single_params(context, gate_weights, device_activation, hidden);
    p.weights[1] = up_weights->data;
    p.rows[1] = up_weights->rows;
    p.segments = 2;
    error = launch_gemv_raw(context, p, kActF32, kEpiSiluPair);
    if (error == cudaSuccess)
        error = launch_planar_prepare(context, hidden, kActF32, down_weights->width,
            down_weights->blocks, hidden_q8);
    if (error == cudaSuccess) {
        const GemvParams d = single_params(context, down_weights, hidden_q8,
            static_cast<float *>(device_output));
        error = launch_gemv_raw(context, d, kActPlanar, kEpiPlain);
    }
    return error == cudaSuccess ? FORTAI_CUDA_OK
                                : fail(context, "allocation-free Qwen FFN device", error);
}

#ifdef FORTAI_MMQ_TRACE
// debug builds only (never declared in the public header)
extern "C" int fortai_cuda_mmq_trace_read(long long *host) {
    return fortai_b200::mmq_trace_read(host) == cudaSuccess ? 0 : 2;
}
#endif

// ---------------------------------------------------------------------------
// device groups
// ---------------------------------------------------------------------------
#include "device_group.cuh"
