// A group of GPUs of one box behind the C ABI: row- and column-sharded Q8_0 projections
// for hosts that are not Python (one host thread drives all devices, as a Fortran caller
// would).  The reference is single-GPU ("deferred", ROADMAP.md:31); the only multi-device
// hook it has is the device index of fortai_cuda_q8_context_create
// (backend/cuda/fortai_cuda_backend.h:22).  The partition is the one its CPU matvec already
// uses across OpenMP threads: contiguous ranges of output rows
// (src/fortai_gguf_runtime.f90:457-463).
//
//   group            one context per device, peer access enabled between all pairs, and on
//                    every device a full-length result vector and a flag array that the
//                    others can write (plain peer stores; no multicast of any kind)
//   row shards       device g owns rows [first_g, first_g + count_g); one launch per device
//                    of the GEMV fused with its all-gather
//                    (fortai_cuda_q8_matvec_device_f32_allgather): every device ends up with
//                    every slice, device 0's copy goes back to the host
//   column shards    device g owns blocks [first_g, +count_g) of every row of the FFN down
//                    matrix and the matching rows of gate/up, so the hidden vector never
//                    crosses devices; the partial outputs are copied to device 0 and summed
//                    there in device order (deterministic)
//
// Everything is enqueued on the devices' streams before the host waits for any of it, so
// the kernels that wait on one another (the fused all-gather) all run.
#pragma once

namespace {

constexpr int kGroupMaxDevices = kMaxPeers;

// out[i] = sum over devices of partial[d][i], in device order
__global__ void __launch_bounds__(256)
group_sum_kernel(const float *__restrict__ partials, int devices, int elements,
    float *__restrict__ out) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < elements;
         i += gridDim.x * blockDim.x) {
        float total = partials[i];
        for (int d = 1; d < devices; ++d) total += partials[static_cast<size_t>(d) * elements + i];
        out[i] = total;
    }
}

}  // namespace

struct fortai_cuda_q8_group {
    int count = 0;
    int devices[kGroupMaxDevices] = {};
    fortai_cuda_q8_context *contexts[kGroupMaxDevices] = {};
    float *result[kGroupMaxDevices] = {};        // full-length vectors, grown on demand
    size_t result_elements = 0;
    unsigned *flags[kGroupMaxDevices] = {};      // kGroupMaxDevices words each, zero at creation
    float *activation[kGroupMaxDevices] = {};    // fp32 input on each device, grown on demand
    size_t activation_elements = 0;
    float *partials = nullptr;                   // device 0: count x elements partial outputs
    size_t partial_elements = 0;
    cudaEvent_t done[kGroupMaxDevices] = {};
    unsigned sequence = 0;                       // flag sequence of the fused all-gather calls
    char error[256] = {};
};

struct fortai_cuda_q8_group_weights {
    fortai_cuda_q8_group *group = nullptr;
    int rows = 0, width = 0, mode = 0;           // mode 0: row shards, 1: column shards
    int first[kGroupMaxDevices] = {};            // first row (mode 0) / first block (mode 1)
    int extent[kGroupMaxDevices] = {};           // rows (mode 0) / blocks (mode 1); may be 0
    fortai_cuda_q8_weights *shards[kGroupMaxDevices] = {};
};

namespace {

int group_fail(fortai_cuda_q8_group *group, const char *operation, cudaError_t error) {
    if (group)
        std::snprintf(group->error, sizeof(group->error), "%s: %s", operation,
            error == cudaSuccess ? "failed" : cudaGetErrorString(error));
    return FORTAI_CUDA_RUNTIME_ERROR;
}

int group_fail_from(fortai_cuda_q8_group *group, const char *operation, int device_slot) {
    if (group)
        std::snprintf(group->error, sizeof(group->error), "%s (device %d): %s", operation,
            group->devices[device_slot],
            fortai_cuda_q8_last_error(group->contexts[device_slot]));
    return FORTAI_CUDA_RUNTIME_ERROR;
}

// contiguous ranges of `total` items in units of `multiple`, sizes differing by one unit
void group_partition(int total, int parts, int multiple, int *first, int *extent) {
    const int units = total / multiple, tail = total % multiple;
    const int base = units / parts, extra = units % parts;
    int at = 0, last_owner = 0;
    for (int g = 0; g < parts; ++g) {
        extent[g] = (base + (g < extra ? 1 : 0)) * multiple;
        first[g] = at;
        at += extent[g];
        if (extent[g]) last_owner = g;
    }
    if (tail) {
        extent[last_owner] += tail;
        for (int g = last_owner + 1; g < parts; ++g) first[g] += tail;
    }
}

cudaError_t group_grow(fortai_cuda_q8_group *group, size_t activation_elements,
    size_t result_elements, size_t partial_elements) {
    cudaError_t error = cudaSuccess;
    if (activation_elements > group->activation_elements) {
        for (int g = 0; g < group->count && error == cudaSuccess; ++g) {
            cudaSetDevice(group->devices[g]);
            cudaFree(group->activation[g]);
            group->activation[g] = nullptr;
            error = cudaMalloc(reinterpret_cast<void **>(&group->activation[g]),
                activation_elements * sizeof(float));
        }
        group->activation_elements = error == cudaSuccess ? activation_elements : 0;
    }
    if (error == cudaSuccess && result_elements > group->result_elements) {
        for (int g = 0; g < group->count && error == cudaSuccess; ++g) {
            cudaSetDevice(group->devices[g]);
            cudaFree(group->result[g]);
            group->result[g] = nullptr;
            error = cudaMalloc(reinterpret_cast<void **>(&group->result[g]),
                result_elements * sizeof(float));
        }
        group->result_elements = error == cudaSuccess ? result_elements : 0;
    }
    if (error == cudaSuccess && partial_elements > group->partial_elements) {
        cudaSetDevice(group->devices[0]);
        cudaFree(group->partials);
        group->partials = nullptr;
        error = cudaMalloc(reinterpret_cast<void **>(&group->partials),
            partial_elements * group->count * sizeof(float));
        group->partial_elements = error == cudaSuccess ? partial_elements : 0;
    }
    return error;
}

}  // namespace

extern "C" int fortai_cuda_q8_group_destroy(fortai_cuda_q8_group *group) {
    if (!group) return FORTAI_CUDA_OK;
    for (int g = 0; g < group->count; ++g) {
        cudaSetDevice(group->devices[g]);
        if (group->contexts[g]) cudaStreamSynchronize(group->contexts[g]->stream);
        cudaFree(group->result[g]);
        cudaFree(group->flags[g]);
        cudaFree(group->activation[g]);
        if (group->done[g]) cudaEventDestroy(group->done[g]);
    }
    if (group->count) {
        cudaSetDevice(group->devices[0]);
        cudaFree(group->partials);
    }
    for (int g = 0; g < group->count; ++g) fortai_cuda_q8_context_destroy(group->contexts[g]);
    delete group;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_group_create(const int *devices, int count,
    fortai_cuda_q8_group **group) {
    if (!devices || !group || count < 1 || count > kGroupMaxDevices) return FORTAI_CUDA_INVALID;
    *group = nullptr;
    int available = 0;
    if (cudaGetDeviceCount(&available) != cudaSuccess) {
        cudaGetLastError();
        return FORTAI_CUDA_RUNTIME_ERROR;
    }
    for (int a = 0; a < count; ++a) {
        if (devices[a] < 0 || devices[a] >= available) return FORTAI_CUDA_INVALID;
        for (int b = 0; b < a; ++b)
            if (devices[a] == devices[b]) return FORTAI_CUDA_INVALID;
    }
    auto *created = new (std::nothrow) fortai_cuda_q8_group;
    if (!created) return FORTAI_CUDA_RUNTIME_ERROR;
    created->count = count;
    bool ok = true;
    for (int g = 0; g < count && ok; ++g) {
        created->devices[g] = devices[g];
        ok = fortai_cuda_q8_context_create(devices[g], &created->contexts[g]) == FORTAI_CUDA_OK;
    }
    // every device must be able to store into every other device's result vector and flags
    for (int a = 0; a < count && ok; ++a) {
        cudaSetDevice(devices[a]);
        for (int b = 0; b < count && ok; ++b) {
            if (a == b) continue;
            int can = 0;
            ok = cudaDeviceCanAccessPeer(&can, devices[a], devices[b]) == cudaSuccess && can;
            if (ok) {
                const cudaError_t error = cudaDeviceEnablePeerAccess(devices[b], 0);
                if (error == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else ok = error == cudaSuccess;
            }
        }
    }
    for (int g = 0; g < count && ok; ++g) {
        cudaSetDevice(devices[g]);
        ok = cudaMalloc(reinterpret_cast<void **>(&created->flags[g]),
                 kGroupMaxDevices * sizeof(unsigned)) == cudaSuccess &&
            cudaMemset(created->flags[g], 0, kGroupMaxDevices * sizeof(unsigned)) == cudaSuccess &&
            cudaEventCreateWithFlags(&created->done[g], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) {
        fortai_cuda_q8_group_destroy(created);
        cudaGetLastError();         // leave no stale error behind for the caller's next call
        return FORTAI_CUDA_RUNTIME_ERROR;
    }
    *group = created;
    return FORTAI_CUDA_OK;
}

extern "C" int fortai_cuda_q8_group_device_count(const fortai_cuda_q8_group *group) {
    return group ? group->count : 0;
}

extern "C" const char *fortai_cuda_q8_group_last_error(const fortai_cuda_q8_group *group) {
    return group ? group->error : "invalid device group";
}

extern "C" int fortai_cuda_q8_group_weights_destroy(fortai_cuda_q8_group_weights *weights) {
    if (!weights) return FORTAI_CUDA_OK;
    for (int g = 0; g < kGroupMaxDevices; ++g)
        if (weights->shards[g]) fortai_cuda_q8_weights_destroy(weights->shards[g]);
    delete weights;
    return FORTAI_CUDA_OK;
}

// shard_mode 0: contiguous row ranges (lm_head, FFN gate/up); 1: block ranges of every row
// (FFN down), cut in the same proportions as a row-sharded matrix of `width` rows would be,
// so that device g's slice of the hidden vector is exactly what its gate/up shard produces.
extern "C" int fortai_cuda_q8_group_weights_upload(fortai_cuda_q8_group *group,
    const void *host_weights, size_t weight_bytes, int rows, int width, int shard_mode,
    fortai_cuda_q8_group_weights **weights) {
    if (!group || !host_weights || !weights || rows <= 0 || width <= 0 ||
        width % kBlockElems != 0 || (shard_mode != 0 && shard_mode != 1))
        return FORTAI_CUDA_INVALID;
    *weights = nullptr;
    const size_t row_bytes = static_cast<size_t>(width / kBlockElems) * kBlockBytes;
    if (weight_bytes < row_bytes * rows) return FORTAI_CUDA_INVALID;
    auto *created = new (std::nothrow) fortai_cuda_q8_group_weights;
    if (!created) return FORTAI_CUDA_RUNTIME_ERROR;
    created->group = group;
    created->rows = rows;
    created->width = width;
    created->mode = shard_mode;
    int first[kGroupMaxDevices], extent[kGroupMaxDevices];
    if (shard_mode == 0) {
        // FFN gate/up rows feed Q8_0 blocks of the hidden vector: cut on multiples of 32 when
        // the row count allows it, so that a column-sharded partner lines up
        group_partition(rows, group->count, rows % kBlockElems == 0 ? kBlockElems : 1, first,
            extent);
    } else {
        group_partition(width, group->count, kBlockElems, first, extent);
        for (int g = 0; g < group->count; ++g) {
            first[g] /= kBlockElems;
            extent[g] /= kBlockElems;
        }
    }
    int code = FORTAI_CUDA_OK;
    for (int g = 0; g < group->count && code == FORTAI_CUDA_OK; ++g) {
        created->first[g] = first[g];
        created->extent[g] = extent[g];
        if (extent[g] == 0) continue;
        if (shard_mode == 0)
            code = fortai_cuda_q8_weights_upload(group->contexts[g],
                static_cast<const uint8_t *>(host_weights) + row_bytes * first[g],
                row_bytes * extent[g], extent[g], width, &created->shards[g]);
        else
            code = fortai_cuda_q8_weights_upload_columns(group->contexts[g], host_weights,
                weight_bytes, rows, width, first[g], extent[g], &created->shards[g]);
        if (code != FORTAI_CUDA_OK) group_fail_from(group, "group weights upload", g);
    }
    if (code != FORTAI_CUDA_OK) {
        fortai_cuda_q8_group_weights_destroy(created);
        return code;
    }
    *weights = created;
    return FORTAI_CUDA_OK;
}

// Row-sharded matvec: host fp32 vector in, host fp32 result out; blocks.  elapsed_ms is host
// time around the whole call (transfers included), as fortai_cuda_q8_matvec_host reports it
// for one device (backend/cuda/fortai_cuda_backend.cu:1097-1129).
extern "C" int fortai_cuda_q8_group_matvec_f32(fortai_cuda_q8_group *group,
    const fortai_cuda_q8_group_weights *weights, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!group || !weights || weights->group != group || weights->mode != 0 || !host_activation ||
        !host_output || !elapsed_ms || activation_elements != static_cast<size_t>(weights->width) ||
        output_bytes < static_cast<size_t>(weights->rows) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    const auto begin = std::chrono::steady_clock::now();
    cudaError_t error = group_grow(group, activation_elements, weights->rows, 0);
    if (error != cudaSuccess) return group_fail(group, "group scratch", error);
    void *outputs[kGroupMaxDevices], *flags[kGroupMaxDevices];
    for (int g = 0; g < group->count; ++g) {
        outputs[g] = group->result[g];
        flags[g] = group->flags[g];
    }
    // enqueue everything on every device before waiting for anything: the fused kernels wait
    // for one another's flags
    for (int g = 0; g < group->count; ++g) {
        fortai_cuda_q8_context *c = group->contexts[g];
        cudaSetDevice(group->devices[g]);
        error = cudaMemcpyAsync(group->activation[g], host_activation,
            activation_elements * sizeof(float), cudaMemcpyHostToDevice, c->stream);
        if (error != cudaSuccess) return group_fail(group, "group activation upload", error);
    }
    // a device without rows still takes part in the flag exchange of the others: give it the
    // protocol without a slice by skipping it on both sides (peer lists hold only owners)
    int owners[kGroupMaxDevices], owner_count = 0;
    for (int g = 0; g < group->count; ++g)
        if (weights->extent[g] > 0) owners[owner_count++] = g;
    void *owner_outputs[kGroupMaxDevices], *owner_flags[kGroupMaxDevices];
    for (int k = 0; k < owner_count; ++k) {
        owner_outputs[k] = outputs[owners[k]];
        owner_flags[k] = flags[owners[k]];
    }
    // every rank of one call must carry the same flag sequence number, whatever else its
    // context has been used for
    ++group->sequence;
    for (int k = 0; k < owner_count; ++k) {
        const int g = owners[k];
        group->contexts[g]->allgather_sequence = group->sequence - 1;
        const int code = fortai_cuda_q8_matvec_device_f32_allgather(group->contexts[g],
            weights->shards[g], group->activation[g], activation_elements, owner_outputs,
            owner_flags, owner_count, k, weights->first[g], weights->rows);
        if (code != FORTAI_CUDA_OK) return group_fail_from(group, "group matvec", g);
    }
    // the first owner's vector holds every slice when its kernel has completed
    const int reader = owners[0];
    cudaSetDevice(group->devices[reader]);
    error = cudaMemcpyAsync(host_output, group->result[reader],
        static_cast<size_t>(weights->rows) * sizeof(float), cudaMemcpyDeviceToHost,
        group->contexts[reader]->stream);
    if (error != cudaSuccess) return group_fail(group, "group result download", error);
    // wait for every device (a rank that ran ahead must not start the next call's stores
    // while this call's result is still being read), and collect device-side give-ups
    for (int g = 0; g < group->count; ++g) {
        if (fortai_cuda_q8_context_synchronize(group->contexts[g]) != FORTAI_CUDA_OK)
            return group_fail_from(group, "group matvec", g);
    }
    *elapsed_ms = std::chrono::duration<float, std::milli>(
        std::chrono::steady_clock::now() - begin).count();
    return FORTAI_CUDA_OK;
}

// FFN with gate/up row-sharded and down column-sharded (all three uploaded through this
// group: gate and up with shard_mode 0, down with shard_mode 1).  Host fp32 in and out;
// blocks.
extern "C" int fortai_cuda_q8_group_ffn_f32(fortai_cuda_q8_group *group,
    const fortai_cuda_q8_group_weights *gate, const fortai_cuda_q8_group_weights *up,
    const fortai_cuda_q8_group_weights *down, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms) {
    if (!group || !gate || !up || !down || gate->group != group || up->group != group ||
        down->group != group || gate->mode != 0 || up->mode != 0 || down->mode != 1 ||
        !host_activation || !host_output || !elapsed_ms) return FORTAI_CUDA_INVALID;
    // the shape rules of fortai_cuda_q8_ffn_device (backend/cuda/fortai_cuda_backend.cu:1257-1262)
    if (gate->rows != up->rows || gate->width != up->width || gate->rows != down->width ||
        activation_elements != static_cast<size_t>(gate->width) ||
        output_bytes < static_cast<size_t>(down->rows) * sizeof(float))
        return FORTAI_CUDA_INVALID;
    for (int g = 0; g < group->count; ++g)
        if (gate->first[g] != down->first[g] * kBlockElems ||
            gate->extent[g] != down->extent[g] * kBlockElems) return FORTAI_CUDA_INVALID;
    const auto begin = std::chrono::steady_clock::now();
    const size_t hidden = static_cast<size_t>(down->rows);
    cudaError_t error = group_grow(group, activation_elements, hidden, hidden);
    if (error != cudaSuccess) return group_fail(group, "group scratch", error);
    int active = 0;
    for (int g = 0; g < group->count; ++g) {
        if (gate->extent[g] == 0) continue;
        fortai_cuda_q8_context *c = group->contexts[g];
        cudaSetDevice(group->devices[g]);
        error = cudaMemcpyAsync(group->activation[g], host_activation,
            activation_elements * sizeof(float), cudaMemcpyHostToDevice, c->stream);
        if (error != cudaSuccess) return group_fail(group, "group activation upload", error);
        if (fortai_cuda_q8_ffn_device(c, gate->shards[g], up->shards[g], down->shards[g],
                group->activation[g], activation_elements, group->result[g], hidden) !=
            FORTAI_CUDA_OK) return group_fail_from(group, "group FFN", g);
        // the partial output goes to its slot on device 0 (a peer copy in this device's stream)
        error = cudaMemcpyPeerAsync(group->partials + static_cast<size_t>(active) * hidden,
            group->devices[0], group->result[g], group->devices[g], hidden * sizeof(float),
            c->stream);
        if (error == cudaSuccess) error = cudaEventRecord(group->done[g], c->stream);
        if (error != cudaSuccess) return group_fail(group, "group partial copy", error);
        ++active;
    }
    fortai_cuda_q8_context *c0 = group->contexts[0];
    cudaSetDevice(group->devices[0]);
    for (int g = 0; g < group->count; ++g) {
        if (gate->extent[g] == 0) continue;
        error = cudaStreamWaitEvent(c0->stream, group->done[g], 0);
        if (error != cudaSuccess) return group_fail(group, "group reduce", error);
    }
    group_sum_kernel<<<static_cast<int>((hidden + 255) / 256), 256, 0, c0->stream>>>(
        group->partials, active, static_cast<int>(hidden), group->result[0]);
    ++c0->launches;
    error = cudaGetLastError();
    if (error == cudaSuccess)
        error = cudaMemcpyAsync(host_output, group->result[0], hidden * sizeof(float),
            cudaMemcpyDeviceToHost, c0->stream);
    if (error != cudaSuccess) return group_fail(group, "group reduce", error);
    for (int g = 0; g < group->count; ++g)
        if (fortai_cuda_q8_context_synchronize(group->contexts[g]) != FORTAI_CUDA_OK)
            return group_fail_from(group, "group FFN", g);
    *elapsed_ms = std::chrono::duration<float, std::milli>(
        std::chrono::steady_clock::now() - begin).count();
    return FORTAI_CUDA_OK;
}
