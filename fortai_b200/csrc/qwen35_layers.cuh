// Device kernels of the two Qwen3.5 layer objects of the C ABI: the gated-delta-net
// ("recurrent") layer and the gated single-query attention layer.  They sit next to the
// Q8_0 hot path (every projection inside them is a Q8_0 GEMV from q8_gemv.cuh) and
// exist so that the reference's device pipeline runs on this backend end to end.
//
// Semantics follow the reference CPU model, which is the correctness reference of that
// project (src/models/qwen35/fortai_qwen35_cpu.f90:801-918 recurrent, :978-1035
// attention, helpers :1434-1539) and its C step function
// (src/backend/cpu/fortai_q8_dot.c:355-445); the reference's own CUDA versions are
// backend/cuda/fortai_cuda_backend.cu:386-481 and :539-669.
#pragma once

#include <cuda_fp16.h>

#include "q8_common.cuh"
#include "q8_gemv.cuh"

namespace fortai_b200 {

__device__ __forceinline__ float sigmoid_stable(float x) {
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float e = expf(x);
    return e / (1.0f + e);
}

__device__ __forceinline__ float softplus_clamped(float x) {
    if (x > 20.0f) return x;
    if (x < -20.0f) return expf(x);
    return logf(1.0f + expf(x));
}

__device__ __forceinline__ double warp_sum_double(double v) {
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Sum over a CTA of up to 1024 threads; every thread gets the result.
__device__ __forceinline__ double cta_sum_double(double v, double *scratch32) {
    v = warp_sum_double(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch32[warp] = v;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) total += scratch32[w];
    return total;
}

// ---- recurrent layer ------------------------------------------------------------
// Causal depthwise convolution over the last `kernel` inputs of every channel, SiLU,
// and the shift of the per-channel history.  conv_state is (kernel - 1) x conv_size,
// oldest first.
__global__ void __launch_bounds__(256)
gdn_conv_silu_kernel(float *__restrict__ qkv, const float *__restrict__ conv_weights,
    float *__restrict__ conv_state, int conv_size, int kernel) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= conv_size) return;
    qkv[c] = conv_silu_channel(conv_weights, conv_state, conv_size, kernel, c, qkv[c]);
}

// One gated-delta-net step for one value head per CTA.  Warps 0 and 1 first L2-normalise
// the head's query and key (sum of squares in double, 1 / max(sqrt(sum), epsilon), as
// l2_normalize_slice of the reference does; the convolved vector itself is left as it
// is), then every warp owns
// rows of the head_size x head_size state (decay, key dot, delta update, query dot), then
// the head's output is RMS-normalised, scaled by ssm_norm and gated by silu(gate).
__global__ void __launch_bounds__(1024)
gdn_step_kernel(const float *__restrict__ conv, const float *__restrict__ gate,
    const float *__restrict__ alpha, const float *__restrict__ beta,
    const float *__restrict__ ssm_a, const float *__restrict__ ssm_dt,
    const float *__restrict__ ssm_norm, float *__restrict__ state, float *__restrict__ output,
    int state_size, int key_heads, int value_heads, int head_size, float epsilon) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    extern __shared__ float gdn_shared[];     // head_size outputs, then query, then key
    __shared__ double reduce[32];
    const int head = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int key_head = head / (value_heads / key_heads);
    float *query = gdn_shared + head_size;
    float *key = query + head_size;
    const float *value = conv + 2 * state_size * key_heads + head * head_size;
    if (warp < 2) {
        const float *raw = warp == 0 ? conv + key_head * head_size
                                     : conv + state_size * key_heads + key_head * head_size;
        float *normalized = warp == 0 ? query : key;
        double sum = 0.0;
        for (int i = lane; i < head_size; i += 32) sum += static_cast<double>(raw[i]) * raw[i];
        sum = warp_sum_double(sum);
        const float inverse = 1.0f / fmaxf(sqrtf(static_cast<float>(sum)), epsilon);
        for (int i = lane; i < head_size; i += 32) normalized[i] = raw[i] * inverse;
    }
    __syncthreads();
    const float decay = expf(ssm_a[head] * softplus_clamped(alpha[head] + ssm_dt[head]));
    const float b = sigmoid_stable(beta[head]);
    const float scale = 1.0f / sqrtf(static_cast<float>(head_size));
    float *head_state = state + static_cast<size_t>(head) * head_size * head_size;
    // Two state rows per warp at a time: their loads and their two warp reductions each are
    // independent, which halves the length of the dependent chain a warp walks through.
    for (int row = warp; row < head_size; row += 2 * warps) {
        const int other = row + warps;
        const bool pair = other < head_size;
        float *s0 = head_state + static_cast<size_t>(row) * head_size;
        float *s1 = head_state + static_cast<size_t>(pair ? other : row) * head_size;
        float key_dot0 = 0.0f, key_dot1 = 0.0f;
        for (int c = lane; c < head_size; c += 32) {
            const float k = key[c];
            const float d0 = s0[c] * decay;
            const float d1 = s1[c] * decay;
            s0[c] = d0;
            if (pair) s1[c] = d1;
            key_dot0 = fmaf(d0, k, key_dot0);
            key_dot1 = fmaf(d1, k, key_dot1);
        }
        key_dot0 = warp_sum(key_dot0);
        key_dot1 = warp_sum(key_dot1);
        const float delta0 = (value[row] - key_dot0) * b;
        const float delta1 = (value[pair ? other : row] - key_dot1) * b;
        float query_dot0 = 0.0f, query_dot1 = 0.0f;
        for (int c = lane; c < head_size; c += 32) {
            const float k = key[c], q = query[c];
            const float u0 = fmaf(delta0, k, s0[c]);
            s0[c] = u0;
            query_dot0 = fmaf(u0, q, query_dot0);
            if (pair) {
                const float u1 = fmaf(delta1, k, s1[c]);
                s1[c] = u1;
                query_dot1 = fmaf(u1, q, query_dot1);
            }
        }
        query_dot0 = warp_sum(query_dot0);
        query_dot1 = warp_sum(query_dot1);
        if (lane == 0) {
            gdn_shared[row] = query_dot0 * scale;
            if (pair) gdn_shared[other] = query_dot1 * scale;
        }
    }
    __syncthreads();
    double sum = 0.0;
    for (int i = threadIdx.x; i < head_size; i += blockDim.x)
        sum += static_cast<double>(gdn_shared[i]) * gdn_shared[i];
    sum = cta_sum_double(sum, reduce);
    const float norm = sqrtf(static_cast<float>(sum / head_size) + epsilon);
    for (int i = threadIdx.x; i < head_size; i += blockDim.x)
        output[head * head_size + i] = gdn_shared[i] / norm * ssm_norm[i] *
            silu_ieee(gate[head * head_size + i]);
}

// ---- attention layer --------------------------------------------------------------
__device__ __forceinline__ void rope_pair(float *v, int dimension, int i, int position,
    float base) {
    const float angle = static_cast<float>(position) /
        powf(base, static_cast<float>(2 * i) / static_cast<float>(dimension));
    const float c = cosf(angle), s = sinf(angle);
    const float first = v[i], second = v[i + dimension / 2];
    v[i] = first * c - second * s;
    v[i + dimension / 2] = first * s + second * c;
}

// Blocks [0, heads): RMS-normalise (learned scale) and rotate the query part of each
// head (the second half of a head's 2 * head_size slot is its output gate and is left
// alone).  Blocks [heads, heads + kv_heads): the same for a key head, then store key and
// value of this position in the binary16 caches.
__global__ void __launch_bounds__(256)
attention_prepare_kernel(float *__restrict__ query, float *__restrict__ key,
    const float *__restrict__ value, const float *__restrict__ query_norm,
    const float *__restrict__ key_norm, __half *__restrict__ key_cache,
    __half *__restrict__ value_cache, int heads, int kv_heads, int head_size, int value_size,
    const int *__restrict__ position_ptr, int rope_dimension, float rope_base, float epsilon,
    int max_context, int *__restrict__ status) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    __shared__ double reduce[32];
    const int position = *position_ptr;
    // The position is a device word (a replayed graph or set_position may have put anything
    // there): one outside the caches is never used as an index.  The CTA records a status
    // and leaves; the next blocking call reports it.
    if (position < 0 || position >= max_context) {
        if (threadIdx.x == 0) atomicExch(status, kStatusPositionOutOfRange);
        return;
    }
    const bool is_query = static_cast<int>(blockIdx.x) < heads;
    const int head = is_query ? blockIdx.x : blockIdx.x - heads;
    float *v = is_query ? query + head * 2 * head_size : key + head * head_size;
    const float *weights = is_query ? query_norm : key_norm;
    double sum = 0.0;
    for (int i = threadIdx.x; i < head_size; i += blockDim.x)
        sum += static_cast<double>(v[i]) * v[i];
    sum = cta_sum_double(sum, reduce);
    const float inverse = 1.0f / sqrtf(static_cast<float>(sum / head_size) + epsilon);
    for (int i = threadIdx.x; i < head_size; i += blockDim.x) v[i] = v[i] * inverse * weights[i];
    __syncthreads();
    if (rope_dimension > 0)
        for (int i = threadIdx.x; i < rope_dimension / 2; i += blockDim.x)
            rope_pair(v, rope_dimension, i, position, rope_base);
    if (is_query) return;
    __syncthreads();
    for (int i = threadIdx.x; i < head_size; i += blockDim.x)
        key_cache[(static_cast<size_t>(position) * kv_heads + head) * head_size + i] =
            __float2half_rn(v[i]);
    for (int i = threadIdx.x; i < value_size; i += blockDim.x)
        value_cache[(static_cast<size_t>(position) * kv_heads + head) * value_size + i] =
            __float2half_rn(value[head * value_size + i]);
}

// Eight binary16 values of a cache row as floats (one 16-byte load).
__device__ __forceinline__ void load_half8(const __half *p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

// One CTA per head: scores against every cached key (one warp per position), softmax over
// positions, weighted sum of cached values (the warps share the positions, every lane owns
// eight value dimensions and reads them with one 16-byte load per position; the warps'
// partial sums meet in shared memory in warp order), sigmoid output gate.  Dynamic shared
// memory: max_context scores, then warps x value_size partial sums.  Head and value sizes
// that are not multiples of 8, or values wider than 256, take the element-wise path.
__global__ void __launch_bounds__(256)
attention_apply_kernel(const float *__restrict__ query, const __half *__restrict__ key_cache,
    const __half *__restrict__ value_cache, float *__restrict__ attention, int heads, int kv_heads,
    int head_size, int value_size, int max_context, const int *__restrict__ position_ptr,
    int context_limit, int *__restrict__ status) {
    grid_dependents_may_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float scores[];      // max_context entries, then partials
    __shared__ float reduce[32];
    const int head = blockIdx.x;
    const int position = *position_ptr;
    // see attention_prepare_kernel: a position outside the caches (and outside scores[]) is
    // reported, not used
    if (position < 0 || position >= context_limit) {
        if (threadIdx.x == 0) atomicExch(status, kStatusPositionOutOfRange);
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int kv_head = head / (heads / kv_heads);
    const float *q = query + head * 2 * head_size;
    const float *gate = q + head_size;
    const float scale = 1.0f / sqrtf(static_cast<float>(head_size));
    const bool wide_keys = (head_size & 7) == 0;
    for (int p = warp; p <= position; p += warps) {
        const __half *k = key_cache + (static_cast<size_t>(p) * kv_heads + kv_head) * head_size;
        float dot = 0.0f;
        if (wide_keys) {
            for (int c = lane; c < (head_size >> 3); c += 32) {
                float kv[8];
                load_half8(k + 8 * c, kv);
                const float4 q0 = *reinterpret_cast<const float4 *>(q + 8 * c);
                const float4 q1 = *reinterpret_cast<const float4 *>(q + 8 * c + 4);
                dot = fmaf(q0.x, kv[0], dot);
                dot = fmaf(q0.y, kv[1], dot);
                dot = fmaf(q0.z, kv[2], dot);
                dot = fmaf(q0.w, kv[3], dot);
                dot = fmaf(q1.x, kv[4], dot);
                dot = fmaf(q1.y, kv[5], dot);
                dot = fmaf(q1.z, kv[6], dot);
                dot = fmaf(q1.w, kv[7], dot);
            }
        } else {
            for (int i = lane; i < head_size; i += 32) dot = fmaf(q[i], __half2float(k[i]), dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) scores[p] = dot * scale;
    }
    __syncthreads();
    float maximum = -3.402823466e+38f;
    for (int p = threadIdx.x; p <= position; p += blockDim.x) maximum = fmaxf(maximum, scores[p]);
#pragma unroll
    for (int offset = 16; offset; offset >>= 1)
        maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
    if (lane == 0) reduce[warp] = maximum;
    __syncthreads();
    maximum = reduce[0];
    for (int w = 1; w < warps; ++w) maximum = fmaxf(maximum, reduce[w]);
    __syncthreads();
    float sum = 0.0f;
    for (int p = threadIdx.x; p <= position; p += blockDim.x) {
        const float e = expf(scores[p] - maximum);
        scores[p] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) reduce[warp] = sum;
    __syncthreads();
    float normalizer = 0.0f;
    for (int w = 0; w < warps; ++w) normalizer += reduce[w];
    if ((value_size & 7) == 0 && value_size <= 256) {
        float *partials = scores + max_context;          // [warps][value_size]
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        const bool owner = lane < (value_size >> 3);
        if (owner) {
            for (int p = warp; p <= position; p += warps) {
                float vv[8];
                load_half8(value_cache + (static_cast<size_t>(p) * kv_heads + kv_head) * value_size +
                    8 * lane, vv);
                const float weight = scores[p];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(weight, vv[i], acc[i]);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) partials[warp * value_size + 8 * lane + i] = acc[i];
        }
        __syncthreads();
        const float inverse = 1.0f / normalizer;
        for (int i = threadIdx.x; i < value_size; i += blockDim.x) {
            float total = 0.0f;
            for (int w = 0; w < warps; ++w) total += partials[w * value_size + i];
            attention[head * value_size + i] = total * inverse * sigmoid_stable(gate[i]);
        }
        return;
    }
    for (int i = threadIdx.x; i < value_size; i += blockDim.x) {
        float total = 0.0f;
        for (int p = 0; p <= position; ++p) {
            const __half *v = value_cache + (static_cast<size_t>(p) * kv_heads + kv_head) * value_size;
            total = fmaf(scores[p] / normalizer, __half2float(v[i]), total);
        }
        attention[head * value_size + i] = total * sigmoid_stable(gate[i]);
    }
}

}  // namespace fortai_b200
