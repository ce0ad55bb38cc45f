/* CPU oracle for the Q8_0 matvec hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in portable scalar C, the arithmetic that the reference
 * runs on an AVX2 host (every x86 machine this project targets takes that
 * path).  It is the checker that the CUDA kernels are compared against; it is
 * never linked into, imported by, or called from the shipped library.  Only
 * the test-suite, the smoke check and the CPU-baseline leg of the benchmark
 * may load it.
 *
 * Reference locations restated here (paths are inside the reference project):
 *   half <-> float          src/backend/cpu/fortai_q8_dot.c:53-113
 *   activation quantizer    src/backend/cpu/fortai_q8_dot.c:153-198 (AVX2 path)
 *                           and :128-150 (scalar path, ties-away rounding)
 *   one-row dot product     src/backend/cpu/fortai_q8_dot.c:287-331 (AVX2 path)
 *                           and :262-284 (scalar path)
 *   row dequantisation      src/backend/cpu/fortai_q8_dot.c:215-227
 *   SiLU(gate) * up         src/backend/cpu/fortai_q8_dot.c:9-51, 484-525
 *   matvec drivers          src/fortai_gguf_runtime.f90:424-465 (single),
 *                           :467-514 (pair), :516-588 (triplet)
 *   FFN composition         src/models/qwen35/fortai_qwen35_cpu.f90:672-677
 *
 * Parity pin: tests compare every function below, bit for bit, with the
 * reference's own C file compiled in place (oracle/_ref, see the Makefile) and
 * with the known answers of test/test_fortai_smoke.f90:213-266.
 *
 * A Q8_0 block is 34 bytes: a little-endian IEEE binary16 scale followed by
 * 32 signed bytes; value = scale * byte.  A matrix is rows x (K/32) blocks,
 * row-major, K contiguous.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { Q8_BLOCK_ELEMS = 32, Q8_BLOCK_BYTES = 34 };

enum {
    ORACLE_OK = 0,
    ORACLE_INVALID = 1
};

/* ---- binary16 conversions (bit-level, round to nearest even) ------------ */

/* Same value the F16C instruction produces (fortai_q8_dot.c:176). */
uint16_t oracle_float_to_half(float value)
{
    uint32_t x;
    memcpy(&x, &value, sizeof x);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t mag = x & 0x7fffffffu;
    if (mag >= 0x7f800000u)                       /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | (mag > 0x7f800000u ? 0x0200u : 0u));
    if (mag >= 0x477ff000u)                       /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    if (mag < 0x33000001u)                        /* <= 2^-25: rounds to zero */
        return (uint16_t)sign;
    int exp = (int)(mag >> 23) - 127;
    uint32_t man = (mag & 0x007fffffu) | 0x00800000u;
    int shift;                                    /* bits to drop from the 24-bit significand */
    uint32_t base;
    if (exp < -14) {                              /* subnormal half */
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x007fffffu;
    }
    const uint32_t kept = man >> shift;
    const uint32_t rest = man & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    uint32_t out = base + kept;
    if (rest > halfway || (rest == halfway && (kept & 1u)))
        ++out;                                    /* carry may roll into the exponent: still correct */
    return (uint16_t)(sign | out);
}

float oracle_half_to_float(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    const uint32_t man = h & 0x03ffu;
    float out;
    uint32_t bits;
    if (exp == 0) {
        /* zero or subnormal: value = man * 2^-24, exact in float */
        out = (float)man * 5.9604644775390625e-08f;
        memcpy(&bits, &out, sizeof bits);
        bits |= sign;
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    memcpy(&out, &bits, sizeof out);
    return out;
}

/* ---- activation quantizer ---------------------------------------------- */

static inline int8_t saturate_i8(float rounded)
{
    /* cvtps2dq then two saturating packs (fortai_q8_dot.c:179-192). */
    if (rounded > 127.0f) return 127;
    if (rounded < -128.0f) return -128;
    return (int8_t)(int32_t)rounded;
}

/* AVX2 path: IEEE division, multiply, round half to even.  Writes 34 bytes per
 * block into `output` and the float value of each stored scale into `scales`.
 * Does nothing when count <= 0 or count is not a multiple of 32
 * (fortai_q8_dot.c:204-205). */
void oracle_q8_quantize(const float *input, int8_t *output, float *scales, int64_t count)
{
    if (count <= 0 || count % Q8_BLOCK_ELEMS != 0)
        return;
    for (int64_t b = 0; b < count / Q8_BLOCK_ELEMS; ++b) {
        const float *x = input + b * Q8_BLOCK_ELEMS;
        int8_t *dst = output + b * Q8_BLOCK_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i) {
            const float a = fabsf(x[i]);
            if (a > amax) amax = a;               /* maxps ignores NaN in the second operand */
        }
        const float scale = amax / 127.0f;
        const float inverse = amax != 0.0f ? 127.0f / amax : 0.0f;
        const uint16_t bits = oracle_float_to_half(scale);
        if (scales) scales[b] = oracle_half_to_float(bits);
        dst[0] = (int8_t)(bits & 0xffu);
        dst[1] = (int8_t)(bits >> 8);
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i) {
            volatile float product = x[i] * inverse;   /* keep the rounding of a separate multiply */
            dst[2 + i] = saturate_i8(nearbyintf(product));
        }
    }
}

/* Scalar fallback of the reference (hosts without AVX2): same scale, but the
 * quants round half away from zero (roundf, fortai_q8_dot.c:148). */
void oracle_q8_quantize_ties_away(const float *input, int8_t *output, float *scales,
    int64_t count)
{
    if (count <= 0 || count % Q8_BLOCK_ELEMS != 0)
        return;
    for (int64_t b = 0; b < count / Q8_BLOCK_ELEMS; ++b) {
        const float *x = input + b * Q8_BLOCK_ELEMS;
        int8_t *dst = output + b * Q8_BLOCK_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i) {
            const float a = fabsf(x[i]);
            if (a > amax) amax = a;
        }
        const float scale = amax / 127.0f;
        const float inverse = amax != 0.0f ? 127.0f / amax : 0.0f;
        const uint16_t bits = oracle_float_to_half(scale);
        if (scales) scales[b] = oracle_half_to_float(bits);
        dst[0] = (int8_t)(bits & 0xffu);
        dst[1] = (int8_t)(bits >> 8);
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i) {
            volatile float product = x[i] * inverse;
            dst[2 + i] = (int8_t)roundf(product);
        }
    }
}

/* ---- dot products -------------------------------------------------------- */

static inline uint16_t block_scale_bits(const int8_t *block)
{
    return (uint16_t)((uint16_t)(uint8_t)block[0] | ((uint16_t)(uint8_t)block[1] << 8));
}

static inline int16_t saturate_i16(int32_t v)
{
    return (int16_t)(v > 32767 ? 32767 : (v < -32768 ? -32768 : v));
}

/* One output row exactly as the AVX2 path forms it (fortai_q8_dot.c:301-329):
 * per block, eight int32 partial sums of four byte-products each (pmaddubsw on
 * |w| and sign-adjusted a, with its int16 saturation, then pmaddwd by ones),
 * each converted to float and fused-multiply-added into its own accumulator
 * lane with scale = half(w scale) * scales[block]; lanes are then summed as
 * (l0+l4)+(l2+l6) and (l1+l5)+(l3+l7), and those two are added. */
float oracle_q8_dot(const int8_t *weights, const int8_t *quantized, const float *scales,
    int64_t row, int64_t block_count)
{
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int8_t *w_row = weights + row * block_count * Q8_BLOCK_BYTES;
    for (int64_t b = 0; b < block_count; ++b) {
        const int8_t *w = w_row + b * Q8_BLOCK_BYTES;
        const int8_t *a = quantized + b * Q8_BLOCK_BYTES;
        const float scale = oracle_half_to_float(block_scale_bits(w)) * scales[b];
        for (int l = 0; l < 8; ++l) {
            int32_t partial = 0;
            for (int p = 0; p < 2; ++p) {
                int32_t pair = 0;
                for (int j = 0; j < 2; ++j) {
                    const int i = 4 * l + 2 * p + j;
                    const int32_t wq = w[2 + i];
                    const int32_t aq = a[2 + i];
                    /* psignb(w, w): |w| as an unsigned byte (|-128| stays 128) */
                    const int32_t wabs = wq < 0 ? -wq : wq;
                    /* psignb(a, w): a negated where w < 0, zero where w == 0;
                     * -(-128) wraps back to -128 in a signed byte */
                    int32_t as = wq == 0 ? 0 : (wq < 0 ? -aq : aq);
                    if (as == 128) as = -128;
                    pair += wabs * as;
                }
                partial += saturate_i16(pair);
            }
            lane[l] = fmaf(scale, (float)partial, lane[l]);
        }
    }
    float s4[4];
    for (int l = 0; l < 4; ++l) s4[l] = lane[l] + lane[l + 4];
    const float s0 = s4[0] + s4[2];
    const float s1 = s4[1] + s4[3];
    return s0 + s1;
}

/* The scalar path of the reference (fortai_q8_dot.c:262-284): one exact int32
 * dot per block, `result += half(w scale) * scales[b] * (float)dot` with a
 * separate multiply and add, blocks in ascending order. */
float oracle_q8_dot_blockwise(const int8_t *weights, const int8_t *quantized,
    const float *scales, int64_t row, int64_t block_count)
{
    volatile float result = 0.0f;
    const int8_t *w_row = weights + row * block_count * Q8_BLOCK_BYTES;
    for (int64_t b = 0; b < block_count; ++b) {
        const int8_t *w = w_row + b * Q8_BLOCK_BYTES;
        const int8_t *a = quantized + b * Q8_BLOCK_BYTES;
        int32_t dot = 0;
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i)
            dot += (int32_t)w[2 + i] * (int32_t)a[2 + i];
        volatile float term = oracle_half_to_float(block_scale_bits(w)) * scales[b];
        term = term * (float)dot;
        result = result + term;
    }
    return result;
}

/* Exact integer dot of every (row, block): out[row * block_count + b].  This is
 * the loop at fortai_q8_dot.c:277-279 kept per block; int8 MMA, dp4a and the
 * AVX2 lane partials all sum to this value. */
void oracle_q8_block_dots(const int8_t *weights, const int8_t *quantized, int64_t rows,
    int64_t block_count, int32_t *out)
{
#pragma omp parallel for schedule(static) if (rows >= 128)
    for (int64_t row = 0; row < rows; ++row) {
        for (int64_t b = 0; b < block_count; ++b) {
            const int8_t *w = weights + (row * block_count + b) * Q8_BLOCK_BYTES;
            const int8_t *a = quantized + b * Q8_BLOCK_BYTES;
            int32_t dot = 0;
            for (int i = 0; i < Q8_BLOCK_ELEMS; ++i)
                dot += (int32_t)w[2 + i] * (int32_t)a[2 + i];
            out[row * block_count + b] = dot;
        }
    }
}

/* fortai_q8_dot.c:215-227 */
void oracle_q8_dequantize_row(const int8_t *weights, float *output, int64_t block_count)
{
    for (int64_t b = 0; b < block_count; ++b) {
        const int8_t *w = weights + b * Q8_BLOCK_BYTES;
        const float scale = oracle_half_to_float(block_scale_bits(w));
        for (int i = 0; i < Q8_BLOCK_ELEMS; ++i)
            output[b * Q8_BLOCK_ELEMS + i] = scale * (float)w[2 + i];
    }
}

/* ---- matvec drivers (the Fortran loops, restated) ------------------------ */

static void rows_loop(const int8_t *weights, const int8_t *quantized, const float *scales,
    int64_t rows, int64_t blocks, float *values, int parallel)
{
    /* serial below 128 rows, otherwise OpenMP static over rows
     * (fortai_gguf_runtime.f90:451-464) */
    if (!parallel) {
        for (int64_t row = 0; row < rows; ++row)
            values[row] = oracle_q8_dot(weights, quantized, scales, row, blocks);
    } else {
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < rows; ++row)
            values[row] = oracle_q8_dot(weights, quantized, scales, row, blocks);
    }
}

/* gguf_tensor_matvec_q8: validate, quantize the vector once, then one dot per
 * row.  `quantized` needs K + K/16 bytes and `scales` K/32 floats; both are
 * outputs the caller may inspect, as in the reference. */
int oracle_matvec_q8(const int8_t *weights, int64_t rows, int64_t width, const float *vector,
    int64_t vector_size, float *values, int64_t values_size, int8_t *quantized,
    int64_t quantized_size, float *scales, int64_t scales_size)
{
    if (vector_size != width || values_size != rows || vector_size % 32 != 0 ||
        quantized_size < vector_size + 2 * ((vector_size + 31) / 32) ||
        scales_size < (vector_size + 31) / 32)
        return ORACLE_INVALID;
    const int64_t blocks = vector_size / 32;
    oracle_q8_quantize(vector, quantized, scales, vector_size);
    rows_loop(weights, quantized, scales, rows, blocks, values, rows >= 128);
    return ORACLE_OK;
}

/* gguf_tensor_matvec_pair_q8: two matrices of identical shape. */
int oracle_matvec_pair_q8(const int8_t *first, const int8_t *second, int64_t rows,
    int64_t width, int64_t second_rows, int64_t second_width, const float *vector,
    int64_t vector_size, float *values, int64_t values_size, float *other_values,
    int64_t other_size, int8_t *quantized, int64_t quantized_size, float *scales,
    int64_t scales_size)
{
    if (width != second_width || rows != second_rows || vector_size != width ||
        values_size != rows || other_size != second_rows || vector_size % 32 != 0 ||
        quantized_size < vector_size + 2 * ((vector_size + 31) / 32) ||
        scales_size < (vector_size + 31) / 32)
        return ORACLE_INVALID;
    const int64_t blocks = vector_size / 32;
    oracle_q8_quantize(vector, quantized, scales, vector_size);
    rows_loop(first, quantized, scales, rows, blocks, values, rows >= 128);
    rows_loop(second, quantized, scales, rows, blocks, other_values, rows >= 128);
    return ORACLE_OK;
}

/* gguf_tensor_matvec_triplet_q8: three matrices sharing K; the parallel
 * decision is taken on the total row count (fortai_gguf_runtime.f90:551). */
int oracle_matvec_triplet_q8(const int8_t *first, const int8_t *second, const int8_t *third,
    int64_t first_rows, int64_t second_rows, int64_t third_rows, int64_t width,
    int64_t second_width, int64_t third_width, const float *vector, int64_t vector_size,
    float *values, int64_t values_size, float *second_values, int64_t second_size,
    float *third_values, int64_t third_size, int8_t *quantized, int64_t quantized_size,
    float *scales, int64_t scales_size)
{
    if (width != second_width || width != third_width || vector_size != width ||
        values_size != first_rows || second_size != second_rows || third_size != third_rows ||
        vector_size % 32 != 0 ||
        quantized_size < vector_size + 2 * ((vector_size + 31) / 32) ||
        scales_size < (vector_size + 31) / 32)
        return ORACLE_INVALID;
    const int64_t blocks = vector_size / 32;
    oracle_q8_quantize(vector, quantized, scales, vector_size);
    const int parallel = first_rows + second_rows + third_rows >= 128;
    rows_loop(first, quantized, scales, first_rows, blocks, values, parallel);
    rows_loop(second, quantized, scales, second_rows, blocks, second_values, parallel);
    rows_loop(third, quantized, scales, third_rows, blocks, third_values, parallel);
    return ORACLE_OK;
}

/* Pre-quantized form used by the CUDA ABI (the caller quantizes first):
 * activation is `blocks` Q8_0 blocks; scales are re-read from its fp16 bytes,
 * which is the same float the quantizer returned. */
int oracle_matvec_q8_prequantized(const int8_t *weights, int64_t rows, int64_t blocks,
    const int8_t *activation, float *values)
{
    if (rows <= 0 || blocks <= 0) return ORACLE_INVALID;
    float scales_stack[1024];
    float *scales = scales_stack;
    if (blocks > 1024) return ORACLE_INVALID;
    for (int64_t b = 0; b < blocks; ++b)
        scales[b] = oracle_half_to_float(block_scale_bits(activation + b * Q8_BLOCK_BYTES));
    rows_loop(weights, activation, scales, rows, blocks, values, rows >= 128);
    return ORACLE_OK;
}

/* Batched (multi-token) product.  The reference evaluates one token per call
 * (src/models/qwen35/fortai_qwen35_cpu.f90:591), so a batch is by definition
 * `tokens` independent matvecs: output[t * rows + r]. */
int oracle_matmul_q8(const int8_t *weights, int64_t rows, int64_t width, const float *matrix,
    int64_t tokens, float *values, int8_t *quantized, float *scales)
{
    if (rows <= 0 || width <= 0 || width % 32 != 0 || tokens <= 0) return ORACLE_INVALID;
    const int64_t blocks = width / 32;
    for (int64_t t = 0; t < tokens; ++t) {
        int8_t *q = quantized + t * blocks * Q8_BLOCK_BYTES;
        float *s = scales + t * blocks;
        oracle_q8_quantize(matrix + t * width, q, s, width);
        rows_loop(weights, q, s, rows, blocks, values + t * rows, rows >= 128);
    }
    return ORACLE_OK;
}

/* ---- SiLU(gate) * up ------------------------------------------------------ */

/* The polynomial exponential of the AVX2 path (fortai_q8_dot.c:9-51), one lane.
 * `contract` selects whether each multiply-add pair is fused: the reference
 * source spells them as separate mul and add intrinsics, but GCC contracts
 * them into FMAs whenever the function is compiled for an FMA target, so both
 * roundings exist in the wild.  Tests accept either within 2e-5. */
static float poly_expf(float value, int contract)
{
    const float log2e = 1.44269504088896341f;
    const float ln2_hi = 0.693359375f;
    const float ln2_lo = -2.12194440e-4f;
    const float c[6] = {1.9875691500e-4f, 1.3981999507e-3f, 8.3334519073e-3f,
        4.1665795894e-2f, 1.6666665459e-1f, 5.0000001201e-1f};
    if (value > 88.3762626647949f) value = 88.3762626647949f;
    if (value < -88.3762626647949f) value = -88.3762626647949f;
    volatile float fx = contract ? fmaf(value, log2e, 0.5f) : (float)(value * log2e) + 0.5f;
    int32_t exponent = (int32_t)fx;                    /* cvttps2dq */
    if ((float)exponent > fx) --exponent;              /* floor */
    const float n = (float)exponent;
    volatile float r;
    if (contract) {
        r = fmaf(-n, ln2_hi, value);
        r = fmaf(-n, ln2_lo, r);
    } else {
        volatile float t = n * ln2_hi;
        r = value - t;
        t = n * ln2_lo;
        r = r - t;
    }
    volatile float z = r * r;
    volatile float p = c[0];
    for (int i = 1; i < 6; ++i) {
        if (contract) p = fmaf(p, r, c[i]);
        else { volatile float t = p * r; p = t + c[i]; }
    }
    if (contract) p = fmaf(p, z, r);
    else { volatile float t = p * z; p = t + r; }
    p = p + 1.0f;
    uint32_t bits = (uint32_t)(exponent + 0x7f) << 23;
    float pow2;
    memcpy(&pow2, &bits, sizeof pow2);
    return p * pow2;
}

/* fortai_silu_product (fortai_q8_dot.c:484-525): left[i] = silu(left[i]) * right[i].
 * Groups of eight use the polynomial exponential with the +-20 clamps; the
 * remainder (and any call with count < 8) uses libm expf without clamps. */
void oracle_silu_product(float *left, const float *right, int64_t count, int contract)
{
    int64_t i = 0;
    if (count >= 8) {
        for (; i + 8 <= count; i += 8) {
            for (int l = 0; l < 8; ++l) {
                const float x = left[i + l];
                float result = x / (1.0f + poly_expf(-x, contract));
                if (x < -20.0f) result = 0.0f;
                if (x > 20.0f) result = x;
                left[i + l] = result * right[i + l];
            }
        }
    }
    for (; i < count; ++i)
        left[i] = left[i] / (1.0f + expf(-left[i])) * right[i];
}

/* FFN as the reference composes it on the CPU
 * (src/models/qwen35/fortai_qwen35_cpu.f90:672-677): pair matvec of gate and
 * up, SiLU product in place, then the down matvec (which quantizes the hidden
 * vector again).  gate/up are `inner` x `hidden`, down is `hidden_out` x `inner`.
 * work_* hold `inner` floats; quantized/scales are sized for max(hidden, inner). */
int oracle_ffn_q8(const int8_t *gate, const int8_t *up, const int8_t *down, int64_t inner,
    int64_t hidden, int64_t hidden_out, const float *input, float *output, float *work_gate,
    float *work_up, int8_t *quantized, float *scales, int contract)
{
    if (inner <= 0 || hidden <= 0 || hidden_out <= 0 || inner % 32 || hidden % 32)
        return ORACLE_INVALID;
    const int64_t qmax = (hidden > inner ? hidden : inner);
    int code = oracle_matvec_pair_q8(gate, up, inner, hidden, inner, hidden, input, hidden,
        work_gate, inner, work_up, inner, quantized, qmax + qmax / 16, scales, qmax / 32);
    if (code != ORACLE_OK) return code;
    oracle_silu_product(work_gate, work_up, inner, contract);
    return oracle_matvec_q8(down, hidden_out, inner, work_gate, inner, output, hidden_out,
        quantized, qmax + qmax / 16, scales, qmax / 32);
}

/* ---- seeded synthetic inputs ---------------------------------------------- */

static inline uint64_t splitmix64(uint64_t *state)
{
    uint64_t z = (*state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

/* Fill `out[0..count)` with N(0, sigma) floats.  Element i depends only on
 * (seed, i / 2), so any sub-range can be regenerated independently (row shards
 * on different ranks produce the same matrix).  Box-Muller on two 53-bit
 * uniforms taken from splitmix64 seeded with seed * 2^32 + pair index. */
void oracle_fill_normal(float *out, int64_t first, int64_t count, uint64_t seed, float sigma)
{
#pragma omp parallel for schedule(static) if (count >= 1 << 16)
    for (int64_t k = 0; k < count; ++k) {
        const int64_t i = first + k;
        uint64_t state = (seed << 32) ^ (uint64_t)(i >> 1) * 0xd1342543de82ef95ull;
        const double u1 = ((double)(splitmix64(&state) >> 11) + 1.0) * (1.0 / 9007199254740992.0);
        const double u2 = (double)(splitmix64(&state) >> 11) * (1.0 / 9007199254740992.0);
        const double radius = sqrt(-2.0 * log(u1));
        const double angle = 6.283185307179586476925 * u2;
        out[k] = (float)(sigma * radius * ((i & 1) ? sin(angle) : cos(angle)));
    }
}

/* rows x width weights ~ N(0, sigma), quantized to Q8_0 with the reference
 * quantizer semantics; rows [first_row, first_row + rows) of the matrix whose
 * element (r, c) is sample r * width + c. */
void oracle_make_weights(int8_t *out, int64_t first_row, int64_t rows, int64_t width,
    uint64_t seed, float sigma)
{
#pragma omp parallel
    {
        float buffer[8192];
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            for (int64_t c0 = 0; c0 < width; c0 += 8192) {
                const int64_t n = width - c0 < 8192 ? width - c0 : 8192;
                const int64_t base = (first_row + r) * width + c0;
                for (int64_t k = 0; k < n; ++k) {
                    const int64_t i = base + k;
                    uint64_t state = (seed << 32) ^ (uint64_t)(i >> 1) * 0xd1342543de82ef95ull;
                    const double u1 = ((double)(splitmix64(&state) >> 11) + 1.0) *
                        (1.0 / 9007199254740992.0);
                    const double u2 = (double)(splitmix64(&state) >> 11) *
                        (1.0 / 9007199254740992.0);
                    buffer[k] = (float)(sigma * sqrt(-2.0 * log(u1)) *
                        ((i & 1) ? sin(6.283185307179586476925 * u2)
                                 : cos(6.283185307179586476925 * u2)));
                }
                oracle_q8_quantize(buffer, out + (r * (width / 32) + c0 / 32) * Q8_BLOCK_BYTES,
                    NULL, n);
            }
        }
    }
}

/* xorshift32 fixture of the reference micro-benchmark
 * (backend/cuda/fortai_q8_bench_spec.h:16-21, 68-80): per block one draw for
 * the scale, 0.004 + 0.012 * (r & 1023) / 1023 stored as fp16, then 32 draws
 * for quants (r % 255) - 127.  With per_row == 0 only one row is written. */
static inline uint32_t xorshift32(uint32_t *state)
{
    uint32_t s = *state;
    s ^= s << 13;
    s ^= s >> 17;
    s ^= s << 5;
    return *state = s;
}

/* Truncating-with-round-bit half conversion used by that fixture
 * (fortai_q8_bench_spec.h:23-45): rounds half up on bit 12, not to even. */
static uint16_t fixture_float_to_half(float value)
{
    uint32_t bits;
    memcpy(&bits, &value, sizeof bits);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exponent = (int32_t)((bits >> 23) & 0xffu) - 127 + 15;
    uint32_t fraction = bits & 0x007fffffu;
    if (exponent <= 0) {
        if (exponent < -10) return (uint16_t)sign;
        fraction = (fraction | 0x00800000u) >> (uint32_t)(1 - exponent);
        if (bits & 0x00001000u) fraction += 0x00002000u;
        return (uint16_t)(sign | (fraction >> 13));
    }
    if (exponent >= 31) return (uint16_t)(sign | 0x7c00u);
    if (fraction & 0x00001000u) {
        fraction += 0x00002000u;
        if (fraction & 0x00800000u) {
            fraction = 0;
            if (++exponent >= 31) return (uint16_t)(sign | 0x7c00u);
        }
    }
    return (uint16_t)(sign | ((uint32_t)exponent << 10) | (fraction >> 13));
}

void oracle_fixture_fill_q8(uint8_t *data, int rows, int blocks, uint32_t seed, int per_row)
{
    for (int row = 0; row < (per_row ? rows : 1); ++row) {
        for (int b = 0; b < blocks; ++b) {
            uint8_t *dst = data + ((size_t)row * blocks + b) * Q8_BLOCK_BYTES;
            const float scale = 0.004f + 0.012f * (float)(xorshift32(&seed) & 1023u) / 1023.0f;
            const uint16_t bits = fixture_float_to_half(scale);
            dst[0] = (uint8_t)(bits & 0xffu);
            dst[1] = (uint8_t)(bits >> 8);
            for (int i = 0; i < Q8_BLOCK_ELEMS; ++i)
                dst[2 + i] = (uint8_t)((int)(xorshift32(&seed) % 255u) - 127);
        }
    }
}

/* Scalar oracle of that fixture (fortai_q8_bench_spec.h:82-101):
 * result += half(ws) * half(as) * (float)dot, blocks ascending. */
void oracle_fixture_matvec(const uint8_t *weights, const uint8_t *activation, int rows,
    int blocks, float *out)
{
#pragma omp parallel for schedule(static) if (rows >= 128)
    for (int row = 0; row < rows; ++row) {
        volatile float result = 0.0f;
        for (int b = 0; b < blocks; ++b) {
            const int8_t *w = (const int8_t *)weights + ((size_t)row * blocks + b) * Q8_BLOCK_BYTES;
            const int8_t *a = (const int8_t *)activation + (size_t)b * Q8_BLOCK_BYTES;
            int32_t dot = 0;
            for (int i = 0; i < Q8_BLOCK_ELEMS; ++i)
                dot += (int32_t)w[2 + i] * (int32_t)a[2 + i];
            volatile float term = oracle_half_to_float(block_scale_bits(w)) *
                oracle_half_to_float(block_scale_bits(a));
            term = term * (float)dot;
            result = result + term;
        }
        out[row] = result;
    }
}

int oracle_thread_count(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int threads)
{
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}
