/* Row-loop driver around the REFERENCE's own compiled arithmetic.
 * TEST AND CPU-BASELINE INFRASTRUCTURE ONLY - never linked into the shipped library.
 *
 * The reference's Q8_0 arithmetic is C (src/backend/cpu/fortai_q8_dot.c) and is
 * compiled unchanged, from where it lies, by oracle/Makefile.  The loop that
 * calls it once per output row is Fortran in the reference
 * (src/fortai_gguf_runtime.f90:449-464) and no Fortran compiler exists in this
 * image, so that loop - and only that loop - is restated here: quantize the
 * vector once, then `fortai_q8_dot` per row, serial below 128 rows, OpenMP
 * `schedule(static)` otherwise.
 */
#include <stdint.h>

#ifdef _OPENMP
#include <omp.h>
#endif

void fortai_q8_quantize(const float *input, int8_t *output, float *scales, int64_t count);
float fortai_q8_dot(const int8_t *weights, const int8_t *quantized, const float *scales,
    int64_t row, int64_t block_count);
void fortai_silu_product(float *left, const float *right, int64_t count);

/* gguf_tensor_matvec_q8 without the shape checks (callers pass agreed sizes). */
void ref_matvec_q8(const int8_t *weights, int64_t rows, int64_t width, const float *vector,
    float *values, int8_t *quantized, float *scales)
{
    const int64_t blocks = width / 32;
    fortai_q8_quantize(vector, quantized, scales, width);
    if (rows < 128) {
        for (int64_t row = 0; row < rows; ++row)
            values[row] = fortai_q8_dot(weights, quantized, scales, row, blocks);
    } else {
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < rows; ++row)
            values[row] = fortai_q8_dot(weights, quantized, scales, row, blocks);
    }
}

/* Rows loop only, for an activation that is already quantized. */
void ref_rows_q8(const int8_t *weights, int64_t rows, int64_t blocks, const int8_t *quantized,
    const float *scales, float *values)
{
    if (rows < 128) {
        for (int64_t row = 0; row < rows; ++row)
            values[row] = fortai_q8_dot(weights, quantized, scales, row, blocks);
    } else {
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < rows; ++row)
            values[row] = fortai_q8_dot(weights, quantized, scales, row, blocks);
    }
}

/* `tokens` independent matvecs (the reference has no batched call). */
void ref_matmul_q8(const int8_t *weights, int64_t rows, int64_t width, const float *matrix,
    int64_t tokens, float *values, int8_t *quantized, float *scales)
{
    for (int64_t t = 0; t < tokens; ++t)
        ref_matvec_q8(weights, rows, width, matrix + t * width, values + t * rows, quantized,
            scales);
}

/* Repeat the matvec `repeats` times and return the last checksum, for timing. */
double ref_matvec_q8_repeat(const int8_t *weights, int64_t rows, int64_t width,
    const float *vector, float *values, int8_t *quantized, float *scales, int repeats)
{
    double checksum = 0.0;
    for (int r = 0; r < repeats; ++r) {
        ref_matvec_q8(weights, rows, width, vector, values, quantized, scales);
        checksum = 0.0;
        for (int64_t row = 0; row < rows; ++row) checksum += values[row];
    }
    return checksum;
}

int ref_thread_count(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* The reference's own thread policy is "all cores" (tools/build_native.sh:7-9 exports
 * OMP_NUM_THREADS=$(nproc)); a launcher that forces OMP_NUM_THREADS=1 on its children
 * (torch.distributed.run does) would otherwise time this baseline on one thread. */
void ref_set_threads(int threads)
{
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

int ref_uses_avx2(void)
{
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("f16c");
}
