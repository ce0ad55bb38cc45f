/* GGUF v3 reader behind a C ABI: the on-disk side of the Q8_0 path.
 *
 * Restates, as host C++ over a memory-mapped file, what the reference's Fortran module
 * does with stream reads into allocated arrays (src/fortai_gguf_runtime.f90):
 *   gguf_file_t%open        :106-197   header, metadata, tensor index, data offsets
 *   find_meta / find_tensor :230-258
 *   meta_int / meta_real    :260-290   (integer kinds only / real kinds only, else the default)
 *   gguf_tensor_t%value     :292-325   F32, F16, Q8_0 element decode
 *   gguf_tensor_t%get_row   :327-349
 *   tensor_bytes            :739-762   F32 4/elem, F16 2/elem, Q8_0 34 bytes per 32, width % 32
 *   gguf_fp16_to_real       :770-789   (exponent 31 decodes to the largest finite float)
 * The reference has no C interface for this (its callers are Fortran); these entry points
 * are what a C or Fortran bind(C) caller would use instead, and what lets real GGUF
 * tensors reach fortai_cuda_q8_weights_upload without a Fortran runtime.
 *
 * Return codes are the reference's status codes (src/fortai_status.f90:6-10):
 * 0 OK, 1 INVALID, 2 UNSUPPORTED, 3 IO_ERROR, 4 OUT_OF_MEMORY; the messages are the
 * reference's own strings.  Tensor data is never copied: pointers returned by
 * fortai_gguf_tensor_data point into the mapping and stay valid until close.  Not
 * thread-safe for concurrent open/close of the same handle; reads are. */
#ifndef FORTAI_GGUF_B200_H
#define FORTAI_GGUF_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FORTAI_GGUF_OK 0
#define FORTAI_GGUF_INVALID 1
#define FORTAI_GGUF_UNSUPPORTED 2
#define FORTAI_GGUF_IO_ERROR 3
#define FORTAI_GGUF_OUT_OF_MEMORY 4

#define FORTAI_GGML_TYPE_F32 0
#define FORTAI_GGML_TYPE_F16 1
#define FORTAI_GGML_TYPE_Q8_0 8

typedef struct fortai_gguf_file fortai_gguf_file;
struct fortai_cuda_q8_context;
struct fortai_cuda_q8_weights;

/* Opens and indexes a GGUF v3 file.  On failure *file is NULL and, if `message` is not
 * NULL, it receives the reason (truncated to message_bytes - 1 characters). */
int fortai_gguf_open(const char *path, fortai_gguf_file **file, char *message,
    size_t message_bytes);
/* Accepts NULL. */
void fortai_gguf_close(fortai_gguf_file *file);

int32_t fortai_gguf_version(const fortai_gguf_file *file);
int64_t fortai_gguf_tensor_count(const fortai_gguf_file *file);
int64_t fortai_gguf_metadata_count(const fortai_gguf_file *file);
/* general.alignment (32 when absent or not positive) and the file offset of the data area. */
int64_t fortai_gguf_alignment(const fortai_gguf_file *file);
int64_t fortai_gguf_data_start(const fortai_gguf_file *file);

/* Zero-based index, or -1. */
int64_t fortai_gguf_find_meta(const fortai_gguf_file *file, const char *key);
int64_t fortai_gguf_find_tensor(const fortai_gguf_file *file, const char *name);

/* Key and GGUF value type (0..12) of metadata entry `index`; NULL / -1 out of range. */
const char *fortai_gguf_meta_key(const fortai_gguf_file *file, int64_t index);
int32_t fortai_gguf_meta_type(const fortai_gguf_file *file, int64_t index);
/* Integer kinds (u8..i64) give their value, anything else or a missing key the default. */
int64_t fortai_gguf_meta_int(const fortai_gguf_file *file, const char *key, int64_t fallback);
/* float32 / float64 give their value (as float), anything else the default. */
float fortai_gguf_meta_real(const fortai_gguf_file *file, const char *key, float fallback);
/* String value (not NUL-terminated in the file: *length receives its size), or NULL. */
const char *fortai_gguf_meta_string(const fortai_gguf_file *file, const char *key,
    int64_t *length);
/* bool value, or `fallback`. */
int fortai_gguf_meta_bool(const fortai_gguf_file *file, const char *key, int fallback);
/* Arrays of 32- or 64-bit integers are kept (as int64); other arrays are skipped, as in
 * the reference.  Returns the element count (or -1) and copies up to `capacity` values. */
int64_t fortai_gguf_meta_int_array(const fortai_gguf_file *file, const char *key,
    int64_t *values, int64_t capacity);

/* Index entry of tensor `index`: name, ggml type, rank (1..4), shape (shape[0] is the
 * contiguous dimension, as stored), offset inside the data area and size in bytes.  Any
 * out-pointer may be NULL. */
int fortai_gguf_tensor_info(const fortai_gguf_file *file, int64_t index, const char **name,
    int32_t *type, int32_t *rank, int64_t shape[4], int64_t *file_offset, int64_t *byte_count);
/* The tensor's bytes inside the mapping (NULL out of range). */
const void *fortai_gguf_tensor_data(const fortai_gguf_file *file, int64_t index);
/* Element `element` (zero-based, storage order) decoded to float; 0 when out of range or
 * of an unsupported type. */
float fortai_gguf_tensor_value(const fortai_gguf_file *file, int64_t index, int64_t element);
/* Row `row` (zero-based) of a rank-2 tensor, shape[0] floats. */
int fortai_gguf_tensor_get_row(const fortai_gguf_file *file, int64_t index, int64_t row,
    float *values, int64_t count);

/* A rank-2 Q8_0 tensor (shape[0] = width, shape[1] = rows) straight from the mapping into a
 * weights handle of `context`: rows [first_row, first_row + row_count) (row_count 0 = all
 * from first_row), i.e. a row shard is a byte range of the file.  Returns the reference
 * status codes; a CUDA-side failure is UNSUPPORTED with the text in the context's
 * last_error, as the Fortran wrappers report it. */
int fortai_gguf_upload_q8(const fortai_gguf_file *file, int64_t index,
    struct fortai_cuda_q8_context *context, int64_t first_row, int64_t row_count,
    struct fortai_cuda_q8_weights **weights);

#ifdef __cplusplus
}
#endif

#endif
