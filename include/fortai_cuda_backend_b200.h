/* C ABI of the B200 (sm_100a) Q8_0 backend.
 *
 * Part 1 declares, symbol for symbol, the interface that the reference's
 * Fortran wrapper binds with ISO_C_BINDING (reference:
 * backend/cuda/fortai_cuda_backend.h:22-152, bound at
 * src/backend/cuda/fortai_backend_cuda.f90:67-414).  A program that links the
 * reference backend object links this library instead without source changes.
 *
 * Part 2 declares entry points that the reference does not have (batched
 * prefill, fp32 host convenience calls, shard uploads, peer-output GEMV,
 * parity probes).  They follow the same conventions.
 *
 * Conventions (reference: backend/cuda/fortai_cuda_backend.cu:42-52, 805-850):
 *  - every function returns FORTAI_CUDA_OK, FORTAI_CUDA_INVALID (bad argument or
 *    shape; nothing was enqueued) or FORTAI_CUDA_RUNTIME_ERROR (a CUDA call or a
 *    device-side wait failed; fortai_cuda_q8_last_error gives the text);
 *  - a context owns one device, one stream, its events and its scratch; it is
 *    not thread-safe; weights and layer handles belong to the context that made
 *    them and must be destroyed before it;
 *  - "host" calls block until the result is in host memory; "device" calls only
 *    enqueue on the context's stream;
 *  - device fp32 activation pointers must be 16-byte aligned and device Q8_0
 *    activation pointers 2-byte aligned (anything from device_buffer_create is);
 *    a misaligned pointer is reported as RUNTIME_ERROR, not dereferenced;
 *  - a Q8_0 block is 34 bytes: little-endian binary16 scale, then 32 int8.
 *    Weight matrices arrive as rows x (width/32) blocks, row-major.  The device
 *    copy is re-laid-out at upload (the handle is opaque), so a weights handle
 *    cannot be reinterpreted as raw GGUF bytes on the device.
 */
#ifndef FORTAI_CUDA_BACKEND_B200_H
#define FORTAI_CUDA_BACKEND_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fortai_cuda_q8_context fortai_cuda_q8_context;
typedef struct fortai_cuda_q8_weights fortai_cuda_q8_weights;
typedef struct fortai_cuda_qwen35_recurrent fortai_cuda_qwen35_recurrent;
typedef struct fortai_cuda_qwen35_attention fortai_cuda_qwen35_attention;

#ifndef FORTAI_CUDA_BACKEND_H   /* the reference header defines the same values */
enum {
    FORTAI_CUDA_OK = 0,
    FORTAI_CUDA_INVALID = 1,
    FORTAI_CUDA_RUNTIME_ERROR = 2
};
#endif

/* ======================================================================= *
 * Part 1 - the reference interface                                          *
 * ======================================================================= */

/* reference header :22-23, implementation backend.cu:805-850 */
int fortai_cuda_q8_context_create(int device, fortai_cuda_q8_context **context);
int fortai_cuda_q8_context_destroy(fortai_cuda_q8_context *context);

/* reference header :24-27, backend.cu:852-893 (device-side position word and
 * CUDA-graph capture of the context's stream) */
int fortai_cuda_q8_context_set_position(fortai_cuda_q8_context *context, int position);
int fortai_cuda_q8_context_capture_begin(fortai_cuda_q8_context *context);
int fortai_cuda_q8_context_capture_end(fortai_cuda_q8_context *context);
int fortai_cuda_q8_context_graph_launch(fortai_cuda_q8_context *context);

/* reference header :29-32, backend.cu:895-931.  host_weights holds at least
 * rows * (width/32) * 34 bytes in GGUF Q8_0 order; width % 32 == 0. */
int fortai_cuda_q8_weights_upload(fortai_cuda_q8_context *context, const void *host_weights,
    size_t weight_bytes, int rows, int width, fortai_cuda_q8_weights **weights);
int fortai_cuda_q8_weights_destroy(fortai_cuda_q8_weights *weights);

/* reference header :36-45, backend.cu:933-990.  upload and download block;
 * upload_ptr only enqueues the copy. */
int fortai_cuda_q8_device_buffer_create(fortai_cuda_q8_context *context, size_t bytes,
    void **device_buffer);
int fortai_cuda_q8_device_buffer_destroy(fortai_cuda_q8_context *context, void *device_buffer);
int fortai_cuda_q8_device_buffer_upload(fortai_cuda_q8_context *context, void *device_buffer,
    const void *host_data, size_t bytes);
int fortai_cuda_q8_device_buffer_upload_ptr(fortai_cuda_q8_context *context, void *device_buffer,
    const void *host_data, size_t bytes);
int fortai_cuda_q8_device_buffer_download(fortai_cuda_q8_context *context, void *host_data,
    const void *device_buffer, size_t bytes);

/* reference header :49-51, backend.cu:992-1011.  device_activation is a Q8_0
 * vector (width/32 blocks of 34 bytes) in device memory; device_output receives
 * `rows` floats; blocks until done; kernel_ms is the kernel alone. */
int fortai_cuda_q8_matvec_resident(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    float *kernel_ms);

/* reference header :52-54, backend.cu:1013-1039.  fp32 activation in device
 * memory; quantization to Q8_0 happens on the device; enqueue only. */
int fortai_cuda_q8_matvec_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements);

/* reference header :55-57, backend.cu:1041-1055: dequantize one weight row. */
int fortai_cuda_qwen35_embedding_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, int64_t token_id, void *device_output,
    size_t output_elements);

/* reference header :59-67, backend.cu:1057-1095 */
int fortai_cuda_qwen35_copy_device(fortai_cuda_q8_context *context, const void *device_input,
    void *device_output, size_t bytes);
int fortai_cuda_qwen35_add_device(fortai_cuda_q8_context *context, const void *device_left,
    const void *device_right, void *device_output, size_t elements);
int fortai_cuda_qwen35_rms_norm_device(fortai_cuda_q8_context *context, const void *device_input,
    const void *device_weights, void *device_output, size_t elements, float epsilon);

/* reference header :72-75, backend.cu:1097-1129.  Q8_0 activation and fp32
 * output live in host memory; elapsed_ms includes both transfers. */
int fortai_cuda_q8_matvec_host(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *host_activation, size_t activation_bytes,
    float *host_output, size_t output_bytes, float *elapsed_ms);

/* reference header :79-100, backend.cu:249-315, 1131-1187.  One activation
 * upload, several matrices with the same width.  The contiguous form returns
 * the three outputs back to back and is accepted only for width < 4096, the
 * condition under which the reference fuses them (backend.cu:257-258). */
int fortai_cuda_q8_matvec_host_pair(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const void *host_activation, size_t activation_bytes, float *first_output,
    size_t first_output_bytes, float *second_output, size_t second_output_bytes,
    float *elapsed_ms);
int fortai_cuda_q8_matvec_host_triplet(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const fortai_cuda_q8_weights *third_weights, const void *host_activation,
    size_t activation_bytes, float *first_output, size_t first_output_bytes,
    float *second_output, size_t second_output_bytes, float *third_output,
    size_t third_output_bytes, float *elapsed_ms);
int fortai_cuda_q8_matvec_host_triplet_contiguous(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *first_weights, const fortai_cuda_q8_weights *second_weights,
    const fortai_cuda_q8_weights *third_weights, const void *host_activation,
    size_t activation_bytes, float *host_output, size_t host_output_bytes, float *elapsed_ms);

/* reference header :102-114, backend.cu:1189-1296.  out = down * Q8(silu(gate*x) .* (up*x));
 * gate and up are inner x hidden, down is hidden_out x inner. */
int fortai_cuda_q8_ffn_host(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *host_activation,
    size_t activation_bytes, float *host_output, size_t output_bytes, float *elapsed_ms);
int fortai_cuda_q8_ffn_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements);

/* reference header :120-139, backend.cu:1298-1567 (gated-delta-net layer) */
int fortai_cuda_qwen35_recurrent_create(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *qkv_weights, const fortai_cuda_q8_weights *gate_weights,
    const fortai_cuda_q8_weights *alpha_weights, const fortai_cuda_q8_weights *beta_weights,
    const fortai_cuda_q8_weights *output_weights, const void *conv_weights,
    size_t conv_weight_bytes, int conv_size, int conv_kernel, const void *ssm_a,
    size_t ssm_a_bytes, const void *ssm_dt, size_t ssm_dt_bytes, const void *ssm_norm,
    size_t ssm_norm_bytes, int state_size, int key_heads, int value_heads, int head_size,
    int inner_size, float norm_epsilon, fortai_cuda_qwen35_recurrent **layer);
int fortai_cuda_qwen35_recurrent_destroy(fortai_cuda_qwen35_recurrent *layer);
int fortai_cuda_qwen35_recurrent_reset(fortai_cuda_qwen35_recurrent *layer);
int fortai_cuda_qwen35_recurrent_run(fortai_cuda_qwen35_recurrent *layer,
    const void *host_activation, size_t activation_bytes, float *host_output,
    size_t output_bytes, float *elapsed_ms);
int fortai_cuda_qwen35_recurrent_run_device(fortai_cuda_qwen35_recurrent *layer,
    const void *device_activation, size_t activation_elements, void *device_output,
    size_t output_elements);

/* reference header :141-154, backend.cu:1569-1731 (single-query attention layer) */
int fortai_cuda_qwen35_attention_create(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *query_weights, const fortai_cuda_q8_weights *key_weights,
    const fortai_cuda_q8_weights *value_weights, const fortai_cuda_q8_weights *output_weights,
    const void *query_norm, size_t query_norm_bytes, const void *key_norm,
    size_t key_norm_bytes, int heads, int key_value_heads, int head_size, int value_size,
    int max_context, int rope_dimension, float rope_base, float norm_epsilon,
    fortai_cuda_qwen35_attention **layer);
int fortai_cuda_qwen35_attention_destroy(fortai_cuda_qwen35_attention *layer);
int fortai_cuda_qwen35_attention_reset(fortai_cuda_qwen35_attention *layer);
int fortai_cuda_qwen35_attention_run_device(fortai_cuda_qwen35_attention *layer,
    const void *device_activation, size_t activation_elements, int position,
    void *device_output, size_t output_elements);

/* reference header :156, backend.cu:1733-1736 */
const char *fortai_cuda_q8_last_error(const fortai_cuda_q8_context *context);

/* ======================================================================= *
 * Part 2 - entry points without a counterpart in the reference              *
 * ======================================================================= */

/* Context on a stream the caller owns (cudaStream_t passed as void*; NULL is
 * the legacy default stream).  Lets a host that already has a stream - for
 * example one that also carries NCCL collectives - order this backend's work
 * on it.  The stream is borrowed, never destroyed here. */
int fortai_cuda_q8_context_create_on_stream(int device, void *stream,
    fortai_cuda_q8_context **context);
/* The context's stream as a cudaStream_t. */
void *fortai_cuda_q8_context_stream(const fortai_cuda_q8_context *context);
/* Kernels launched through this context since it was created. */
uint64_t fortai_cuda_q8_context_launch_count(const fortai_cuda_q8_context *context);
/* Blocks until the stream is idle, then reports any device-side wait that gave
 * up (bounded mbarrier waits in the staged kernels) as RUNTIME_ERROR. */
int fortai_cuda_q8_context_synchronize(fortai_cuda_q8_context *context);
/* Tuning knobs, by name: "gemv_variant" (0 = automatic: slice kernel for few long rows,
 * register-pipelined kernel where the width is one of its granule counts, else the
 * half-block-per-lane kernel; 1 = always the half-block-per-lane kernel), "gemv_split" (warps
 * that share a row in the slice kernel: 0 = automatic, 1 = never, 4, 8), "gemv_ctas_per_sm",
 * "gemv_depth", "gemv_balance", "host_flush_rows" and "peer_flush_rows" (rows per store group
 * of a GEMV that writes a page-locked host vector / peers' vectors: a power of two up to 32),
 * "gemv_rows_per_warp", "mmq_min_tokens" (first token count that
 * goes to the tcgen05 prefill kernel, default 65: up to 64 tokens the few-token kernel is faster), "prefill_kind" (0 = kind::f16 MMAs with the
 * activation scale folded into the operand, the default; 1 = kind::i8 MMAs scaled per block on
 * the CUDA cores, the kernel that also serves the block-dot probe), "peer_wait_clocks_millions".
 * Zero means automatic.  Unknown names return INVALID. */
int fortai_cuda_q8_context_set_option(fortai_cuda_q8_context *context, const char *name,
    int value);

/* Shape of a weights handle. */
int fortai_cuda_q8_weights_shape(const fortai_cuda_q8_weights *weights, int *rows, int *width);

/* Upload only blocks [first_block, first_block + block_count) of every row of a
 * rows x width host matrix: the K-slice that one rank of a column-sharded
 * (reduce-after) projection owns.  The handle reports width = 32 * block_count. */
int fortai_cuda_q8_weights_upload_columns(fortai_cuda_q8_context *context,
    const void *host_weights, size_t weight_bytes, int rows, int width, int first_block,
    int block_count, fortai_cuda_q8_weights **weights);

/* fp32 -> Q8_0 on the device: `elements` floats (a multiple of 32) become
 * elements/32 blocks of 34 bytes, byte-identical to the reference CPU quantizer
 * (src/backend/cpu/fortai_q8_dot.c:153-198).  Enqueue only. */
int fortai_cuda_q8_quantize_device(fortai_cuda_q8_context *context, const void *device_input,
    size_t elements, void *device_output, size_t output_bytes);

/* Parity probe: the exact int32 dot of every (row, block) pair, rows x (width/32) values.
 * It runs the half-block-per-lane GEMV kernel with an epilogue that joins a block's two
 * half dots; the default register-pipelined kernel forms the same two exact half-block
 * dots per lane but scales each on its own and never materialises their sum, so on that
 * kernel the integer arithmetic is covered through this sibling and the fp32 result through
 * the 1e-5 * L2 bound.  Enqueue only. */
int fortai_cuda_q8_block_dots_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    size_t output_elements);

/* fortai_cuda_q8_matvec_resident (backend/cuda/fortai_cuda_backend.h:56-58) without its event
 * pair and wait: device Q8_0 activation (width/32 blocks of 34 bytes) in, `rows` floats out.
 * Enqueue only. */
int fortai_cuda_q8_matvec_device_q8(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, void *device_output,
    size_t output_elements);

/* Host fp32 in, host fp32 out: H2D of `activation_elements` floats, quantize and
 * GEMV in one kernel, D2H of `rows` floats; blocks; elapsed_ms covers all of it. */
int fortai_cuda_q8_matvec_host_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms);

/* Batched product (batched decode, speculative decoding, prefill): `tokens` rows of
 * `width` floats in, tokens x rows floats out (token-major: out[t * rows + r]).  Each
 * token row is quantized to Q8_0 exactly as a single activation would be.  2..64 tokens
 * stream the weights once through a warp-level int8 MMA kernel, more go to the tcgen05
 * kernel; the reference runs one GEMV per token.  Enqueue only. */
int fortai_cuda_q8_matmul_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements);
/* Same with a pre-quantized activation (tokens x width/32 blocks of 34 bytes);
 * blocks; kernel_ms is the product kernel alone. */
int fortai_cuda_q8_matmul_resident(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, float *kernel_ms);
/* Host fp32 in/out form of the batched product; blocks. */
int fortai_cuda_q8_matmul_host_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const float *host_activation, int tokens,
    float *host_output, size_t output_bytes, float *elapsed_ms);
/* Parity probe for the batched path: int32 dot of every (token, row, block),
 * out[(t * rows + r) * blocks + b], taken from the tensor-core accumulators. */
int fortai_cuda_q8_matmul_block_dots_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements);

/* Measured tensor-core peak of this GPU, the denominator for the prefill kernel's
 * utilisation: a bare tcgen05.mma loop (128 x 256 tiles, operands resident in shared memory,
 * nothing drained) on every SM, `iterations` commits of four MMAs each.  kind 0 = kind::i8
 * (int8 TOPS), 1 = kind::f16 (binary16 TFLOPS).  No counterpart in the reference; blocks. */
int fortai_cuda_tensor_peak(fortai_cuda_q8_context *context, int kind, int iterations,
    float *tera_ops_per_second, float *elapsed_ms);

/* FFN for `tokens` activations at once: out[t] = down . Q8(silu(gate . x[t]) * (up . x[t])),
 * x and out token-major fp32 in device memory.  Same shape rules as
 * fortai_cuda_q8_ffn_device (backend/cuda/fortai_cuda_backend.cu:1247-1296), which it
 * equals token by token.  Enqueue only. */
int fortai_cuda_q8_ffn_batch_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation, int tokens,
    void *device_output, size_t output_elements);

/* Residual-stream steps.  The reference's caller wraps every layer object and FFN in
 * copy -> rms_norm -> ... -> add (src/models/qwen35/fortai_qwen35_cpu.f90:713-747, 764-800);
 * these take the residual stream x itself (fp32, device, 16-byte aligned, `elements` =
 * hidden size) and do x <- x + f(rms_norm(x) * norm_weights) in place: the norm runs in the
 * first GEMV's prologue, the add in the last GEMV's epilogue.  norm_weights: `elements`
 * floats in device memory, 16-byte aligned; epsilon > 0.  Enqueue only. */
int fortai_cuda_qwen35_recurrent_step_device(fortai_cuda_qwen35_recurrent *layer, void *device_x,
    size_t elements, const void *device_norm_weights, float epsilon);
int fortai_cuda_qwen35_attention_step_device(fortai_cuda_qwen35_attention *layer, void *device_x,
    size_t elements, int position, const void *device_norm_weights, float epsilon);
int fortai_cuda_q8_ffn_step_device(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, void *device_x, size_t elements,
    const void *device_norm_weights, float epsilon);
/* out = weights . Q8(rms_norm(x) * norm_weights): the output head (:749-762) in one launch. */
int fortai_cuda_q8_matvec_norm_device_f32(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_x, size_t elements,
    const void *device_norm_weights, float epsilon, void *device_output,
    size_t output_elements);

/* Row-sharded GEMV whose epilogue stores this rank's slice into every rank's
 * output vector: peer_outputs[p] is rank p's full-length output buffer (device
 * pointers valid on this device, e.g. from symmetric memory); the slice is
 * written at element offset `first_row`.  Enqueue only; the caller provides the
 * cross-rank barrier before the outputs are read. */
int fortai_cuda_q8_matvec_device_f32_peers(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_outputs, int peer_count, size_t first_row,
    size_t output_elements);

/* The same with the all-gather fused into the kernel: peer_flags[p] is rank p's flag array
 * (peer_count 32-bit words, zero-initialised once, e.g. in symmetric memory); word
 * [my_rank] of every array belongs to this rank.  When the launch completes, every rank's
 * slice is in this rank's output vector.  Two protocols, chosen by option
 * "peer_publish_per_cta" (all ranks must use the same one, on flag arrays of its own):
 *   0 (default)  every CTA publishes its stores and counts itself; the rank's last CTA
 *     writes a per-context call number into its word in every rank's array and waits - for
 *     about a second at most - until every word of its own array has reached that number.
 *     The number is a launch argument, so the call cannot be captured into a CUDA graph (a
 *     replay would not wait): during capture it returns INVALID with a message.
 *   1  every CTA, once its rows are stored, adds its share of 2^20 to the rank's word in
 *     every array, so a launch adds exactly 2^20 per sender, and one CTA waits until every
 *     word of the rank's own array has reached (calls made on these arrays) * 2^20 modulo
 *     2^32.  The count is read from the rank's own word: the call may be captured and
 *     replayed.  Measured 2-3 us slower per call on two B200s than protocol 0.
 * Every rank must make the same sequence of these calls, each on its own GPU (the kernels
 * wait on one another).  A wait that runs out is reported as RUNTIME_ERROR by the next
 * synchronizing call (option "peer_wait_clocks_millions" sets the limit, default 2000).
 * The flags say that a slice has ARRIVED, not that it has been CONSUMED: a rank that runs
 * ahead stores call n+1's slice into a peer's vector while that peer may still read call
 * n's result.  Alternate two output vectors between consecutive calls, or put a cross-rank
 * barrier between reading the result and the next call.  Enqueue only. */
int fortai_cuda_q8_matvec_device_f32_allgather(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_outputs, void *const *peer_flags,
    int peer_count, int my_rank, size_t first_row, size_t output_elements);

/* The all-gather matvec without flags: a result travels to the other ranks as one aligned
 * 8-byte store of (value bits, call number), which arrives whole, so the sender fences nothing
 * and raises no flag, and the receiver knows a value by the number beside it (the scheme of
 * low-latency collectives).  peer_pairs[p] is rank p's pair array: 2 * output_elements pairs of
 * 8 bytes, 8-byte aligned, zeroed once, reachable from every rank; its two halves alternate
 * between consecutive calls.  After its rows, every CTA collects the other ranks' slices from
 * this rank's own pair array into device_output (output_elements floats, this rank's memory;
 * the own slice is stored there directly).  Waits are bounded as in the flag form (same option,
 * same RUNTIME_ERROR).  Every rank must make the same sequence of these calls, each on its own
 * GPU, on pair arrays used for nothing else.  Not capturable (INVALID during capture).
 * Measured on the lm_head: see the scaling profile.  Enqueue only. */
int fortai_cuda_q8_matvec_device_f32_allgather_ll(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *weights, const void *device_activation,
    size_t activation_elements, void *const *peer_pairs, int peer_count, int my_rank,
    size_t first_row, void *device_output, size_t output_elements);

/* The FFN of fortai_cuda_q8_ffn_device for ranks that hold gate/up row shards and the
 * matching column shard of down, with the sum over ranks inside the call (no reference
 * counterpart: the reference is single-GPU).  peer_pairs[p] is rank p's pair array:
 * 2 * peer_count * hidden pairs of 8 bytes, 8-byte aligned, zeroed once, reachable from every
 * rank (peer access or symmetric memory), used for nothing else.  The down GEMV stores this
 * rank's partial vector as (value bits, call number) pairs into slot my_rank of every rank's
 * array (the two halves of the array alternate between consecutive calls), and its tail adds
 * the slots in rank order into device_output as they arrive: no flags, no fence, no collective
 * library, and every rank gets the same bits.  Waits are bounded as in the all-gather matvec
 * (same option, same RUNTIME_ERROR).  Every rank must make the same sequence of pair-exchanging
 * calls, each on its own GPU.  Not capturable.  Enqueue only. */
int fortai_cuda_q8_ffn_device_allreduce(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *const *peer_pairs, int peer_count, int my_rank,
    void *device_output, size_t output_elements);

/* ----------------------------------------------------------------------- *
 * Device groups: the sharded path for hosts that drive several GPUs of one box from one
 * thread (the reference is single-GPU, ROADMAP.md:31; its only multi-device hook is the
 * device index of fortai_cuda_q8_context_create, reference header :22).  A group owns one
 * context per device, enables peer access between them and keeps, on every device, a result
 * vector and a flag array that the others store into.  Same return codes as everything
 * above; messages through fortai_cuda_q8_group_last_error.  Not thread-safe.
 * ----------------------------------------------------------------------- */
typedef struct fortai_cuda_q8_group fortai_cuda_q8_group;
typedef struct fortai_cuda_q8_group_weights fortai_cuda_q8_group_weights;

/* `count` distinct device indices (1..8), every pair peer-accessible. */
int fortai_cuda_q8_group_create(const int *devices, int count, fortai_cuda_q8_group **group);
int fortai_cuda_q8_group_destroy(fortai_cuda_q8_group *group);
int fortai_cuda_q8_group_device_count(const fortai_cuda_q8_group *group);
const char *fortai_cuda_q8_group_last_error(const fortai_cuda_q8_group *group);

/* A rows x width GGUF Q8_0 matrix cut over the group's devices.  shard_mode 0: contiguous
 * row ranges (the partition of the reference's OpenMP row loop,
 * src/fortai_gguf_runtime.f90:457-463; multiples of 32 rows when rows % 32 == 0);
 * shard_mode 1: block ranges of every row (the K-slices of an FFN down matrix, matching
 * the row ranges of its gate/up partners). */
int fortai_cuda_q8_group_weights_upload(fortai_cuda_q8_group *group, const void *host_weights,
    size_t weight_bytes, int rows, int width, int shard_mode,
    fortai_cuda_q8_group_weights **weights);
int fortai_cuda_q8_group_weights_destroy(fortai_cuda_q8_group_weights *weights);

/* gguf_tensor_matvec_q8 (src/fortai_gguf_runtime.f90:424-465) over a row-sharded matrix:
 * host fp32 vector in, every device computes its slice with the GEMV fused with its
 * all-gather, host fp32 result out.  Per-row results are bit-identical to the one-device
 * kernel.  Blocks; elapsed_ms is host time around the call, transfers included. */
int fortai_cuda_q8_group_matvec_f32(fortai_cuda_q8_group *group,
    const fortai_cuda_q8_group_weights *weights, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms);

/* fortai_cuda_q8_ffn_host's computation (reference header :97-103) with gate/up
 * row-sharded (shard_mode 0) and down column-sharded (shard_mode 1): no exchange between
 * the halves; the partial outputs are summed on the first device in device order. */
int fortai_cuda_q8_group_ffn_f32(fortai_cuda_q8_group *group,
    const fortai_cuda_q8_group_weights *gate, const fortai_cuda_q8_group_weights *up,
    const fortai_cuda_q8_group_weights *down, const float *host_activation,
    size_t activation_elements, float *host_output, size_t output_bytes, float *elapsed_ms);

/* Has no counterpart in the reference.  Same contract and same result as
 * fortai_cuda_q8_ffn_device, for hosts that must not allocate while they run (all
 * free device memory already belongs to their own pools, or a cudaMalloc/cudaFree
 * in the middle of a decode step would stall the whole device): this call makes
 * no cudaMalloc, cudaFree or other allocating call.  Its two intermediates (the
 * fp32 hidden vector and its Q8_0 image) live in a fixed 164 KB array inside the
 * library image, held on every GPU that loads the library until the process
 * exits.  Limit: gate/up rows (the FFN inner size) <= 32768; larger shapes
 * return FORTAI_CUDA_INVALID with a message in fortai_cuda_q8_last_error.
 * The first call on a device looks the array's address up
 * (cudaGetSymbolAddress); make that first call before any stream capture.
 * The array is shared by every context and every call on that device and keeps
 * the previous call's contents; each call rewrites all of the part it reads, so
 * nothing needs clearing, but two calls that overlap on the GPU (different
 * streams) race on it.  Enqueue only. */
int fortai_cuda_q8_ffn_device_noalloc(fortai_cuda_q8_context *context,
    const fortai_cuda_q8_weights *gate_weights, const fortai_cuda_q8_weights *up_weights,
    const fortai_cuda_q8_weights *down_weights, const void *device_activation,
    size_t activation_elements, void *device_output, size_t output_elements);

#ifdef __cplusplus
}
#endif

#endif
