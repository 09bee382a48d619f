/* tensorfuse_b200.h -- flat-pointer entry points of libtensorfuse.so.
 *
 * Part 1 are the C symbols the reference's benchmarks and C++ tests bind
 * (plain device pointers and sizes); part 2 are additions of this build.
 */
#ifndef TENSORFUSE_B200_H_
#define TENSORFUSE_B200_H_

#include "tensorfuse/types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ part 1
 * C = gelu(alpha * A[M,K] * B[K,N] + beta * bias[N]); all row-major device
 * memory, bias and C of the operand type.
 * reference declarations benchmarks/tensorfuse_c_api.h:44-52, definitions
 * src/kernels/fused_gemm_bias_gelu.cu:352-370 (fp32/fp16),
 * src/kernels/fused_gemm_bias_gelu_optimized.cu:314-328 (optimized_*). */
TensorFuseStatus fused_gemm_bias_gelu_fp32_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t stream);
TensorFuseStatus fused_gemm_bias_gelu_fp16_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t stream);
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp32_wrapper(const void* A, const void* B,
                                                             const void* bias, void* C, int M,
                                                             int N, int K, float alpha, float beta,
                                                             cudaStream_t stream);
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp16_wrapper(const void* A, const void* B,
                                                             const void* bias, void* C, int M,
                                                             int N, int K, float alpha, float beta,
                                                             cudaStream_t stream);

/* INT8 operands, FP32 bias, FP32 output, the reference's scale convention
 * (scale = 127/max|x|): C = gelu_clamped(acc/(scale_A*scale_B) + bias) * (scale_A*scale_B),
 * non-finite results replaced by 0; alpha and beta are accepted and, as in the
 * reference, have no effect.  The variant without scales uses 1, 1.
 * reference src/kernels/fused_gemm_bias_gelu_int8.cu:364-378 */
TensorFuseStatus fused_gemm_bias_gelu_int8_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t stream);
TensorFuseStatus fused_gemm_bias_gelu_int8_wrapper_with_scales(const void* A, const void* B,
                                                               const void* bias, void* C, int M,
                                                               int N, int K, float alpha, float beta,
                                                               float scale_A, float scale_B,
                                                               cudaStream_t stream);

/* Softmax over the innermost axis of a [batch, num_heads, seq_len, head_dim]
 * tensor followed by dropout.  NOTE the argument order (seq_len, head_dim,
 * num_heads) and that `head_dim` is the softmax axis: for attention
 * probabilities [B,H,S,S] pass seq_len = S, head_dim = S.
 * reference src/kernels/fused_softmax_dropout.cu:324-342 */
TensorFuseStatus fused_softmax_dropout_fp16_wrapper(const void* input, void* output,
                                                    unsigned char* dropout_mask, int batch_size,
                                                    int seq_len, int head_dim, int num_heads,
                                                    float dropout_prob, unsigned long long seed,
                                                    cudaStream_t stream);
TensorFuseStatus fused_softmax_dropout_fp32_wrapper(const void* input, void* output,
                                                    unsigned char* dropout_mask, int batch_size,
                                                    int seq_len, int head_dim, int num_heads,
                                                    float dropout_prob, unsigned long long seed,
                                                    cudaStream_t stream);

/* ------------------------------------------------------------------ part 2
 * Additions of this build; no reference declaration unless stated. */

/* General INT8 entry: in-kernel dequantisation with selectable bias / output
 * type and convention.
 *   epilogue 1: out = gelu(fma(float(acc), scale_A*scale_B, bias)), out FLOAT16 or FLOAT32
 *   epilogue 2: the reference convention above, bias FLOAT32, out FLOAT32
 *   epilogue 3: out = acc (INT32), bias unused
 * bias_dtype / out_dtype are TensorFuseDataType values. */
TensorFuseStatus tensorfuse_b200_gemm_int8(const void* A, const void* B, const void* bias, void* C,
                                           int M, int N, int K, float scale_A, float scale_B,
                                           int bias_dtype, int out_dtype, int epilogue,
                                           cudaStream_t stream);

/* FP8 (E4M3, one byte per element, as in TENSORFUSE_FP8_E4M3) operands with
 * per-tensor dequantisation factors: C = gelu(acc * scale_A * scale_B + bias),
 * FP32 accumulation on the tensor cores, FP16 or FP32 bias and output.  The
 * reference enumerates the type (src/tensorfuse/types.h:56) and has no kernel
 * for it.  Through the struct entry point the scales are the device-resident
 * `scale` fields of the input and weight tensors, exactly as for INT8. */
TensorFuseStatus tensorfuse_b200_gemm_fp8(const void* A, const void* B, const void* bias, void* C,
                                          int M, int N, int K, float scale_A, float scale_B,
                                          int bias_dtype, int out_dtype, cudaStream_t stream);

/* C = act(alpha * A[M,K] * B[K,N] + beta * bias[N]) for FP16, BF16 or FP32 operands
 * (dtype; BF16 is also accepted by tensorfuse_fused_gemm_bias_gelu, which the
 * reference enumerates in src/tensorfuse/types.h:52 without a kernel), activation = TENSORFUSE_ACTIVATION_GELU or TENSORFUSE_ACTIVATION_NONE.
 * NONE is the FFN-down form: the reference's benchmark applies GELU to that
 * projection too because its only entry point always does
 * (benchmarks/bert_baseline.cu:318-322); the activation enum is the reference's
 * (src/tensorfuse/types.h:74-81). */
TensorFuseStatus tensorfuse_b200_gemm_bias_act(const void* A, const void* B, const void* bias, void* C,
                                               int M, int N, int K, int dtype, int activation,
                                               float alpha, float beta, cudaStream_t stream);

/* Scaled-dot-product attention over heads, fused (the computation behind
 * tensorfuse_fused_multi_head_attention, which the reference leaves as a
 * placeholder: src/tensorfuse_c_api.cpp:288-311):
 *   out[b,i,h,:] = sum_j keep_j/(1-p) * softmax_j(scale * q[b,i,h,:].k[b,j,h,:]) * v[b,j,h,:]
 * Element (b, s, h, c) of a tensor is at base + b*bs + s*ld + h*hs + c, strides
 * in elements; hs = 0 means head_dim and bs = 0 means seq*ld, i.e. rows of
 * [batch, seq, heads*head_dim] (a fused QKV buffer is ld = 3*hidden with three
 * base pointers).  scale <= 0 selects 1/sqrt(head_dim).  kv_lengths (device,
 * `batch` ints, may be NULL) masks keys j >= kv_lengths[b]; a row without a
 * valid key yields zeros.  Dropout decisions are those the softmax+dropout
 * operator makes for a [batch, heads, seq_q, seq_kv] tensor with the same seed.
 * FP16 with head_dim 64 and 16-byte aligned pointers / strides runs on the
 * tensor cores; other FP16 / FP32 shapes (head_dim <= 256) on CUDA cores. */
TensorFuseStatus tensorfuse_b200_attention(const void* q, const void* k, const void* v, void* out, int batch,
                                           int seq_q, int seq_kv, int heads, int head_dim, long long ld_q,
                                           long long ld_k, long long ld_v, long long ld_o, long long hs_q,
                                           long long hs_k, long long hs_v, long long hs_o, long long bs_q,
                                           long long bs_k, long long bs_v, long long bs_o, int dtype,
                                           float scale, float dropout_prob, unsigned long long seed,
                                           const int* kv_lengths, cudaStream_t stream);

/* softmax(scale * x) + dropout over rows of `row_len` with the key positions
 * >= kv_lengths[b] of batch item b masked inside the kernel (no -inf scores
 * have to be materialised by the caller): input/output/mask are
 * [batch, rows_per_item, row_len] (for attention probabilities rows_per_item =
 * heads * seq_q), kv_lengths is a device array of `batch` ints or NULL, scale
 * > 0.  A row with no valid position yields zeros.  Same Philox stream as
 * tensorfuse_fused_softmax_dropout; FP32 arithmetic for both storage types.
 * No reference counterpart: the reference's operator takes neither a scale nor
 * a mask (src/tensorfuse/tensorfuse.h:72-88). */
TensorFuseStatus tensorfuse_b200_softmax_dropout_masked(const void* input, void* output,
                                                        unsigned char* dropout_mask, long long batch,
                                                        long long rows_per_item, int row_len, int dtype,
                                                        float scale, const int* kv_lengths, float dropout_prob,
                                                        unsigned long long seed, cudaStream_t stream);

/* Per-tensor symmetric INT8 quantisation of n FP16 / FP32 elements on the
 * device: *scale_dev = max|x| / 127 (1 for an all-zero tensor), q[i] =
 * clip(rint(x[i] / scale), -127, 127).  The scale stays in device memory, which
 * is where TensorFuseTensor.scale of the INT8 GEMM expects it.  (The reference
 * has no quantiser; its Python binding guesses scales from the INT8 data on the
 * host, src/python/core_bindings.cpp:467-491.)  Asynchronous, allocates nothing. */
TensorFuseStatus tensorfuse_b200_quantize_int8(const void* x, int dtype, long long n, signed char* q,
                                               float* scale_dev, cudaStream_t stream);

/* out = LayerNorm(x + residual) * gamma + beta over rows of `hidden` elements,
 * FP16 or FP32 storage, FP32 arithmetic (residual may be NULL).  The glue
 * between the fused operators inside tensorfuse_fused_transformer_layer; the
 * reference carries layer-norm weights in TensorFuseTransformerParams
 * (src/tensorfuse/types.h:153-185) but has no kernel for them. */
TensorFuseStatus tensorfuse_b200_add_layernorm(const void* x, const void* residual, const void* gamma,
                                               const void* beta, void* out, long long rows, int hidden,
                                               int dtype, float eps, cudaStream_t stream);

/* Channel-wise variant for weights w[K, N] (row-major FP16 / FP32): one scale per
 * output column, scales_dev[n] = max_k |w[k,n]| / 127 (1 for an all-zero column),
 * q[k,n] = clip(rint(w[k,n] / scales_dev[n]), -127, 127). */
TensorFuseStatus tensorfuse_b200_quantize_int8_columns(const void* w, int dtype, int K, int N, signed char* q,
                                                       float* scales_dev, cudaStream_t stream);

/* INT8 GEMM with a per-tensor activation scale and per-column weight scales, both
 * read on the device: C[m,n] = gelu(acc[m,n] * *scale_A_dev * scale_B_cols_dev[n] + bias[n]),
 * FP16 or FP32 bias and output.  scale_A_dev may be NULL (= 1). */
TensorFuseStatus tensorfuse_b200_gemm_int8_channelwise(const void* A, const void* B, const void* bias, void* C,
                                                       int M, int N, int K, const float* scale_A_dev,
                                                       const float* scale_B_cols_dev, int bias_dtype,
                                                       int out_dtype, cudaStream_t stream);

/* Row-sharded softmax+dropout: `rows` rows of length `row_len`; `first_row`
 * is the index of the first of them inside the whole tensor, so that a shard
 * draws exactly the dropout decisions it would get as part of the whole.
 * dtype is TENSORFUSE_FLOAT16 or TENSORFUSE_FLOAT32. */
TensorFuseStatus tensorfuse_b200_softmax_dropout_rows(const void* input, void* output,
                                                      unsigned char* dropout_mask, long long rows,
                                                      int row_len, int dtype, float dropout_prob,
                                                      unsigned long long seed,
                                                      unsigned long long first_row,
                                                      cudaStream_t stream);

/* The summation schedule the softmax kernel uses for a row of `row_len`
 * elements (vec = elements per thread step, warps = warps per row); a CPU that
 * follows the same schedule reproduces the result bit for bit. */
void tensorfuse_b200_softmax_schedule(int row_len, int dtype, int aligned16, int* vec, int* warps);
/* The same with the third property of the schedule: online = 1 for rows too
 * long to be held in shared memory (more than 200 KiB), whose sum of
 * exponentials is formed in a single sweep with a running maximum. */
void tensorfuse_b200_softmax_schedule_ex(int row_len, int dtype, int aligned16, int* vec, int* warps, int* online);

/* Seed source of tensorfuse_fused_softmax_dropout: after this call the n-th
 * dropout call uses a seed derived from (seed, n).  Declared, but a no-op, in
 * the reference (src/tensorfuse.h:60, src/python/core_bindings.cpp:840-843). */
void tensorfuse_b200_set_random_seed(unsigned long long seed);
/* The seed the most recent tensorfuse_fused_softmax_dropout call on this thread used. */
unsigned long long tensorfuse_b200_last_softmax_seed(void);

/* Host-buffer operators: the operands live in host memory (pinned memory is
 * copied asynchronously, pageable memory works but is slower).  Rows are split
 * over the devices chosen at tensorfuse_init; on every device the shard moves
 * through a copy-in / compute / copy-out pipeline on three streams, weights are
 * replicated.  Blocking.  These replace the staging the reference's Python
 * binding performs (src/python/core_bindings.cpp:360-633 and 635-771:
 * cudaMalloc, synchronous copies, one device).
 * dtypes are TensorFuseDataType values; for INT8 operands `epilogue` is as for
 * tensorfuse_b200_gemm_int8, otherwise it is ignored. */
TensorFuseStatus tensorfuse_b200_gemm_bias_gelu_host(const void* A, const void* B, const void* bias,
                                                     void* C, int M, int N, int K, int in_dtype,
                                                     int bias_dtype, int out_dtype, int epilogue,
                                                     float scale_A, float scale_B);
TensorFuseStatus tensorfuse_b200_softmax_dropout_host(const void* input, void* output,
                                                      unsigned char* dropout_mask, long long rows,
                                                      int row_len, int dtype, float dropout_prob,
                                                      unsigned long long seed);
/* Concurrency of the two host-buffer operators above: they may be called from
 * several threads; calls that use the same device are serialised (they share
 * that device's staging buffers and streams).  tensorfuse_shutdown must not
 * run while one of them is in flight.
 *
 * Weights that do not change between calls: register the host range of B (and
 * of bias) once and the GEMM operator keeps one device copy per selected
 * device instead of uploading it on every call (the reference's binding
 * uploads every operand per call, src/python/core_bindings.cpp:402-461).
 * The range must stay unmodified and allocated until it is invalidated;
 * invalidate (NULL = every range) before changing or freeing the memory.
 * Lookup is by the exact start address passed to the operator.
 * Device memory may be registered too: tensorfuse_fused_transformer_layer then
 * builds its fused [hidden, 3*hidden] query/key/value weight (and bias) once per
 * device for a layer whose three projection matrices are registered, instead of
 * concatenating them on every call. */
TensorFuseStatus tensorfuse_b200_register_weights(const void* host_ptr, size_t bytes);
TensorFuseStatus tensorfuse_b200_invalidate_weights(const void* host_ptr);

/* The same operator as tensorfuse_b200_softmax_dropout_host for callers that
 * must not allocate device memory -- a process whose device memory already
 * belongs to another allocator or sits at an MPS / MIG cap, or a serving thread
 * that cannot take the device-wide synchronisation of cudaMalloc / cudaFree.
 * It has no counterpart in the reference.  Operands are staged in a fixed
 * 16 MiB area that is part of the library image on every GPU that loads it; no
 * memory is allocated or freed, on the device or pinned, by this call.
 *   - limit: 2 * round256(rows*row_len*elem_size) + round256(rows*row_len) must
 *     not exceed 16 MiB (1-device, whole tensor at once); a larger request
 *     returns TENSORFUSE_ERROR_OUT_OF_MEMORY and touches nothing;
 *   - runs on the current device and on `stream`, returns after the results are
 *     in `output` / `dropout_mask`;
 *   - the first call on a device looks up the address of the staging area; make
 *     that first call before any stream capture begins;
 *   - all calls share the one staging area, whose contents persist from call to
 *     call: each call overwrites every byte it later reads (nothing has to
 *     start at zero), but two calls that overlap in time on the same GPU race. */
TensorFuseStatus tensorfuse_b200_softmax_dropout_host_noalloc(const void* input, void* output,
                                                              unsigned char* dropout_mask,
                                                              long long rows, int row_len, int dtype,
                                                              float dropout_prob,
                                                              unsigned long long seed,
                                                              cudaStream_t stream);
/* Device selection of the reference's benchmark programs: cudaSetDevice and
 * nothing else.  reference benchmarks/tensorfuse_wrappers.cpp:30-46 (compiled
 * into those programs there; exported here so that they link against the
 * library alone).  Only the value 0 of the status is portable: the benchmark
 * header declares its own enumerators (benchmarks/tensorfuse_c_api.h:20-28). */
TensorFuseStatus tensorfuse_simple_init(int device_id);
void tensorfuse_simple_cleanup(void);

/* Helpers of the Python binding, in place of its direct CUDA runtime calls
 * (reference src/python/core_bindings.cpp:402-461, memory_bindings.cpp:46-61,
 * core_bindings.cpp:830-838 -- the last two return constants there).
 * kind: 1 host->device, 2 device->host, 3 device->device; synchronous. */
TensorFuseStatus tensorfuse_b200_memcpy(void* dst, const void* src, size_t bytes, int kind);
TensorFuseStatus tensorfuse_b200_mem_info(int device, size_t* free_bytes, size_t* total_bytes);
/* device < 0: the current device.  Any output pointer may be NULL. */
TensorFuseStatus tensorfuse_b200_device_info(int device, char* name, int name_capacity, int* cc_major,
                                             int* cc_minor, size_t* total_memory, int* multiprocessors);

/* Page-locked host memory for the calls above. */
void* tensorfuse_b200_alloc_pinned(size_t bytes);
void tensorfuse_b200_free_pinned(void* p);

/* The row split the host-buffer operators use: `parts` contiguous ranges whose
 * starts are multiples of `align`; begins/counts receive `parts` entries. */
void tensorfuse_b200_plan_shards(long long rows, int parts, int align, long long* begins,
                                 long long* counts);

/* Devices selected at init (count, and the ordinal of the i-th). */
int tensorfuse_b200_device_count(void);
int tensorfuse_b200_device_id(int i);

/* Device-side watchdog: every wait inside the kernels is bounded; 0 = no wait
 * has expired since the last reset, otherwise the code of the first one. */
int tensorfuse_b200_watchdog_status(void);
void tensorfuse_b200_watchdog_reset(void);

/* Number of CUDA kernels this library has launched in this process. */
unsigned long long tensorfuse_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TENSORFUSE_B200_H_ */
