/* tensorfuse/tensorfuse.h -- the struct-based C interface of TensorFuse, as
 * implemented by the B200 build (libtensorfuse.so).
 *
 * Each declaration names the reference declaration (header) and definition it
 * replaces; argument meaning, validation order and status codes are the
 * reference's.  Operators run asynchronously on the caller's stream.
 */
#ifndef TENSORFUSE_B200_TENSORFUSE_H_
#define TENSORFUSE_B200_TENSORFUSE_H_

#include "types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TENSORFUSE_VERSION_STRING "1.0.0"

/* reference src/tensorfuse/tensorfuse.h:27, src/tensorfuse_c_api.cpp:58-85.
 * NULL config = defaults.  Idempotent.  Unlike the reference (which always
 * selects device 0 and ignores the device list) config->device_count and
 * config->device_ids select the GPUs that the host-buffer entry points of
 * tensorfuse_b200.h shard rows over. */
TensorFuseStatus tensorfuse_init(const TensorFuseConfig* config);

/* reference src/tensorfuse/tensorfuse.h:33, src/tensorfuse_c_api.cpp:87-97.
 * Releases the library's own streams and staging buffers.  It does NOT reset
 * the device (the reference calls cudaDeviceReset, which would destroy every
 * other CUDA user in the process). */
TensorFuseStatus tensorfuse_shutdown(void);
/* Name used by the reference README (README.md:230); same as tensorfuse_shutdown. */
TensorFuseStatus tensorfuse_cleanup(void);

/* reference src/tensorfuse/tensorfuse.h:39,46; src/tensorfuse_c_api.cpp:99-133 */
const char* tensorfuse_get_version(void);
const char* tensorfuse_get_error_string(TensorFuseStatus status);

/* output[M,N] = gelu(input[M,K] * weight[K,N] + bias[N]), tanh-form GELU.
 * reference src/tensorfuse/tensorfuse.h:64, src/tensorfuse_c_api.cpp:139-216.
 *   FLOAT32 / FLOAT16 : input, weight, output share the dtype; bias is read as that dtype.
 *   INT8 input+weight : `scale` of input and weight is a device pointer to one float.
 *       output FLOAT32, bias FLOAT32 : the reference convention,
 *           out = gelu(acc/(sA*sB) + bias) * (sA*sB)            (scale = 127/max|x|)
 *       output FLOAT16, bias FLOAT16 or FLOAT32 : out = gelu(acc*sA*sB + bias)   (scale = max|x|/127)
 *       output INT32 : the raw accumulator, bias ignored (may be any [N] tensor)
 * Extension: input and output may be 3-D [batch, seq, hidden]; they are
 * flattened to [batch*seq, hidden]. */
TensorFuseStatus tensorfuse_fused_gemm_bias_gelu(const TensorFuseTensor* input,
                                                 const TensorFuseTensor* weight,
                                                 const TensorFuseTensor* bias,
                                                 TensorFuseTensor* output, cudaStream_t stream);

/* output = dropout(softmax(input over the last of 4 dims), p); dropout_mask
 * (same shape, one byte per element, 1 = kept) is mandatory.
 * reference src/tensorfuse/tensorfuse.h:84, src/tensorfuse_c_api.cpp:218-286.
 * The seed of each call comes from the library's seed source
 * (tensorfuse_b200_set_random_seed); at p = 0 no random numbers are drawn. */
TensorFuseStatus tensorfuse_fused_softmax_dropout(const TensorFuseTensor* input,
                                                  TensorFuseTensor* output,
                                                  unsigned char* dropout_mask, float dropout_prob,
                                                  cudaStream_t stream);

/* reference src/tensorfuse/tensorfuse.h:106,127; src/tensorfuse_c_api.cpp:288-329.
 * The reference validates its arguments and computes nothing.  Here the same
 * validation (same order, same codes) is followed by the computation:
 *   attention   - query/key/value/output [batch, seq, hidden], FP16 or BF16,
 *                 hidden / num_heads == 64: softmax(Q K^T / 8) V per head with
 *                 dropout on the probabilities, one fused kernel;
 *   transformer - a post-LayerNorm encoder layer (QKV projection, attention,
 *                 output projection, residual + LayerNorm, FFN with GELU,
 *                 residual + LayerNorm) on the caller's stream.
 * Shapes or types outside those return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION. */
TensorFuseStatus tensorfuse_fused_multi_head_attention(const TensorFuseTensor* query,
                                                       const TensorFuseTensor* key,
                                                       const TensorFuseTensor* value,
                                                       TensorFuseTensor* output, int num_heads,
                                                       float dropout_prob, cudaStream_t stream);
TensorFuseStatus tensorfuse_fused_transformer_layer(const TensorFuseTensor* input,
                                                    TensorFuseTensor* output,
                                                    const TensorFuseTransformerParams* params,
                                                    cudaStream_t stream);

/* reference src/tensorfuse/tensorfuse.h:145-176; src/tensorfuse_c_api.cpp:335-392 (placeholders) */
TensorFuseStatus tensorfuse_autotune(const TensorFuseModelConfig* model_config, const char* output_path);
TensorFuseStatus tensorfuse_load_tuned_config(const char* config_path);
TensorFuseStatus tensorfuse_start_profiling(const TensorFuseProfileConfig* profile_config);
TensorFuseStatus tensorfuse_stop_profiling(const char* output_path);

/* reference src/tensorfuse/tensorfuse.h:191-204; src/tensorfuse_c_api.cpp:398-456 */
TensorFuseStatus tensorfuse_allocate_tensor(TensorFuseTensor* tensor, const TensorFuseShape* shape,
                                            TensorFuseDataType dtype, int device_id);
TensorFuseStatus tensorfuse_free_tensor(TensorFuseTensor* tensor);

#ifdef __cplusplus
}
#endif
#endif /* TENSORFUSE_B200_TENSORFUSE_H_ */
