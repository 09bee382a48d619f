/* tensorfuse/kernels.h -- the C++ kernel launchers of namespace
 * tensorfuse::kernels (flat device pointers), exported by libtensorfuse.so
 * with C++ linkage.  Their mangled names are part of the binary interface:
 * the reference's tests resolve them with dlsym
 * (src/tests/test_kernels_simple.cpp:62-63, test_working_kernel.cu:75-76) or
 * declare them inline (src/tests/test_kernels.cu:26-40, test_gemm_edge_cases.cu:28-36).
 *
 * C[M,N] = gelu(alpha * A[M,K] * B[K,N] + beta * bias[N]); everything row-major
 * device memory.  All launches are asynchronous on `stream`.
 */
#ifndef TENSORFUSE_B200_KERNELS_H_
#define TENSORFUSE_B200_KERNELS_H_

#include "types.h"

#ifdef __cplusplus
namespace tensorfuse {
namespace kernels {

/* reference src/kernels/fused_gemm_bias_gelu.h:36,61 (definitions
 * src/kernels/fused_gemm_bias_gelu.cu:306-348) */
TensorFuseStatus fused_gemm_bias_gelu_fp32(const void* A, const void* B, const void* bias, void* C, int M, int N,
                                           int K, float alpha, float beta, cudaStream_t stream);
TensorFuseStatus fused_gemm_bias_gelu_fp16(const void* A, const void* B, const void* bias, void* C, int M, int N,
                                           int K, float alpha, float beta, cudaStream_t stream);
/* reference src/kernels/fused_gemm_bias_gelu_optimized.cu:262-306: the same
 * computation; both names reach the same kernels here. */
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp32(const void* A, const void* B, const void* bias, void* C, int M,
                                                     int N, int K, float alpha, float beta, cudaStream_t stream);
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp16(const void* A, const void* B, const void* bias, void* C, int M,
                                                     int N, int K, float alpha, float beta, cudaStream_t stream);
/* INT8 operands, FP32 bias and output, the reference's scale convention
 * (scale = 127 / max|x|): C = gelu_clamped(acc / (sA*sB) + bias) * (sA*sB);
 * alpha and beta are accepted and have no effect, as in the reference.
 * reference src/kernels/fused_gemm_bias_gelu.h:88, src/kernels/fused_gemm_bias_gelu_int8.cu:294-362 */
TensorFuseStatus fused_gemm_bias_gelu_int8(const void* A, const void* B, const void* bias, void* C, int M, int N,
                                           int K, float alpha, float beta, cudaStream_t stream);
TensorFuseStatus fused_gemm_bias_gelu_int8_with_scales(const void* A, const void* B, const void* bias, void* C,
                                                       int M, int N, int K, float alpha, float beta, float scale_A,
                                                       float scale_B, cudaStream_t stream);

/* Softmax over the innermost axis (`head_dim` elements) of a
 * [batch_size, num_heads, seq_len, head_dim] tensor, then dropout with a
 * one-byte-per-element mask.  Argument order as in the reference:
 * (batch_size, seq_len, head_dim, num_heads).
 * reference src/kernels/fused_softmax_dropout.h:28,55 */
TensorFuseStatus fused_softmax_dropout_fp16(const void* input, void* output, unsigned char* dropout_mask,
                                            int batch_size, int seq_len, int head_dim, int num_heads,
                                            float dropout_prob, unsigned long long seed, cudaStream_t stream);
TensorFuseStatus fused_softmax_dropout_fp32(const void* input, void* output, unsigned char* dropout_mask,
                                            int batch_size, int seq_len, int head_dim, int num_heads,
                                            float dropout_prob, unsigned long long seed, cudaStream_t stream);

}  // namespace kernels
}  // namespace tensorfuse
#endif
#endif /* TENSORFUSE_B200_KERNELS_H_ */
