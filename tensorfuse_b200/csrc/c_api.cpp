// c_api.cpp -- the exported C ABI (and the C++ symbols the reference's tests
// resolve with dlsym) on top of the launchers in kernels.h.
//
// Validation order and status codes follow reference src/tensorfuse_c_api.cpp:
// not initialised -> 4, NULL -> 1, wrong rank/shape -> 11, dtype mismatch -> 1,
// unsupported dtype -> 10.  There is no CPU fallback: every operator either
// launches a CUDA kernel or returns an error status.
#include <string.h>

#include "kernels.h"
#include "runtime.h"
#include "tensorfuse/kernels.h"
#include "tensorfuse/tensorfuse.h"
#include "tensorfuse_b200.h"

using namespace tfb;

namespace {

TensorFuseStatus to_status(LaunchResult r) {
  switch (r) {
    case kOk: return TENSORFUSE_SUCCESS;
    case kInvalidArgument: return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    case kCudaError: return TENSORFUSE_ERROR_CUDA_ERROR;
    case kLaunchFailed: return TENSORFUSE_ERROR_KERNEL_LAUNCH_FAILED;
    case kUnsupported: return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  }
  return TENSORFUSE_ERROR_UNKNOWN;
}

thread_local unsigned long long t_last_seed = 0;

// Launch on the device that owns the output buffer (the caller may have another
// device current).
struct OwnerGuard {
  DeviceGuard g;
  explicit OwnerGuard(const void* out) : g(device_of_pointer(out)) {}
};

TensorFuseStatus gemm_flat(const void* A, const void* B, const void* bias, void* C, int M, int N,
                           int K, int in_dtype, int bias_dtype, int out_dtype, int epilogue,
                           float alpha, float beta, float scale, const float* sa_dev,
                           const float* sb_dev, cudaStream_t stream) {
  if (!A || !B || !C || (!bias && epilogue != kEpiI8Raw)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (M <= 0 || N <= 0 || K <= 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  GemmArgs a{};
  a.A = A; a.B = B; a.bias = bias; a.C = C;
  a.M = M; a.N = N; a.K = K;
  a.in_dtype = in_dtype; a.bias_dtype = bias_dtype; a.out_dtype = out_dtype;
  a.epilogue = epilogue;
  a.alpha = alpha; a.beta = beta; a.scale = scale;
  a.scale_a_dev = sa_dev; a.scale_b_dev = sb_dev;
  OwnerGuard og(C);
  return to_status(launch_gemm(a, stream));
}

}  // namespace

// ===================================================== C++ symbols (mangled)
// The reference's tests look these up by their mangled names
// (reference src/tests/test_kernels_simple.cpp:62-63, test_working_kernel.cu:75-76),
// so they are part of the binary interface.
namespace tensorfuse {
namespace kernels {

TensorFuseStatus fused_gemm_bias_gelu_fp32(const void* A, const void* B, const void* bias, void* C,
                                           int M, int N, int K, float alpha, float beta,
                                           cudaStream_t stream) {
  return gemm_flat(A, B, bias, C, M, N, K, kF32, kF32, kF32, kEpiGelu, alpha, beta, 1.0f, nullptr,
                   nullptr, stream);
}
TensorFuseStatus fused_gemm_bias_gelu_fp16(const void* A, const void* B, const void* bias, void* C,
                                           int M, int N, int K, float alpha, float beta,
                                           cudaStream_t stream) {
  return gemm_flat(A, B, bias, C, M, N, K, kF16, kF16, kF16, kEpiGelu, alpha, beta, 1.0f, nullptr,
                   nullptr, stream);
}
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp32(const void* A, const void* B, const void* bias,
                                                     void* C, int M, int N, int K, float alpha,
                                                     float beta, cudaStream_t stream) {
  return fused_gemm_bias_gelu_fp32(A, B, bias, C, M, N, K, alpha, beta, stream);
}
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp16(const void* A, const void* B, const void* bias,
                                                     void* C, int M, int N, int K, float alpha,
                                                     float beta, cudaStream_t stream) {
  return fused_gemm_bias_gelu_fp16(A, B, bias, C, M, N, K, alpha, beta, stream);
}
TensorFuseStatus fused_gemm_bias_gelu_int8_with_scales(const void* A, const void* B,
                                                       const void* bias, void* C, int M, int N,
                                                       int K, float alpha, float beta,
                                                       float scale_A, float scale_B,
                                                       cudaStream_t stream) {
  (void)alpha; (void)beta;  // no effect in the reference either (fused_gemm_bias_gelu_int8.cu:73,185)
  return gemm_flat(A, B, bias, C, M, N, K, kI8, kF32, kF32, kEpiI8Legacy, 1.0f, 1.0f,
                   scale_A * scale_B, nullptr, nullptr, stream);
}
TensorFuseStatus fused_gemm_bias_gelu_int8(const void* A, const void* B, const void* bias, void* C,
                                           int M, int N, int K, float alpha, float beta,
                                           cudaStream_t stream) {
  return fused_gemm_bias_gelu_int8_with_scales(A, B, bias, C, M, N, K, alpha, beta, 1.0f, 1.0f,
                                               stream);
}

static TensorFuseStatus softmax_flat(const void* in, void* out, unsigned char* mask, int batch,
                                     int seq_len, int head_dim, int num_heads, float p,
                                     unsigned long long seed, int dtype, cudaStream_t stream) {
  if (!in || !out || !mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (batch < 0 || seq_len < 0 || head_dim < 0 || num_heads < 0)
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const long long rows = (long long)batch * num_heads * seq_len;
  OwnerGuard og(out);
  return to_status(launch_softmax_dropout(in, out, mask, rows, head_dim, dtype, p, seed, 0, stream));
}
TensorFuseStatus fused_softmax_dropout_fp16(const void* in, void* out, unsigned char* mask,
                                            int batch, int seq_len, int head_dim, int num_heads,
                                            float p, unsigned long long seed, cudaStream_t stream) {
  return softmax_flat(in, out, mask, batch, seq_len, head_dim, num_heads, p, seed, kF16, stream);
}
TensorFuseStatus fused_softmax_dropout_fp32(const void* in, void* out, unsigned char* mask,
                                            int batch, int seq_len, int head_dim, int num_heads,
                                            float p, unsigned long long seed, cudaStream_t stream) {
  return softmax_flat(in, out, mask, batch, seq_len, head_dim, num_heads, p, seed, kF32, stream);
}

}  // namespace kernels
}  // namespace tensorfuse

namespace tk = tensorfuse::kernels;

extern "C" {

// ============================================================ flat wrappers
TensorFuseStatus fused_gemm_bias_gelu_fp32_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_fp32(A, B, bias, C, M, N, K, alpha, beta, s);
}
TensorFuseStatus fused_gemm_bias_gelu_fp16_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_fp16(A, B, bias, C, M, N, K, alpha, beta, s);
}
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp32_wrapper(const void* A, const void* B,
                                                             const void* bias, void* C, int M,
                                                             int N, int K, float alpha, float beta,
                                                             cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_fp32(A, B, bias, C, M, N, K, alpha, beta, s);
}
TensorFuseStatus optimized_fused_gemm_bias_gelu_fp16_wrapper(const void* A, const void* B,
                                                             const void* bias, void* C, int M,
                                                             int N, int K, float alpha, float beta,
                                                             cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_fp16(A, B, bias, C, M, N, K, alpha, beta, s);
}
TensorFuseStatus fused_gemm_bias_gelu_int8_wrapper(const void* A, const void* B, const void* bias,
                                                   void* C, int M, int N, int K, float alpha,
                                                   float beta, cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_int8(A, B, bias, C, M, N, K, alpha, beta, s);
}
TensorFuseStatus fused_gemm_bias_gelu_int8_wrapper_with_scales(const void* A, const void* B,
                                                               const void* bias, void* C, int M,
                                                               int N, int K, float alpha, float beta,
                                                               float scale_A, float scale_B,
                                                               cudaStream_t s) {
  return tk::fused_gemm_bias_gelu_int8_with_scales(A, B, bias, C, M, N, K, alpha, beta, scale_A,
                                                   scale_B, s);
}
TensorFuseStatus fused_softmax_dropout_fp16_wrapper(const void* in, void* out, unsigned char* mask,
                                                    int batch, int seq_len, int head_dim,
                                                    int num_heads, float p, unsigned long long seed,
                                                    cudaStream_t s) {
  return tk::fused_softmax_dropout_fp16(in, out, mask, batch, seq_len, head_dim, num_heads, p, seed, s);
}
TensorFuseStatus fused_softmax_dropout_fp32_wrapper(const void* in, void* out, unsigned char* mask,
                                                    int batch, int seq_len, int head_dim,
                                                    int num_heads, float p, unsigned long long seed,
                                                    cudaStream_t s) {
  return tk::fused_softmax_dropout_fp32(in, out, mask, batch, seq_len, head_dim, num_heads, p, seed, s);
}

// ========================================================= library lifetime
TensorFuseStatus tensorfuse_init(const TensorFuseConfig* config) { return Runtime::get().init(config); }
TensorFuseStatus tensorfuse_shutdown(void) { return Runtime::get().shutdown(); }
TensorFuseStatus tensorfuse_cleanup(void) { return Runtime::get().shutdown(); }
const char* tensorfuse_get_version(void) { return TENSORFUSE_VERSION_STRING; }

const char* tensorfuse_get_error_string(TensorFuseStatus status) {
  switch (status) {
    case TENSORFUSE_SUCCESS: return "Success";
    case TENSORFUSE_ERROR_INVALID_ARGUMENT: return "Invalid argument";
    case TENSORFUSE_ERROR_CUDA_ERROR: return "CUDA error";
    case TENSORFUSE_ERROR_OUT_OF_MEMORY: return "Out of memory";
    case TENSORFUSE_ERROR_NOT_INITIALIZED: return "Library not initialized";
    case TENSORFUSE_ERROR_INVALID_CONFIGURATION: return "Invalid configuration";
    case TENSORFUSE_ERROR_KERNEL_LAUNCH_FAILED: return "Kernel launch failed";
    case TENSORFUSE_ERROR_AUTOTUNER_FAILED: return "Autotuner failed";
    case TENSORFUSE_ERROR_PROFILING_FAILED: return "Profiling failed";
    case TENSORFUSE_ERROR_FILE_IO: return "File I/O error";
    case TENSORFUSE_ERROR_UNSUPPORTED_OPERATION: return "Unsupported operation";
    case TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE: return "Invalid tensor shape";
    default: return "Unknown error";
  }
}

// ================================================================ operators
TensorFuseStatus tensorfuse_fused_gemm_bias_gelu(const TensorFuseTensor* input,
                                                 const TensorFuseTensor* weight,
                                                 const TensorFuseTensor* bias,
                                                 TensorFuseTensor* output, cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!input || !weight || !bias || !output) return TENSORFUSE_ERROR_INVALID_ARGUMENT;

  const bool rank2 = input->shape.ndims == 2 && output->shape.ndims == 2;
  const bool rank3 = input->shape.ndims == 3 && output->shape.ndims == 3;  // [batch, seq, hidden]
  if ((!rank2 && !rank3) || weight->shape.ndims != 2 || bias->shape.ndims != 1)
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;

  long long M64;
  int K, out_cols;
  if (rank2) {
    M64 = input->shape.dims[0];
    K = input->shape.dims[1];
    if (output->shape.dims[0] != input->shape.dims[0]) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
    out_cols = output->shape.dims[1];
  } else {
    M64 = (long long)input->shape.dims[0] * input->shape.dims[1];
    K = input->shape.dims[2];
    if (output->shape.dims[0] != input->shape.dims[0] || output->shape.dims[1] != input->shape.dims[1])
      return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
    out_cols = output->shape.dims[2];
  }
  const int N = weight->shape.dims[1];
  if (weight->shape.dims[0] != K || bias->shape.dims[0] != N || out_cols != N || M64 > 0x7fffffffLL)
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const int M = (int)M64;

  const float alpha = 1.0f, beta = 1.0f;
  if (input->dtype == TENSORFUSE_INT8) {
    if (weight->dtype != TENSORFUSE_INT8) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    const float* sa = static_cast<const float*>(input->scale);
    const float* sb = static_cast<const float*>(weight->scale);
    if (output->dtype == TENSORFUSE_FLOAT32 && bias->dtype == TENSORFUSE_FLOAT32)
      return gemm_flat(input->data, weight->data, bias->data, output->data, M, N, K, kI8, kF32, kF32,
                       kEpiI8Legacy, 1.0f, 1.0f, 1.0f, sa, sb, stream);
    if (output->dtype == TENSORFUSE_FLOAT16 &&
        (bias->dtype == TENSORFUSE_FLOAT16 || bias->dtype == TENSORFUSE_FLOAT32))
      return gemm_flat(input->data, weight->data, bias->data, output->data, M, N, K, kI8,
                       bias->dtype == TENSORFUSE_FLOAT16 ? kF16 : kF32, kF16, kEpiI8Dequant, 1.0f, 1.0f,
                       1.0f, sa, sb, stream);
    if (output->dtype == TENSORFUSE_INT32)
      return gemm_flat(input->data, weight->data, bias->data, output->data, M, N, K, kI8, kF32, kI32,
                       kEpiI8Raw, 1.0f, 1.0f, 1.0f, nullptr, nullptr, stream);
    // The reference's validation also lets INT8 bias / INT8 output through
    // (src/tensorfuse_c_api.cpp:171-177) but has no kernel for them.
    if ((bias->dtype == TENSORFUSE_INT8 || bias->dtype == TENSORFUSE_FLOAT32) &&
        (output->dtype == TENSORFUSE_INT8 || output->dtype == TENSORFUSE_FLOAT32))
      return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
    return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  }
  if (input->dtype == TENSORFUSE_FP8_E4M3) {
    // FP8 operands with per-tensor dequantisation scales (device pointers, as for INT8):
    // out = gelu(acc * sA * sB + bias), FP16 or FP32 output
    if (weight->dtype != TENSORFUSE_FP8_E4M3) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    if ((output->dtype != TENSORFUSE_FLOAT16 && output->dtype != TENSORFUSE_FLOAT32) ||
        (bias->dtype != TENSORFUSE_FLOAT16 && bias->dtype != TENSORFUSE_FLOAT32))
      return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
    return gemm_flat(input->data, weight->data, bias->data, output->data, M, N, K, kFp8E4M3,
                     bias->dtype == TENSORFUSE_FLOAT16 ? kF16 : kF32, output->dtype == TENSORFUSE_FLOAT16 ? kF16 : kF32,
                     kEpiI8Dequant, 1.0f, 1.0f, 1.0f, static_cast<const float*>(input->scale),
                     static_cast<const float*>(weight->scale), stream);
  }
  if (input->dtype != weight->dtype || input->dtype != output->dtype)
    return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (input->dtype == TENSORFUSE_BFLOAT16)
    return gemm_flat(input->data, weight->data, bias->data, output->data, M, N, K, kBF16,
                     bias->dtype == TENSORFUSE_FLOAT32 ? kF32 : kBF16, kBF16, kEpiGelu, alpha, beta, 1.0f, nullptr,
                     nullptr, stream);
  if (input->dtype == TENSORFUSE_FLOAT16)
    return tk::fused_gemm_bias_gelu_fp16(input->data, weight->data, bias->data, output->data, M, N, K,
                                         alpha, beta, stream);
  if (input->dtype == TENSORFUSE_FLOAT32)
    return tk::fused_gemm_bias_gelu_fp32(input->data, weight->data, bias->data, output->data, M, N, K,
                                         alpha, beta, stream);
  return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
}

TensorFuseStatus tensorfuse_fused_softmax_dropout(const TensorFuseTensor* input,
                                                  TensorFuseTensor* output,
                                                  unsigned char* dropout_mask, float dropout_prob,
                                                  cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!input || !output) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (!(dropout_prob >= 0.0f && dropout_prob <= 1.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (input->shape.ndims != 4 || output->shape.ndims != 4) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  for (int i = 0; i < 4; ++i)
    if (input->shape.dims[i] != output->shape.dims[i] || input->shape.dims[i] < 0)
      return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (input->dtype != output->dtype) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (!dropout_mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (input->dtype != TENSORFUSE_FLOAT16 && input->dtype != TENSORFUSE_FLOAT32)
    return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (!input->data || !output->data) return TENSORFUSE_ERROR_INVALID_ARGUMENT;

  const unsigned long long seed = Runtime::get().next_seed();
  t_last_seed = seed;
  const long long rows =
      (long long)input->shape.dims[0] * input->shape.dims[1] * input->shape.dims[2];
  OwnerGuard og(output->data);
  return to_status(launch_softmax_dropout(input->data, output->data, dropout_mask, rows,
                                          input->shape.dims[3],
                                          input->dtype == TENSORFUSE_FLOAT16 ? kF16 : kF32,
                                          dropout_prob, seed, 0, stream));
}

// The reference validates and returns (src/tensorfuse_c_api.cpp:288-311); this
// computes.  query/output [batch, seq_q, hidden], key/value [batch, seq_kv,
// hidden] (src/tensorfuse/tensorfuse.h:95-98), heads split the hidden dimension,
// scores scaled by 1/sqrt(hidden / heads), dropout on the attention weights
// with a seed from the library's seed source.
TensorFuseStatus tensorfuse_fused_multi_head_attention(const TensorFuseTensor* query,
                                                       const TensorFuseTensor* key,
                                                       const TensorFuseTensor* value,
                                                       TensorFuseTensor* output, int num_heads,
                                                       float dropout_prob, cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!query || !key || !value || !output) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (num_heads <= 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (!(dropout_prob >= 0.0f && dropout_prob <= 1.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  const TensorFuseTensor* ts[4] = {query, key, value, output};
  for (const TensorFuseTensor* t : ts) {
    if (t->shape.ndims != 3) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
    for (int i = 0; i < 3; ++i)
      if (t->shape.dims[i] < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  }
  const int B = query->shape.dims[0], Sq = query->shape.dims[1], H = query->shape.dims[2];
  const int Skv = key->shape.dims[1];
  if (H % num_heads != 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (key->shape.dims[0] != B || value->shape.dims[0] != B || output->shape.dims[0] != B ||
      key->shape.dims[2] != H || value->shape.dims[2] != H || output->shape.dims[2] != H ||
      value->shape.dims[1] != Skv || output->shape.dims[1] != Sq)
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (query->dtype != key->dtype || query->dtype != value->dtype || query->dtype != output->dtype)
    return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (query->dtype != TENSORFUSE_FLOAT16 && query->dtype != TENSORFUSE_BFLOAT16 && query->dtype != TENSORFUSE_FLOAT32)
    return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (B == 0 || Sq == 0 || H == 0) return TENSORFUSE_SUCCESS;
  if (!query->data || !key->data || !value->data || !output->data) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  const unsigned long long seed = Runtime::get().next_seed();
  t_last_seed = seed;
  return tensorfuse_b200_attention(query->data, key->data, value->data, output->data, B, Sq, Skv, num_heads,
                                   H / num_heads, H, H, H, H, 0, 0, 0, 0, 0, 0, 0, 0,
                                   query->dtype == TENSORFUSE_FLOAT16 ? kF16 : query->dtype == TENSORFUSE_BFLOAT16 ? kBF16 : kF32,
                                   0.0f, dropout_prob, seed,
                                   nullptr, stream);
}

// tensorfuse_fused_transformer_layer: transformer_layer.cpp

TensorFuseStatus tensorfuse_autotune(const TensorFuseModelConfig* model_config, const char* output_path) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!model_config || !output_path) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_load_tuned_config(const char* config_path) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!config_path) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_start_profiling(const TensorFuseProfileConfig* profile_config) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!profile_config) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_stop_profiling(const char* output_path) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!output_path) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_allocate_tensor(TensorFuseTensor* tensor, const TensorFuseShape* shape,
                                            TensorFuseDataType dtype, int device_id) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!tensor || !shape) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (shape->ndims < 0 || shape->ndims > TENSORFUSE_MAX_DIMS) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  for (int i = 0; i < shape->ndims; ++i)
    if (shape->dims[i] < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const size_t bytes = tensorfuse_tensor_size_bytes(shape, dtype);
  void* data = nullptr;
  DeviceGuard g(device_id);
  if (cudaMalloc(&data, bytes ? bytes : 1) != cudaSuccess) {
    cudaGetLastError();
    return TENSORFUSE_ERROR_OUT_OF_MEMORY;
  }
  tensor->data = data;
  tensor->shape = *shape;
  tensor->dtype = dtype;
  tensor->layout = TENSORFUSE_LAYOUT_ROW_MAJOR;
  tensor->device_id = device_id;
  tensor->size_bytes = bytes;
  tensor->is_contiguous = true;
  tensor->scale = nullptr;
  tensor->zero_point = nullptr;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_free_tensor(TensorFuseTensor* tensor) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!tensor || !tensor->data) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (cudaFree(tensor->data) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  tensor->data = nullptr;
  tensor->size_bytes = 0;
  return TENSORFUSE_SUCCESS;
}

// ================================================================ additions
TensorFuseStatus tensorfuse_b200_gemm_int8(const void* A, const void* B, const void* bias, void* C,
                                           int M, int N, int K, float scale_A, float scale_B,
                                           int bias_dtype, int out_dtype, int epilogue,
                                           cudaStream_t stream) {
  if (epilogue != kEpiI8Dequant && epilogue != kEpiI8Legacy && epilogue != kEpiI8Raw)
    return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (epilogue == kEpiI8Raw) bias_dtype = kF32;
  return gemm_flat(A, B, bias, C, M, N, K, kI8, bias_dtype, out_dtype, epilogue, 1.0f, 1.0f,
                   scale_A * scale_B, nullptr, nullptr, stream);
}

TensorFuseStatus tensorfuse_b200_gemm_fp8(const void* A, const void* B, const void* bias, void* C, int M,
                                        int N, int K, float scale_A, float scale_B, int bias_dtype,
                                        int out_dtype, cudaStream_t stream) {
  if (out_dtype != kF16 && out_dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (bias_dtype != kF16 && bias_dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  return gemm_flat(A, B, bias, C, M, N, K, kFp8E4M3, bias_dtype, out_dtype, kEpiI8Dequant, 1.0f, 1.0f,
                   scale_A * scale_B, nullptr, nullptr, stream);
}

TensorFuseStatus tensorfuse_b200_softmax_dropout_rows(const void* input, void* output,
                                                      unsigned char* dropout_mask, long long rows,
                                                      int row_len, int dtype, float dropout_prob,
                                                      unsigned long long seed,
                                                      unsigned long long first_row,
                                                      cudaStream_t stream) {
  if (!input || !output || !dropout_mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (rows < 0 || row_len < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  OwnerGuard og(output);
  return to_status(launch_softmax_dropout(input, output, dropout_mask, rows, row_len, dtype,
                                          dropout_prob, seed, first_row, stream));
}

TensorFuseStatus tensorfuse_b200_softmax_dropout_masked(const void* input, void* output, unsigned char* dropout_mask,
                                                      long long batch, long long rows_per_item, int row_len,
                                                      int dtype, float scale, const int* kv_lengths,
                                                      float dropout_prob, unsigned long long seed,
                                                      cudaStream_t stream) {
  if (!input || !output || !dropout_mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (batch < 0 || rows_per_item <= 0 || row_len < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (!(scale > 0.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  OwnerGuard og(output);
  return to_status(launch_softmax_dropout_ext(input, output, dropout_mask, batch * rows_per_item, row_len, dtype,
                                              dropout_prob, seed, 0, scale, kv_lengths, rows_per_item, true, stream));
}

TensorFuseStatus tensorfuse_b200_gemm_bias_act(const void* A, const void* B, const void* bias, void* C, int M,
                                             int N, int K, int dtype, int activation, float alpha, float beta,
                                             cudaStream_t stream) {
  if (dtype != kF16 && dtype != kF32 && dtype != kBF16) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  int epi;
  if (activation == TENSORFUSE_ACTIVATION_GELU) epi = kEpiGelu;
  else if (activation == TENSORFUSE_ACTIVATION_NONE) epi = kEpiLinear;
  else return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  return gemm_flat(A, B, bias, C, M, N, K, dtype, dtype, dtype, epi, alpha, beta, 1.0f, nullptr, nullptr, stream);
}

TensorFuseStatus tensorfuse_b200_attention(const void* q, const void* k, const void* v, void* out, int batch,
                                         int seq_q, int seq_kv, int heads, int head_dim, long long ld_q,
                                         long long ld_k, long long ld_v, long long ld_o, long long hs_q,
                                         long long hs_k, long long hs_v, long long hs_o, long long bs_q,
                                         long long bs_k, long long bs_v, long long bs_o, int dtype, float scale,
                                         float dropout_prob, unsigned long long seed, const int* kv_lengths,
                                         cudaStream_t stream) {
  if (!q || !k || !v || !out) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (heads <= 0 || head_dim <= 0 || batch < 0 || seq_q < 0 || seq_kv < 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  AttnArgs a;
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.batch = batch; a.seq_q = seq_q; a.seq_kv = seq_kv; a.heads = heads; a.head_dim = head_dim;
  a.ld_q = ld_q; a.ld_k = ld_k; a.ld_v = ld_v; a.ld_o = ld_o;
  // zero strides select the packed [batch, seq, heads * head_dim] arrangement of a row pitch
  a.hs_q = hs_q ? hs_q : head_dim; a.hs_k = hs_k ? hs_k : head_dim;
  a.hs_v = hs_v ? hs_v : head_dim; a.hs_o = hs_o ? hs_o : head_dim;
  a.bs_q = bs_q ? bs_q : (long long)seq_q * ld_q; a.bs_k = bs_k ? bs_k : (long long)seq_kv * ld_k;
  a.bs_v = bs_v ? bs_v : (long long)seq_kv * ld_v; a.bs_o = bs_o ? bs_o : (long long)seq_q * ld_o;
  a.dtype = dtype; a.scale = scale; a.p = dropout_prob; a.seed = seed; a.kv_lengths = kv_lengths;
  OwnerGuard og(out);
  return to_status(launch_attention(a, stream));
}

TensorFuseStatus tensorfuse_b200_quantize_int8_columns(const void* w, int dtype, int K, int N, signed char* q,
                                                     float* scales_dev, cudaStream_t stream) {
  if (!w || !q || !scales_dev || K < 0 || N < 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  OwnerGuard og(q);
  return to_status(launch_quantize_int8_columns(w, dtype, K, N, q, scales_dev, stream));
}

TensorFuseStatus tensorfuse_b200_gemm_int8_channelwise(const void* A, const void* B, const void* bias, void* C, int M,
                                                     int N, int K, const float* scale_A_dev,
                                                     const float* scale_B_cols_dev, int bias_dtype, int out_dtype,
                                                     cudaStream_t stream) {
  if (!A || !B || !C || !bias || !scale_B_cols_dev) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (M <= 0 || N <= 0 || K <= 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (out_dtype != kF16 && out_dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (bias_dtype != kF16 && bias_dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  GemmArgs a{};
  a.A = A; a.B = B; a.bias = bias; a.C = C;
  a.M = M; a.N = N; a.K = K;
  a.in_dtype = kI8; a.bias_dtype = bias_dtype; a.out_dtype = out_dtype;
  a.epilogue = kEpiI8Dequant;
  a.alpha = 1.0f; a.beta = 1.0f; a.scale = 1.0f;
  a.scale_a_dev = scale_A_dev; a.scale_b_dev = nullptr; a.scale_b_cols = scale_B_cols_dev;
  OwnerGuard og(C);
  return to_status(launch_gemm(a, stream));
}

TensorFuseStatus tensorfuse_b200_quantize_int8(const void* x, int dtype, long long n, signed char* q,
                                             float* scale_dev, cudaStream_t stream) {
  if (!x || !q || !scale_dev || n < 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  OwnerGuard og(q);
  return to_status(launch_quantize_int8(x, dtype, n, q, scale_dev, stream));
}

TensorFuseStatus tensorfuse_b200_add_layernorm(const void* x, const void* residual, const void* gamma,
                                             const void* beta, void* out, long long rows, int hidden, int dtype,
                                             float eps, cudaStream_t stream) {
  if (!x || !gamma || !beta || !out || rows < 0 || hidden <= 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  OwnerGuard og(out);
  return to_status(launch_add_layernorm(x, residual, gamma, beta, out, rows, hidden, dtype, eps, stream));
}

void tensorfuse_b200_softmax_schedule(int row_len, int dtype, int aligned16, int* vec, int* warps) {
  const SoftmaxSchedule s = softmax_schedule(row_len, dtype, aligned16 != 0);
  if (vec) *vec = s.vec;
  if (warps) *warps = s.warps;
}

void tensorfuse_b200_softmax_schedule_ex(int row_len, int dtype, int aligned16, int* vec, int* warps, int* online) {
  const SoftmaxSchedule s = softmax_schedule(row_len, dtype, aligned16 != 0);
  if (vec) *vec = s.vec;
  if (warps) *warps = s.warps;
  if (online) *online = s.online;
}

void tensorfuse_b200_set_random_seed(unsigned long long seed) { Runtime::get().set_seed(seed); }
unsigned long long tensorfuse_b200_last_softmax_seed(void) { return t_last_seed; }

int tensorfuse_b200_device_count(void) { return (int)Runtime::get().devices().size(); }
int tensorfuse_b200_device_id(int i) {
  const std::vector<int> d = Runtime::get().devices();
  return (i >= 0 && (size_t)i < d.size()) ? d[i] : -1;
}

int tensorfuse_b200_watchdog_status(void) { return watchdog_status(); }
void tensorfuse_b200_watchdog_reset(void) { watchdog_reset(); }
unsigned long long tensorfuse_b200_launch_count(void) { return launch_count(); }

void tensorfuse_b200_plan_shards(long long rows, int parts, int align, long long* begins,
                                 long long* counts) {
  plan_shards(rows, parts, align, begins, counts);
}

}  // extern "C"
