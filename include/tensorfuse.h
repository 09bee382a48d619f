/* tensorfuse.h -- the C++ `namespace tensorfuse` interface of TensorFuse
 * (flat device pointers and sizes), implemented by libtensorfuse.so.
 *
 * The reference declares this interface in src/tensorfuse.h:36-246 and never
 * defines it; its README quick start (README.md:36-40, 221-230) is written
 * against it.  Every declaration below keeps the reference's name, argument
 * order and defaults and cites the line it stands for.
 *
 * Two parts of the reference header are deliberately absent:
 *   - its trailing `extern "C"` block (src/tensorfuse.h:254-313) re-declares
 *     tensorfuse_init / tensorfuse_fused_gemm_bias_gelu / ... with signatures
 *     that differ from the struct interface of tensorfuse/tensorfuse.h under
 *     the same C symbol names; one library cannot export both, and the struct
 *     interface is the one the reference implements;
 *   - runtime::RuntimeContext is declared here as a small query class; the
 *     reference's version (src/runtime/runtime_context.h) additionally owns
 *     cuBLAS / cuDNN / cuRAND handles and a memory pool that no operator uses.
 */
#ifndef TENSORFUSE_B200_CXX_API_H_
#define TENSORFUSE_B200_CXX_API_H_

#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "tensorfuse/profiler.h"
#include "tensorfuse/tensorfuse.h"
#include "tensorfuse/types.h"

namespace tensorfuse {

namespace runtime {
/* reference src/runtime/runtime_context.h:29-211 (query and stream subset). */
class RuntimeContext {
 public:
  TensorFuseStatus initialize(int device_id = -1);
  void cleanup();
  bool is_initialized() const;
  int get_device_id() const;
  cudaStream_t get_main_stream() const;   /* the stream operators use when given nullptr: the default stream */
  cudaStream_t create_stream();
  void destroy_stream(cudaStream_t stream);
  TensorFuseStatus synchronize();
  TensorFuseStatus synchronize_stream(cudaStream_t stream = nullptr);
  const cudaDeviceProp& get_device_properties() const;
  int get_compute_capability_major() const;
  int get_compute_capability_minor() const;
  int get_multiprocessor_count() const;
  int get_max_threads_per_block() const;
  size_t get_max_shared_memory_per_block() const;
  size_t get_total_global_memory() const;
  bool supports_tensor_cores() const;
  bool supports_fp16() const;
  bool supports_bf16() const;
  bool supports_fp8() const;
  TensorFuseStatus set_random_seed(unsigned long long seed);
  RuntimeContext(const RuntimeContext&) = delete;
  RuntimeContext& operator=(const RuntimeContext&) = delete;
  RuntimeContext() = default;

 private:
  int device_id_ = -1;
  bool initialized_ = false;
  cudaDeviceProp props_{};
};
}  // namespace runtime

/* reference src/tensorfuse.h:36.  device_id -1 keeps the calling thread's
 * current device.  Initialises the library for that one device (the struct
 * interface's tensorfuse_init with a one-entry device list); idempotent. */
TensorFuseStatus initialize(int device_id = -1);
/* reference src/tensorfuse.h:41 */
void cleanup();
/* reference src/tensorfuse.h:47 */
runtime::RuntimeContext& get_context();
/* reference src/tensorfuse.h:53 */
DeviceInfo get_device_info();
/* reference src/tensorfuse.h:60 (a no-op in the reference's binding): seeds the
 * dropout stream of fused_softmax_dropout. */
TensorFuseStatus set_random_seed(unsigned long long seed);

/* output[M,N] = gelu(alpha * A[M,K] * B[K,N] + beta * bias[N]), all row-major
 * device memory of `data_type` (FLOAT32, FLOAT16 or BFLOAT16).
 * reference src/tensorfuse.h:84-94 */
TensorFuseStatus fused_gemm_bias_gelu(const void* A, const void* B, const void* bias, void* output,
                                      int M, int N, int K, DataType data_type, float alpha = 1.0f,
                                      float beta = 1.0f, cudaStream_t stream = nullptr);

/* Softmax over the last axis of a [batch_size, num_heads, seq_len, head_dim]
 * tensor, then dropout; dropout_mask has one byte per element.  NOTE: the
 * argument order here is (seq_len, num_heads, head_dim); the kernel-level
 * wrappers of tensorfuse_b200.h take (seq_len, head_dim, num_heads).  For
 * attention probabilities [B, H, S, S] pass seq_len = S and head_dim = S.
 * reference src/tensorfuse.h:113-124 */
TensorFuseStatus fused_softmax_dropout(const void* input, void* output, unsigned char* dropout_mask,
                                       int batch_size, int seq_len, int num_heads, int head_dim,
                                       float dropout_prob, DataType data_type,
                                       cudaStream_t stream = nullptr);

/* reference src/tensorfuse.h:136-157.  `alignment` above 256 bytes is honoured
 * by over-allocation; the returned pointer must go back to the matching
 * deallocate function.  Host memory is page-locked. */
void* allocate_device(size_t size, size_t alignment = 128);
void deallocate_device(void* ptr);
void* allocate_host(size_t size, size_t alignment = 128);
void deallocate_host(void* ptr);

/* reference src/tensorfuse.h:167-177.  With a null stream the copy is
 * synchronous, otherwise it is enqueued on the stream. */
TensorFuseStatus copy_host_to_device(void* dst, const void* src, size_t size, cudaStream_t stream = nullptr);
TensorFuseStatus copy_device_to_host(void* dst, const void* src, size_t size, cudaStream_t stream = nullptr);
/* reference src/tensorfuse.h:183 */
MemoryStats get_memory_stats();

/* reference src/tensorfuse.h:193-212 */
cudaStream_t create_stream();
void destroy_stream(cudaStream_t stream);
TensorFuseStatus synchronize();
TensorFuseStatus synchronize_stream(cudaStream_t stream = nullptr);

/* reference src/tensorfuse.h:222-246 */
const char* get_version();
const char* get_build_info();
const char* get_error_string(TensorFuseStatus status);
bool is_gpu_supported();
std::vector<DataType> get_supported_data_types();

}  // namespace tensorfuse

#endif /* TENSORFUSE_B200_CXX_API_H_ */
