/* tensorfuse/types.h -- ABI types of the TensorFuse C interface, B200 build.
 *
 * Binary layout (enumerator values, field order, field types) follows the
 * reference header src/tensorfuse/types.h so that a caller compiled against
 * the reference can be relinked against this library unchanged:
 *   TensorFuseStatus      reference src/tensorfuse/types.h:26-40
 *   TensorFuseDataType    reference src/tensorfuse/types.h:49-58
 *   TensorFuseLayout      reference src/tensorfuse/types.h:63-69
 *   TensorFuseActivation  reference src/tensorfuse/types.h:74-81
 *   TensorFuseShape       reference src/tensorfuse/types.h:98-102
 *   TensorFuseTensor      reference src/tensorfuse/types.h:104-114
 *   TensorFuseConfig      reference src/tensorfuse/types.h:123-132
 * Only the fields the two fused operators read are documented in detail.
 */
#ifndef TENSORFUSE_B200_TYPES_H_
#define TENSORFUSE_B200_TYPES_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

/* The stream argument is a CUDA stream handle.  Callers that do not include
 * the CUDA headers may treat it as an opaque pointer. */
#if defined(__CUDACC__) || defined(__CUDA_RUNTIME_H__) || defined(TENSORFUSE_WITH_CUDA_RUNTIME)
#include <cuda_runtime.h>
#else
typedef struct CUstream_st* cudaStream_t;
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TENSORFUSE_SUCCESS = 0,
  TENSORFUSE_ERROR_INVALID_ARGUMENT = 1,
  TENSORFUSE_ERROR_CUDA_ERROR = 2,
  TENSORFUSE_ERROR_OUT_OF_MEMORY = 3,
  TENSORFUSE_ERROR_NOT_INITIALIZED = 4,
  TENSORFUSE_ERROR_INVALID_CONFIGURATION = 5,
  TENSORFUSE_ERROR_KERNEL_LAUNCH_FAILED = 6,
  TENSORFUSE_ERROR_AUTOTUNER_FAILED = 7,
  TENSORFUSE_ERROR_PROFILING_FAILED = 8,
  TENSORFUSE_ERROR_FILE_IO = 9,
  TENSORFUSE_ERROR_UNSUPPORTED_OPERATION = 10,
  TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE = 11,
  TENSORFUSE_ERROR_UNKNOWN = 99
} TensorFuseStatus;

typedef enum {
  TENSORFUSE_FLOAT32 = 0,
  TENSORFUSE_FLOAT16 = 1,
  TENSORFUSE_BFLOAT16 = 2,
  TENSORFUSE_INT8 = 3,
  TENSORFUSE_UINT8 = 4,
  TENSORFUSE_INT32 = 5,
  TENSORFUSE_FP8_E4M3 = 6,
  TENSORFUSE_FP8_E5M2 = 7
} TensorFuseDataType;

typedef enum {
  TENSORFUSE_LAYOUT_ROW_MAJOR = 0,
  TENSORFUSE_LAYOUT_COL_MAJOR = 1,
  TENSORFUSE_LAYOUT_NCHW = 2,
  TENSORFUSE_LAYOUT_NHWC = 3,
  TENSORFUSE_LAYOUT_CUSTOM = 4
} TensorFuseLayout;

typedef enum {
  TENSORFUSE_ACTIVATION_NONE = 0,
  TENSORFUSE_ACTIVATION_RELU = 1,
  TENSORFUSE_ACTIVATION_GELU = 2,
  TENSORFUSE_ACTIVATION_SILU = 3,
  TENSORFUSE_ACTIVATION_TANH = 4,
  TENSORFUSE_ACTIVATION_SIGMOID = 5
} TensorFuseActivation;

#define TENSORFUSE_MAX_DIMS 8

typedef struct {
  int ndims;
  int dims[TENSORFUSE_MAX_DIMS];
  int strides[TENSORFUSE_MAX_DIMS]; /* carried, never read: tensors are dense row-major */
} TensorFuseShape;

typedef struct {
  void* data;             /* device pointer, owned by the caller                     */
  TensorFuseShape shape;
  TensorFuseDataType dtype;
  TensorFuseLayout layout; /* carried, never read                                     */
  int device_id;           /* carried, never read                                     */
  size_t size_bytes;       /* carried, never read                                     */
  bool is_contiguous;      /* carried, never read                                     */
  void* scale;             /* INT8 only: device pointer to one float, may be NULL (=1) */
  void* zero_point;        /* carried, never read (quantisation is symmetric)         */
} TensorFuseTensor;

typedef struct {
  int device_count;            /* devices the batch/token dimension is sharded over; <=0 means 1 */
  int* device_ids;             /* device_count ordinals, NULL means 0..device_count-1            */
  size_t workspace_size_bytes; /* per-device staging pool used by the host-buffer entry points   */
  bool enable_profiling;
  bool enable_autotuning;
  bool enable_fp8;
  int log_level;               /* 0 quiet, 1 info, 2 debug */
  const char* cache_dir;
} TensorFuseConfig;

typedef struct {
  int batch_size, seq_length, hidden_dim, num_heads, ffn_dim, num_layers;
  TensorFuseDataType dtype;
  bool use_flash_attention, use_mixed_precision;
  const char* model_name;
} TensorFuseModelConfig;

typedef struct {
  TensorFuseTensor *query_weight, *key_weight, *value_weight, *output_weight;
  TensorFuseTensor *query_bias, *key_bias, *value_bias, *output_bias;
  TensorFuseTensor *ffn_weight1, *ffn_weight2, *ffn_bias1, *ffn_bias2;
  TensorFuseTensor *ln1_weight, *ln1_bias, *ln2_weight, *ln2_bias;
  int num_heads;
  float dropout_prob;
  TensorFuseActivation ffn_activation;
  float layer_norm_eps;
  bool use_bias, use_flash_attention;
} TensorFuseTransformerParams;

typedef struct {
  bool enable_nsight_systems, enable_nsight_compute, enable_nvtx, enable_cuda_events,
      enable_memory_tracking;
  const char* output_prefix;
  int warmup_iterations, profile_iterations;
} TensorFuseProfileConfig;

typedef struct {
  float kernel_time_ms, memory_bandwidth_gbps, tensor_core_utilization, flops_per_second;
  size_t memory_used_bytes, memory_peak_bytes;
  int num_kernel_launches;
  float cpu_time_ms, total_time_ms;
} TensorFuseMetrics;

/* reference src/tensorfuse/types.h:226-253: carried for source compatibility;
 * no entry point of either library reads them. */
typedef struct {
  int tile_m, tile_n, tile_k, warp_m, warp_n, warp_k, stages, split_k;
} TensorFuseKernelConfig;

typedef struct {
  int max_iterations;
  float time_limit_seconds;
  int num_warmup_runs, num_timing_runs;
  float relative_threshold;
  bool use_heuristics, cache_results;
  const char* cache_file;
} TensorFuseAutotunerConfig;

static inline size_t tensorfuse_sizeof_dtype(TensorFuseDataType t) {
  switch (t) {
    case TENSORFUSE_FLOAT32: case TENSORFUSE_INT32: return 4;
    case TENSORFUSE_FLOAT16: case TENSORFUSE_BFLOAT16: return 2;
    case TENSORFUSE_INT8: case TENSORFUSE_UINT8:
    case TENSORFUSE_FP8_E4M3: case TENSORFUSE_FP8_E5M2: return 1;
    default: return 0;
  }
}

static inline size_t tensorfuse_tensor_size_bytes(const TensorFuseShape* s, TensorFuseDataType t) {
  size_t n = 1;
  for (int i = 0; i < s->ndims; ++i) n *= (size_t)s->dims[i];
  return n * tensorfuse_sizeof_dtype(t);
}

#ifdef __cplusplus
}

/* C++ spellings of the types above, and the two C++-only structures the
 * namespace interface returns.  reference src/tensorfuse/types.h:293-332 */
#include <string>
namespace tensorfuse {
using Status = TensorFuseStatus;
using DataType = TensorFuseDataType;
using Layout = TensorFuseLayout;
using Activation = TensorFuseActivation;
using Shape = TensorFuseShape;
using Tensor = TensorFuseTensor;
using Config = TensorFuseConfig;
using ModelConfig = TensorFuseModelConfig;
using TransformerParams = TensorFuseTransformerParams;
using ProfileConfig = TensorFuseProfileConfig;
using Metrics = TensorFuseMetrics;
using KernelConfig = TensorFuseKernelConfig;
using AutotunerConfig = TensorFuseAutotunerConfig;

struct DeviceInfo {
  int device_id;
  std::string device_name;
  int compute_capability_major;
  int compute_capability_minor;
  size_t total_global_memory;
  int multiprocessor_count;
  int max_threads_per_block;
  size_t max_shared_memory_per_block;
  bool supports_tensor_cores;
  bool supports_fp16;
  bool supports_bf16;
  bool supports_fp8;
};

struct MemoryStats {
  size_t total_allocated; /* bytes handed out by allocate_device and not yet returned */
  size_t free_memory;     /* cudaMemGetInfo of the library's device                    */
  size_t used_memory;
  size_t peak_usage;      /* high-water mark of total_allocated                        */
  size_t num_blocks;
};
}  // namespace tensorfuse
#endif
#endif /* TENSORFUSE_B200_TYPES_H_ */
