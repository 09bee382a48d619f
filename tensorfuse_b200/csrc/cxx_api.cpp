// cxx_api.cpp -- the C++ `namespace tensorfuse` interface (include/tensorfuse.h)
// and the two benchmark-side helpers tensorfuse_simple_init / _cleanup.
//
// The reference declares the namespace interface (src/tensorfuse.h:36-246) and
// has no definition for any of it; here every function is a thin layer over
// the launchers of kernels.h, the runtime singleton and the CUDA runtime.
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "kernels.h"
#include "runtime.h"
#include "tensorfuse.h"
#include "tensorfuse/kernels.h"
#include "tensorfuse_b200.h"

using namespace tfb;

namespace {

std::mutex g_alloc_mu;
// user pointer -> (pointer to hand back to the CUDA runtime, bytes)
std::unordered_map<void*, std::pair<void*, size_t>> g_dev_allocs, g_host_allocs;
size_t g_dev_bytes = 0, g_dev_peak = 0;

TensorFuseStatus from_cuda(cudaError_t e) {
  if (e == cudaSuccess) return TENSORFUSE_SUCCESS;
  cudaGetLastError();
  return e == cudaErrorMemoryAllocation ? TENSORFUSE_ERROR_OUT_OF_MEMORY : TENSORFUSE_ERROR_CUDA_ERROR;
}

size_t pad_for(size_t alignment) {
  // cudaMalloc / cudaHostAlloc return at least 256-byte aligned memory
  if (alignment <= 256 || (alignment & (alignment - 1)) != 0) return 0;
  return alignment;
}

void* align_up(void* p, size_t alignment) {
  if (pad_for(alignment) == 0) return p;
  const uintptr_t v = reinterpret_cast<uintptr_t>(p);
  return reinterpret_cast<void*>((v + alignment - 1) & ~(uintptr_t)(alignment - 1));
}

}  // namespace

namespace tensorfuse {

// --------------------------------------------------------------- context
namespace runtime {

TensorFuseStatus RuntimeContext::initialize(int device_id) {
  int dev = device_id;
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  if (dev >= count) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (initialized_ && dev == device_id_) return TENSORFUSE_SUCCESS;
  TensorFuseStatus st = from_cuda(cudaSetDevice(dev));
  if (st != TENSORFUSE_SUCCESS) return st;
  st = from_cuda(cudaGetDeviceProperties(&props_, dev));
  if (st != TENSORFUSE_SUCCESS) return st;
  TensorFuseConfig cfg{};
  int ids[1] = {dev};
  cfg.device_count = 1;
  cfg.device_ids = ids;
  cfg.workspace_size_bytes = size_t(1) << 30;
  cfg.enable_autotuning = true;
  cfg.log_level = 0;
  cfg.cache_dir = "./cache";
  st = Runtime::get().init(&cfg);
  if (st != TENSORFUSE_SUCCESS) return st;
  device_id_ = dev;
  initialized_ = true;
  return TENSORFUSE_SUCCESS;
}

void RuntimeContext::cleanup() {
  if (!initialized_) return;
  Runtime::get().shutdown();
  initialized_ = false;
  device_id_ = -1;
}

bool RuntimeContext::is_initialized() const { return initialized_; }
int RuntimeContext::get_device_id() const { return device_id_; }
cudaStream_t RuntimeContext::get_main_stream() const { return nullptr; }

cudaStream_t RuntimeContext::create_stream() {
  DeviceGuard g(device_id_);
  cudaStream_t s = nullptr;
  if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  return s;
}
void RuntimeContext::destroy_stream(cudaStream_t stream) {
  if (stream) cudaStreamDestroy(stream);
}
TensorFuseStatus RuntimeContext::synchronize() {
  DeviceGuard g(device_id_);
  return from_cuda(cudaDeviceSynchronize());
}
TensorFuseStatus RuntimeContext::synchronize_stream(cudaStream_t stream) {
  DeviceGuard g(device_id_);
  return from_cuda(cudaStreamSynchronize(stream));
}
const cudaDeviceProp& RuntimeContext::get_device_properties() const { return props_; }
int RuntimeContext::get_compute_capability_major() const { return props_.major; }
int RuntimeContext::get_compute_capability_minor() const { return props_.minor; }
int RuntimeContext::get_multiprocessor_count() const { return props_.multiProcessorCount; }
int RuntimeContext::get_max_threads_per_block() const { return props_.maxThreadsPerBlock; }
size_t RuntimeContext::get_max_shared_memory_per_block() const { return props_.sharedMemPerBlockOptin; }
size_t RuntimeContext::get_total_global_memory() const { return props_.totalGlobalMem; }
// The kernels of this library are sm_100a code: "supported" means a compute
// capability 10.x device, on which all four operand families run.
bool RuntimeContext::supports_tensor_cores() const { return props_.major == 10; }
bool RuntimeContext::supports_fp16() const { return props_.major == 10; }
bool RuntimeContext::supports_bf16() const { return props_.major == 10; }
bool RuntimeContext::supports_fp8() const { return props_.major == 10; }
TensorFuseStatus RuntimeContext::set_random_seed(unsigned long long seed) {
  Runtime::get().set_seed(seed);
  return TENSORFUSE_SUCCESS;
}

}  // namespace runtime

runtime::RuntimeContext& get_context() {
  static runtime::RuntimeContext ctx;
  return ctx;
}

TensorFuseStatus initialize(int device_id) { return get_context().initialize(device_id); }
void cleanup() { get_context().cleanup(); }

DeviceInfo get_device_info() {
  DeviceInfo info{};
  int dev = get_context().get_device_id();
  if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); info.device_id = -1; return info; }
  cudaDeviceProp p{};
  if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) { cudaGetLastError(); info.device_id = -1; return info; }
  info.device_id = dev;
  info.device_name = p.name;
  info.compute_capability_major = p.major;
  info.compute_capability_minor = p.minor;
  info.total_global_memory = p.totalGlobalMem;
  info.multiprocessor_count = p.multiProcessorCount;
  info.max_threads_per_block = p.maxThreadsPerBlock;
  info.max_shared_memory_per_block = p.sharedMemPerBlockOptin;
  info.supports_tensor_cores = info.supports_fp16 = info.supports_bf16 = info.supports_fp8 = p.major == 10;
  return info;
}

TensorFuseStatus set_random_seed(unsigned long long seed) { return get_context().set_random_seed(seed); }

// ------------------------------------------------------------- operators
TensorFuseStatus fused_gemm_bias_gelu(const void* A, const void* B, const void* bias, void* output, int M, int N,
                                      int K, DataType data_type, float alpha, float beta, cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  switch (data_type) {
    case TENSORFUSE_FLOAT32:
      return kernels::fused_gemm_bias_gelu_fp32(A, B, bias, output, M, N, K, alpha, beta, stream);
    case TENSORFUSE_FLOAT16:
      return kernels::fused_gemm_bias_gelu_fp16(A, B, bias, output, M, N, K, alpha, beta, stream);
    case TENSORFUSE_BFLOAT16:
      return tensorfuse_b200_gemm_bias_act(A, B, bias, output, M, N, K, kBF16, TENSORFUSE_ACTIVATION_GELU, alpha,
                                           beta, stream);
    default:
      return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  }
}

TensorFuseStatus fused_softmax_dropout(const void* input, void* output, unsigned char* dropout_mask, int batch_size,
                                       int seq_len, int num_heads, int head_dim, float dropout_prob,
                                       DataType data_type, cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!(dropout_prob >= 0.0f && dropout_prob <= 1.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (data_type != TENSORFUSE_FLOAT16 && data_type != TENSORFUSE_FLOAT32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  const unsigned long long seed = Runtime::get().next_seed();
  // the kernel-level entry points take (seq_len, head_dim, num_heads)
  if (data_type == TENSORFUSE_FLOAT16)
    return kernels::fused_softmax_dropout_fp16(input, output, dropout_mask, batch_size, seq_len, head_dim, num_heads,
                                               dropout_prob, seed, stream);
  return kernels::fused_softmax_dropout_fp32(input, output, dropout_mask, batch_size, seq_len, head_dim, num_heads,
                                             dropout_prob, seed, stream);
}

// ---------------------------------------------------------------- memory
void* allocate_device(size_t size, size_t alignment) {
  DeviceGuard g(get_context().get_device_id());
  const size_t pad = pad_for(alignment);
  void* raw = nullptr;
  if (cudaMalloc(&raw, (size ? size : 1) + pad) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  void* user = align_up(raw, alignment);
  std::lock_guard<std::mutex> lk(g_alloc_mu);
  g_dev_allocs[user] = {raw, size};
  g_dev_bytes += size;
  if (g_dev_bytes > g_dev_peak) g_dev_peak = g_dev_bytes;
  return user;
}

void deallocate_device(void* ptr) {
  if (!ptr) return;
  void* raw = ptr;
  {
    std::lock_guard<std::mutex> lk(g_alloc_mu);
    auto it = g_dev_allocs.find(ptr);
    if (it != g_dev_allocs.end()) {
      raw = it->second.first;
      g_dev_bytes -= it->second.second;
      g_dev_allocs.erase(it);
    }
  }
  if (cudaFree(raw) != cudaSuccess) cudaGetLastError();
}

void* allocate_host(size_t size, size_t alignment) {
  const size_t pad = pad_for(alignment);
  void* raw = nullptr;
  if (cudaHostAlloc(&raw, (size ? size : 1) + pad, cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  void* user = align_up(raw, alignment);
  std::lock_guard<std::mutex> lk(g_alloc_mu);
  g_host_allocs[user] = {raw, size};
  return user;
}

void deallocate_host(void* ptr) {
  if (!ptr) return;
  void* raw = ptr;
  {
    std::lock_guard<std::mutex> lk(g_alloc_mu);
    auto it = g_host_allocs.find(ptr);
    if (it != g_host_allocs.end()) {
      raw = it->second.first;
      g_host_allocs.erase(it);
    }
  }
  if (cudaFreeHost(raw) != cudaSuccess) cudaGetLastError();
}

TensorFuseStatus copy_host_to_device(void* dst, const void* src, size_t size, cudaStream_t stream) {
  if ((!dst || !src) && size != 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (size == 0) return TENSORFUSE_SUCCESS;
  if (stream == nullptr) return from_cuda(cudaMemcpy(dst, src, size, cudaMemcpyHostToDevice));
  return from_cuda(cudaMemcpyAsync(dst, src, size, cudaMemcpyHostToDevice, stream));
}

TensorFuseStatus copy_device_to_host(void* dst, const void* src, size_t size, cudaStream_t stream) {
  if ((!dst || !src) && size != 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (size == 0) return TENSORFUSE_SUCCESS;
  if (stream == nullptr) return from_cuda(cudaMemcpy(dst, src, size, cudaMemcpyDeviceToHost));
  return from_cuda(cudaMemcpyAsync(dst, src, size, cudaMemcpyDeviceToHost, stream));
}

MemoryStats get_memory_stats() {
  MemoryStats s{};
  DeviceGuard g(get_context().get_device_id());
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) cudaGetLastError();
  std::lock_guard<std::mutex> lk(g_alloc_mu);
  s.total_allocated = g_dev_bytes;
  s.free_memory = free_b;
  s.used_memory = total_b - free_b;
  s.peak_usage = g_dev_peak;
  s.num_blocks = g_dev_allocs.size();
  return s;
}

// --------------------------------------------------------------- streams
cudaStream_t create_stream() { return get_context().create_stream(); }
void destroy_stream(cudaStream_t stream) { get_context().destroy_stream(stream); }
TensorFuseStatus synchronize() { return get_context().synchronize(); }
TensorFuseStatus synchronize_stream(cudaStream_t stream) { return get_context().synchronize_stream(stream); }

// ------------------------------------------------------------- utilities
const char* get_version() { return tensorfuse_get_version(); }
const char* get_build_info() { return "tensorfuse " TENSORFUSE_VERSION_STRING " (sm_100a: TMA + tcgen05 kernels)"; }
const char* get_error_string(TensorFuseStatus status) { return tensorfuse_get_error_string(status); }

bool is_gpu_supported() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return major == 10;
}

std::vector<DataType> get_supported_data_types() {
  if (!is_gpu_supported()) return {};
  return {TENSORFUSE_FLOAT32, TENSORFUSE_FLOAT16, TENSORFUSE_BFLOAT16, TENSORFUSE_INT8, TENSORFUSE_FP8_E4M3};
}

}  // namespace tensorfuse

// ------------------------------------------------ benchmark-side helpers
// reference benchmarks/tensorfuse_wrappers.cpp:30-46 (compiled into the
// reference's benchmark programs, declared in benchmarks/tensorfuse_c_api.h:33-38):
// select the device, nothing else.  Exported here so that those programs link
// against the library alone.  The return type is an int-sized enum whose only
// portable value is 0 (the benchmark header has its own enumerators).
extern "C" {
TensorFuseStatus tensorfuse_simple_init(int device_id) {
  if (cudaSetDevice(device_id) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  return TENSORFUSE_SUCCESS;
}
void tensorfuse_simple_cleanup(void) {}

// ------------------------------------------ helpers of the Python binding
// What the reference's pybind module does with the CUDA runtime directly
// (src/python/core_bindings.cpp:402-461 copies, memory_bindings.cpp:46-61 and
// core_bindings.cpp:830-838, which return constants instead of asking the device).
TensorFuseStatus tensorfuse_b200_memcpy(void* dst, const void* src, size_t bytes, int kind) {
  if (bytes == 0) return TENSORFUSE_SUCCESS;
  if (!dst || !src) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  cudaMemcpyKind k;
  switch (kind) {
    case 1: k = cudaMemcpyHostToDevice; break;
    case 2: k = cudaMemcpyDeviceToHost; break;
    case 3: k = cudaMemcpyDeviceToDevice; break;
    default: return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  }
  return from_cuda(cudaMemcpy(dst, src, bytes, k));
}

TensorFuseStatus tensorfuse_b200_mem_info(int device, size_t* free_bytes, size_t* total_bytes) {
  if (!free_bytes || !total_bytes) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  DeviceGuard g(device);
  return from_cuda(cudaMemGetInfo(free_bytes, total_bytes));
}

TensorFuseStatus tensorfuse_b200_device_info(int device, char* name, int name_capacity, int* cc_major, int* cc_minor,
                                             size_t* total_memory, int* multiprocessors) {
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  cudaDeviceProp p{};
  const TensorFuseStatus st = from_cuda(cudaGetDeviceProperties(&p, device));
  if (st != TENSORFUSE_SUCCESS) return st;
  if (name && name_capacity > 0) {
    int i = 0;
    for (; i < name_capacity - 1 && p.name[i]; ++i) name[i] = p.name[i];
    name[i] = 0;
  }
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  if (total_memory) *total_memory = p.totalGlobalMem;
  if (multiprocessors) *multiprocessors = p.multiProcessorCount;
  return TENSORFUSE_SUCCESS;
}
}
