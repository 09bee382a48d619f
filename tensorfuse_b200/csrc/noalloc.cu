// noalloc.cu -- softmax+dropout on host buffers for callers that must not
// allocate device memory.
//
// tensorfuse_b200_softmax_dropout_host stages its operands in device buffers it
// obtains with cudaMalloc and grows on demand.  That is unusable for a caller
// whose process has handed all device memory to another allocator (a framework's
// caching pool, an MPS / MIG memory cap that is already reached), and unwelcome
// for a serving thread that cannot afford the device-wide synchronisation a
// cudaMalloc or cudaFree implies.  The entry point below runs the same kernel on
// a fixed staging area that is part of the library image: a file-scope
// __device__ array.  Every GPU that loads the library carries those 16 MiB until
// the process exits; nothing is allocated or freed at run time.
//
// The array's name is only a host-side handle.  Its device address is looked up
// once per device with cudaGetSymbolAddress (with that device current) and it is
// that address which is handed to the copies and to the kernel.
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "runtime.h"
#include "tensorfuse_b200.h"

namespace {

constexpr size_t kScratchBytes = size_t(16) << 20;   // 16 MiB per device
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {};

// Device address of the staging area on the current device; the first call on
// a device resolves the symbol.  Returns nullptr (and sets *err) on failure.
unsigned char* scratch_on_current_device(cudaError_t* err) {
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) { *err = cudaErrorInvalidDevice; return nullptr; }
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    *err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (*err != cudaSuccess) return nullptr;
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  return g_scratch_addr[dev];
}

size_t round_up_256(size_t n) { return (n + 255) & ~size_t(255); }

}  // namespace

extern "C" TensorFuseStatus tensorfuse_b200_softmax_dropout_host_noalloc(
    const void* input, void* output, unsigned char* dropout_mask, long long rows, int row_len, int dtype,
    float dropout_prob, unsigned long long seed, cudaStream_t stream) {
  using namespace tfb;
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!input || !output || !dropout_mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (!(dropout_prob >= 0.0f && dropout_prob <= 1.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (rows < 0 || row_len < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (dtype != kF16 && dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (rows == 0 || row_len == 0) return TENSORFUSE_SUCCESS;

  // Staging layout: [input | output | mask], each part 256-byte aligned.
  const size_t es = dtype == kF16 ? 2 : 4;
  const size_t elems = (size_t)rows * (size_t)row_len;
  if (elems / (size_t)row_len != (size_t)rows) return TENSORFUSE_ERROR_OUT_OF_MEMORY;
  const size_t data_bytes = round_up_256(elems * es), mask_bytes = round_up_256(elems);
  if (elems > kScratchBytes || 2 * data_bytes + mask_bytes > kScratchBytes)
    return TENSORFUSE_ERROR_OUT_OF_MEMORY;   // larger than the fixed staging area: use the allocating entry point

  cudaError_t err;
  unsigned char* base = scratch_on_current_device(&err);
  if (!base) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  unsigned char* d_in = base;
  unsigned char* d_out = base + data_bytes;
  unsigned char* d_mask = base + 2 * data_bytes;

  if (cudaMemcpyAsync(d_in, input, elems * es, cudaMemcpyHostToDevice, stream) != cudaSuccess) {
    cudaGetLastError();
    return TENSORFUSE_ERROR_CUDA_ERROR;
  }
  const LaunchResult lr =
      launch_softmax_dropout(d_in, d_out, d_mask, rows, row_len, dtype, dropout_prob, seed, 0, stream);
  if (lr != kOk) {
    cudaStreamSynchronize(stream);
    return lr == kInvalidArgument ? TENSORFUSE_ERROR_INVALID_ARGUMENT
         : lr == kUnsupported     ? TENSORFUSE_ERROR_UNSUPPORTED_OPERATION
                                  : TENSORFUSE_ERROR_CUDA_ERROR;
  }
  if (cudaMemcpyAsync(output, d_out, elems * es, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaMemcpyAsync(dropout_mask, d_mask, elems, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    // whatever was enqueued before the failure must not still be using the shared
    // staging area, or writing the caller's buffers, once this call has returned
    cudaStreamSynchronize(stream);
    cudaGetLastError();
    return TENSORFUSE_ERROR_CUDA_ERROR;
  }
  return TENSORFUSE_SUCCESS;
}
