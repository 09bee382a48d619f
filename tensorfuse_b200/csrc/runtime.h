// runtime.h -- process-wide state of the library: the initialised flag, the
// device list chosen at init, per-device streams / events / staging buffers for
// the host-buffer operators, the dropout seed source and the watchdog word.
//
// Stands where the reference has src/runtime/runtime_context.{h,cpp} and
// memory_manager.{h,cpp} (a single-device context with cuBLAS/cuDNN/cuRAND
// handles and a first-fit pool that no operator ever calls): here the state is
// what the two fused operators actually need, and the device list is honoured.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "tensorfuse/types.h"

namespace tfb {

// Grow-only device buffer.
struct DevBuffer {
  void* ptr = nullptr;
  size_t cap = 0;
  cudaError_t reserve(size_t bytes);
  void release();
};

// Per-device state of the host-buffer operators.  One call at a time may use
// it: the operators hold `mu` from the first reservation to the final
// synchronisation, so concurrent callers are serialised per device.
struct DeviceCtx {
  int id = 0;
  bool ready = false;
  std::mutex mu;
  // device copies of host weight ranges registered as immutable, keyed by host address
  std::map<const void*, DevBuffer> weights;
  cudaStream_t s_in = nullptr, s_compute = nullptr, s_out = nullptr;
  std::vector<cudaEvent_t> ev_in, ev_done;  // one pair per in-flight chunk
  cudaEvent_t ev_weights = nullptr;
  DevBuffer a, b, bias, c, mask;            // staging for the host-buffer operators
  cudaError_t ensure(size_t chunks);
  void destroy();
};

class Runtime {
 public:
  static Runtime& get();
  TensorFuseStatus init(const TensorFuseConfig* cfg);
  TensorFuseStatus shutdown();
  bool initialized();
  int log_level();
  std::vector<int> devices();
  DeviceCtx* ctx(size_t i);  // i-th selected device; contexts are created lazily

  // Host ranges the caller has declared immutable: the host-buffer operators
  // keep one device copy per selected device instead of uploading per call.
  // Concatenated copy of three registered device weight matrices (and biases),
  // kept per device until the registration of any of them is invalidated.
  // Returns null when it has to be (re)built: the caller fills `*slot` then.
  struct FusedQkv {
    std::mutex mu;       // held while the copy is (re)built: two first calls may arrive together
    void* w = nullptr; void* b = nullptr; size_t w_bytes = 0, b_bytes = 0;
  };
  FusedQkv* fused_qkv_slot(int device, const void* wq, const void* wk, const void* wv, bool* fresh);
  void register_weights(const void* host_ptr, size_t bytes);
  void invalidate_weights(const void* host_ptr);   // null: all of them
  size_t registered_bytes(const void* host_ptr);   // 0 when not registered

  // Stream-ordered workspace pool owned by the library, one per device, created
  // on first use and destroyed at shutdown.  Its release threshold is unlimited,
  // so workspace freed by one call is reused by the next without a trip to the
  // driver; the device's default pool (shared with the host process) is left alone.
  cudaMemPool_t workspace_pool(int device);

  void set_seed(unsigned long long seed);
  unsigned long long next_seed();

 private:
  std::mutex mu_;
  bool initialized_ = false;
  TensorFuseConfig cfg_{};
  std::vector<int> devices_;
  std::vector<std::unique_ptr<DeviceCtx>> ctxs_;
  std::map<const void*, size_t> static_weights_;   // registered host ranges: address -> bytes
  std::map<int, cudaMemPool_t> pools_;
  struct QkvKey {
    int dev; const void* q; const void* k; const void* v;
    bool operator<(const QkvKey& o) const {
      if (dev != o.dev) return dev < o.dev;
      if (q != o.q) return q < o.q;
      if (k != o.k) return k < o.k;
      return v < o.v;
    }
  };
  std::map<QkvKey, FusedQkv> fused_qkv_;
  void drop_fused_qkv_locked(const void* ptr);   // entries that involve ptr (null: all)
  bool seeded_ = false;
  unsigned long long seed_base_ = 0, seed_calls_ = 0;
};

// Sets the current device for the lifetime of the object when it differs.
class DeviceGuard {
 public:
  explicit DeviceGuard(int dev);
  ~DeviceGuard();
 private:
  int prev_ = -1;
  bool switched_ = false;
};

// Device that owns a device pointer, or -1 when it cannot be told (host memory,
// unregistered, error).
int device_of_pointer(const void* p);
// True when p is page-locked host memory known to the CUDA runtime.
bool is_pinned_host(const void* p);

// Contiguous, balanced split of `rows` rows into `parts` ranges whose starts are
// multiples of `align` (the last range absorbs the remainder; empty ranges are
// legal when rows < parts * align).
void plan_shards(long long rows, int parts, int align, long long* begins, long long* counts);

}  // namespace tfb
