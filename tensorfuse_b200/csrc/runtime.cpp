// runtime.cpp -- see runtime.h.
#include "runtime.h"

#include <atomic>
#include <random>

#include "kernels.h"

namespace tfb {

// ------------------------------------------------------------- buffers
cudaError_t DevBuffer::reserve(size_t bytes) {
  if (bytes <= cap) return cudaSuccess;
  if (ptr) cudaFree(ptr);
  ptr = nullptr;
  cap = 0;
  // Round up so that slightly different problem sizes reuse the allocation.
  const size_t want = (bytes + (size_t(1) << 21) - 1) & ~((size_t(1) << 21) - 1);
  cudaError_t e = cudaMalloc(&ptr, want);
  if (e == cudaSuccess) cap = want;
  return e;
}
void DevBuffer::release() {
  if (ptr) cudaFree(ptr);
  ptr = nullptr;
  cap = 0;
}

cudaError_t DeviceCtx::ensure(size_t chunks) {
  cudaError_t e;
  if (!ready) {
    if ((e = cudaStreamCreateWithFlags(&s_in, cudaStreamNonBlocking)) != cudaSuccess) return e;
    if ((e = cudaStreamCreateWithFlags(&s_compute, cudaStreamNonBlocking)) != cudaSuccess) return e;
    if ((e = cudaStreamCreateWithFlags(&s_out, cudaStreamNonBlocking)) != cudaSuccess) return e;
    if ((e = cudaEventCreateWithFlags(&ev_weights, cudaEventDisableTiming)) != cudaSuccess) return e;
    ready = true;
  }
  while (ev_in.size() < chunks) {
    cudaEvent_t a, b;
    if ((e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming)) != cudaSuccess) return e;
    if ((e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming)) != cudaSuccess) return e;
    ev_in.push_back(a);
    ev_done.push_back(b);
  }
  return cudaSuccess;
}

void DeviceCtx::destroy() {
  if (!ready && !a.ptr && !b.ptr && !bias.ptr && !c.ptr && !mask.ptr && weights.empty()) return;
  DeviceGuard g(id);
  a.release(); b.release(); bias.release(); c.release(); mask.release();
  for (auto& kv : weights) kv.second.release();
  weights.clear();
  for (cudaEvent_t e : ev_in) cudaEventDestroy(e);
  for (cudaEvent_t e : ev_done) cudaEventDestroy(e);
  ev_in.clear(); ev_done.clear();
  if (ready) {
    cudaEventDestroy(ev_weights);
    cudaStreamDestroy(s_in); cudaStreamDestroy(s_compute); cudaStreamDestroy(s_out);
  }
  ready = false;
}

// ------------------------------------------------------------- runtime
Runtime& Runtime::get() {
  static Runtime r;
  return r;
}

TensorFuseStatus Runtime::init(const TensorFuseConfig* cfg) {
  std::lock_guard<std::mutex> g(mu_);
  if (initialized_) return TENSORFUSE_SUCCESS;
  if (cfg) {
    cfg_ = *cfg;
  } else {
    cfg_.device_count = 1;
    cfg_.device_ids = nullptr;
    cfg_.workspace_size_bytes = size_t(1) << 30;
    cfg_.enable_profiling = false;
    cfg_.enable_autotuning = true;
    cfg_.enable_fp8 = false;
    cfg_.log_level = 1;
    cfg_.cache_dir = "./cache";
  }
  int visible = 0;
  if (cudaGetDeviceCount(&visible) != cudaSuccess || visible < 1) {
    cudaGetLastError();
    return TENSORFUSE_ERROR_CUDA_ERROR;
  }
  std::vector<int> devs;
  const int n = cfg_.device_count > 0 ? cfg_.device_count : 1;
  if (n > 16) return TENSORFUSE_ERROR_INVALID_CONFIGURATION;
  for (int i = 0; i < n; ++i) {
    int d;
    if (cfg_.device_ids) d = cfg_.device_ids[i];
    else if (n == 1) { if (cudaGetDevice(&d) != cudaSuccess) d = 0; }
    else d = i;
    if (d < 0 || d >= visible) return TENSORFUSE_ERROR_INVALID_CONFIGURATION;
    for (int prev : devs)
      if (prev == d) return TENSORFUSE_ERROR_INVALID_CONFIGURATION;
    devs.push_back(d);
  }
  cfg_.device_ids = nullptr;  // the caller's array is not retained
  devices_ = devs;
  ctxs_.clear();
  for (size_t i = 0; i < devs.size(); ++i) {
    ctxs_.emplace_back(new DeviceCtx());
    ctxs_[i]->id = devs[i];
  }
  initialized_ = true;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus Runtime::shutdown() {
  std::lock_guard<std::mutex> g(mu_);
  if (!initialized_) return TENSORFUSE_SUCCESS;
  for (auto& c : ctxs_) {
    std::lock_guard<std::mutex> lk(c->mu);   // a host-buffer call still in flight finishes first
    c->destroy();
  }
  ctxs_.clear();
  static_weights_.clear();
  drop_fused_qkv_locked(nullptr);
  for (auto& kv : pools_) {
    DeviceGuard dg(kv.first);
    cudaDeviceSynchronize();           // stream-ordered frees into the pool have completed
    cudaMemPoolDestroy(kv.second);
  }
  pools_.clear();
  cudaGetLastError();
  devices_.clear();
  initialized_ = false;
  return TENSORFUSE_SUCCESS;
}

bool Runtime::initialized() {
  std::lock_guard<std::mutex> g(mu_);
  return initialized_;
}
int Runtime::log_level() {
  std::lock_guard<std::mutex> g(mu_);
  return cfg_.log_level;
}
std::vector<int> Runtime::devices() {
  std::lock_guard<std::mutex> g(mu_);
  return devices_;
}
DeviceCtx* Runtime::ctx(size_t i) {
  std::lock_guard<std::mutex> g(mu_);
  return i < ctxs_.size() ? ctxs_[i].get() : nullptr;
}

cudaMemPool_t Runtime::workspace_pool(int device) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = pools_.find(device);
  if (it != pools_.end()) return it->second;
  cudaMemPoolProps props{};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = device;
  cudaMemPool_t pool = nullptr;
  if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  unsigned long long threshold = ~0ull;
  cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &threshold);
  cudaGetLastError();
  pools_[device] = pool;
  return pool;
}

Runtime::FusedQkv* Runtime::fused_qkv_slot(int device, const void* wq, const void* wk, const void* wv, bool* fresh) {
  std::lock_guard<std::mutex> g(mu_);
  if (!static_weights_.count(wq) || !static_weights_.count(wk) || !static_weights_.count(wv)) return nullptr;
  const QkvKey key{device, wq, wk, wv};
  auto it = fused_qkv_.find(key);
  *fresh = it == fused_qkv_.end();
  return &fused_qkv_[key];
}

void Runtime::drop_fused_qkv_locked(const void* ptr) {
  for (auto it = fused_qkv_.begin(); it != fused_qkv_.end();) {
    if (ptr == nullptr || it->first.q == ptr || it->first.k == ptr || it->first.v == ptr) {
      DeviceGuard dg(it->first.dev);
      cudaDeviceSynchronize();          // a layer that reads the copy may still be running
      if (it->second.w) cudaFree(it->second.w);
      if (it->second.b) cudaFree(it->second.b);
      it = fused_qkv_.erase(it);
    } else {
      ++it;
    }
  }
  cudaGetLastError();
}

void Runtime::register_weights(const void* host_ptr, size_t bytes) {
  std::lock_guard<std::mutex> g(mu_);
  if (host_ptr && bytes) static_weights_[host_ptr] = bytes;
}
size_t Runtime::registered_bytes(const void* host_ptr) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = static_weights_.find(host_ptr);
  return it == static_weights_.end() ? 0 : it->second;
}
void Runtime::invalidate_weights(const void* host_ptr) {
  std::vector<DeviceCtx*> ctxs;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (host_ptr) static_weights_.erase(host_ptr);
    else static_weights_.clear();
    drop_fused_qkv_locked(host_ptr);
    for (auto& c : ctxs_) ctxs.push_back(c.get());
  }
  for (DeviceCtx* c : ctxs) {
    std::lock_guard<std::mutex> lk(c->mu);   // no call is using the copies while they are dropped
    DeviceGuard dg(c->id);
    if (host_ptr) {
      auto it = c->weights.find(host_ptr);
      if (it != c->weights.end()) { it->second.release(); c->weights.erase(it); }
    } else {
      for (auto& kv : c->weights) kv.second.release();
      c->weights.clear();
    }
  }
}

static inline unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

void Runtime::set_seed(unsigned long long seed) {
  std::lock_guard<std::mutex> g(mu_);
  seeded_ = true;
  seed_base_ = seed;
  seed_calls_ = 0;
}

unsigned long long Runtime::next_seed() {
  std::lock_guard<std::mutex> g(mu_);
  if (!seeded_) {
    std::random_device rd;
    seed_base_ = (static_cast<unsigned long long>(rd()) << 32) ^ rd();
    seeded_ = true;
    seed_calls_ = 0;
  }
  return splitmix64(seed_base_ + 0x632BE59BD9B4E019ull * (seed_calls_++));
}

// ------------------------------------------------------------- helpers
DeviceGuard::DeviceGuard(int dev) {
  if (dev < 0) return;
  if (cudaGetDevice(&prev_) != cudaSuccess) { prev_ = -1; return; }
  if (prev_ != dev) {
    if (cudaSetDevice(dev) == cudaSuccess) switched_ = true;
  }
}
DeviceGuard::~DeviceGuard() {
  if (switched_) cudaSetDevice(prev_);
}

int device_of_pointer(const void* p) {
  if (!p) return -1;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return -1; }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return at.device;
  return -1;
}

bool is_pinned_host(const void* p) {
  if (!p) return false;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return at.type == cudaMemoryTypeHost;
}

void plan_shards(long long rows, int parts, int align, long long* begins, long long* counts) {
  if (parts < 1) return;
  if (align < 1) align = 1;
  if (rows < 0) rows = 0;
  const long long units = (rows + align - 1) / align;  // aligned blocks, the last may be short
  long long at = 0;
  for (int i = 0; i < parts; ++i) {
    const long long u = units / parts + (i < units % parts ? 1 : 0);
    long long cnt = u * align;
    if (at + cnt > rows) cnt = rows - at;
    begins[i] = at;
    counts[i] = cnt;
    at += cnt;
  }
}

// ------------------------------------------------------------- watchdog / counters
static std::atomic<unsigned long long> g_launches{0};
unsigned long long launch_count() { return g_launches.load(); }
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n); }

static std::mutex g_wd_mu;
static int* g_wd_word = nullptr;
static bool g_wd_tried = false;

int* watchdog_word() {
  std::lock_guard<std::mutex> g(g_wd_mu);
  if (!g_wd_tried) {
    g_wd_tried = true;
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      g_wd_word = static_cast<int*>(p);
      *g_wd_word = 0;
    } else {
      cudaGetLastError();
    }
  }
  return g_wd_word;
}
int watchdog_status() {
  int* w = watchdog_word();
  return w ? *static_cast<volatile int*>(w) : 0;
}
void watchdog_reset() {
  int* w = watchdog_word();
  if (w) *static_cast<volatile int*>(w) = 0;
}

}  // namespace tfb
