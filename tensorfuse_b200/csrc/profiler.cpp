// profiler.cpp -- the timing / accounting helpers declared in
// tensorfuse/profiler.h.  The reference defines all of them as placeholders
// (reference src/tensorfuse_c_api.cpp:462-643: timer_stop sets end_time = 1.0,
// get_metrics zeroes the struct, roofline uses 1 TFLOP/s and 1 TB/s); these
// measure.  Host-side only: no kernel is launched from here.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "kernels.h"
#include "tensorfuse/profiler.h"

namespace {

double now_ms() {
  using clock = std::chrono::steady_clock;
  return std::chrono::duration<double, std::milli>(clock::now().time_since_epoch()).count();
}

struct Region {
  std::string name, category;
  double start_ms = 0.0, end_ms = -1.0;
};

struct ProfilerState {
  std::mutex mu;
  std::vector<Region> regions;
  unsigned long long launches_at_reset = 0;
  unsigned long long recorded_kernels = 0, recorded_memcpy_bytes = 0;
  unsigned long long next_range = 1;
} g;

}  // namespace

extern "C" {

TensorFuseStatus tensorfuse_profiler_init(const TensorFuseProfileConfig*) { return tensorfuse_profiler_reset(); }
TensorFuseStatus tensorfuse_profiler_shutdown(void) { return TENSORFUSE_SUCCESS; }

int tensorfuse_profiler_start_region(const char* name, const char* category) {
  std::lock_guard<std::mutex> l(g.mu);
  Region r;
  r.name = name ? name : "";
  r.category = category ? category : "";
  r.start_ms = now_ms();
  g.regions.push_back(r);
  return (int)g.regions.size();   // ids start at 1, as the reference's constant did
}

TensorFuseStatus tensorfuse_profiler_end_region(int region_id) {
  std::lock_guard<std::mutex> l(g.mu);
  if (region_id < 1 || (size_t)region_id > g.regions.size()) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  g.regions[region_id - 1].end_ms = now_ms();
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_profiler_record_kernel(const char*, TensorFuseDim3, TensorFuseDim3, size_t, cudaStream_t) {
  std::lock_guard<std::mutex> l(g.mu);
  ++g.recorded_kernels;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_profiler_record_memcpy(const char*, const char*, size_t size_bytes, cudaStream_t) {
  std::lock_guard<std::mutex> l(g.mu);
  g.recorded_memcpy_bytes += size_bytes;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_profiler_get_metrics(TensorFuseMetrics* m) {
  if (!m) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  memset(m, 0, sizeof(*m));
  std::lock_guard<std::mutex> l(g.mu);
  double closed = 0.0;
  for (const Region& r : g.regions)
    if (r.end_ms >= 0.0) closed += r.end_ms - r.start_ms;
  m->cpu_time_ms = (float)closed;
  m->total_time_ms = (float)closed;
  m->num_kernel_launches = (int)(tfb::launch_count() - g.launches_at_reset + g.recorded_kernels);
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) m->memory_used_bytes = total_b - free_b;
  else cudaGetLastError();
  m->memory_peak_bytes = m->memory_used_bytes;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_profiler_reset(void) {
  std::lock_guard<std::mutex> l(g.mu);
  g.regions.clear();
  g.launches_at_reset = tfb::launch_count();
  g.recorded_kernels = 0;
  g.recorded_memcpy_bytes = 0;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_profiler_save(const char* filename, const char* format) {
  if (!filename || !format) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  const bool csv = strcmp(format, "csv") == 0;
  FILE* f = fopen(filename, "w");
  if (!f) return TENSORFUSE_ERROR_FILE_IO;
  std::lock_guard<std::mutex> l(g.mu);
  if (csv) {
    fprintf(f, "name,category,ms\n");
    for (const Region& r : g.regions)
      fprintf(f, "%s,%s,%.6f\n", r.name.c_str(), r.category.c_str(), r.end_ms >= 0 ? r.end_ms - r.start_ms : -1.0);
  } else {
    fprintf(f, "{\"kernel_launches\": %llu, \"regions\": [", tfb::launch_count() - g.launches_at_reset);
    for (size_t i = 0; i < g.regions.size(); ++i) {
      const Region& r = g.regions[i];
      fprintf(f, "%s{\"name\": \"%s\", \"category\": \"%s\", \"ms\": %.6f}", i ? ", " : "", r.name.c_str(),
              r.category.c_str(), r.end_ms >= 0 ? r.end_ms - r.start_ms : -1.0);
    }
    fprintf(f, "]}\n");
  }
  fclose(f);
  return TENSORFUSE_SUCCESS;
}

TensorFuseNvtxRange tensorfuse_nvtx_range_start(const char*, uint32_t) {
  std::lock_guard<std::mutex> l(g.mu);
  TensorFuseNvtxRange r;
  r.range_id = g.next_range++;
  r.active = true;
  return r;
}
void tensorfuse_nvtx_range_end(TensorFuseNvtxRange* range) {
  if (range) range->active = false;
}
void tensorfuse_nvtx_mark(const char*, uint32_t) {}

void tensorfuse_timer_start(TensorFuseTimer* t) {
  if (!t) return;
  t->start_time = now_ms();
  t->end_time = t->start_time;
  t->running = true;
}
void tensorfuse_timer_stop(TensorFuseTimer* t) {
  if (!t) return;
  t->end_time = now_ms();
  t->running = false;
}
double tensorfuse_timer_elapsed_ms(const TensorFuseTimer* t) {
  return (t && !t->running) ? t->end_time - t->start_time : 0.0;
}

TensorFuseStatus tensorfuse_cuda_timer_create(TensorFuseCudaTimer* t) {
  if (!t) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  t->events_created = false;
  t->timing_started = false;
  if (cudaEventCreate(&t->start_event) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  if (cudaEventCreate(&t->stop_event) != cudaSuccess) {
    cudaGetLastError();
    cudaEventDestroy(t->start_event);
    return TENSORFUSE_ERROR_CUDA_ERROR;
  }
  t->events_created = true;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_cuda_timer_destroy(TensorFuseCudaTimer* t) {
  if (!t) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (t->events_created) { cudaEventDestroy(t->start_event); cudaEventDestroy(t->stop_event); }
  t->events_created = false;
  t->timing_started = false;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_cuda_timer_start(TensorFuseCudaTimer* t, cudaStream_t stream) {
  if (!t || !t->events_created) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (cudaEventRecord(t->start_event, stream) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  t->timing_started = true;
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_cuda_timer_stop(TensorFuseCudaTimer* t, cudaStream_t stream) {
  if (!t || !t->events_created || !t->timing_started) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (cudaEventRecord(t->stop_event, stream) != cudaSuccess) { cudaGetLastError(); return TENSORFUSE_ERROR_CUDA_ERROR; }
  return TENSORFUSE_SUCCESS;
}
TensorFuseStatus tensorfuse_cuda_timer_elapsed_ms(TensorFuseCudaTimer* t, float* elapsed_ms) {
  if (!t || !elapsed_ms || !t->events_created || !t->timing_started) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (cudaEventSynchronize(t->stop_event) != cudaSuccess ||
      cudaEventElapsedTime(elapsed_ms, t->start_event, t->stop_event) != cudaSuccess) {
    cudaGetLastError();
    return TENSORFUSE_ERROR_CUDA_ERROR;
  }
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_calculate_roofline(size_t ops_count, size_t bytes_transferred, float time_ms,
                                               TensorFuseRooflineModel* m) {
  if (!m || !(time_ms > 0.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  m->peak_flops = 2.25e15f;       // dense FP16/BF16 tensor rate of a B200
  m->peak_bandwidth = 8.0e12f;    // HBM3e
  m->arithmetic_intensity = bytes_transferred ? (float)((double)ops_count / (double)bytes_transferred) : 0.0f;
  m->achieved_flops = (float)((double)ops_count / (time_ms * 1e-3));
  m->achieved_bandwidth = (float)((double)bytes_transferred / (time_ms * 1e-3));
  m->efficiency_flops = m->achieved_flops / m->peak_flops * 100.0f;
  m->efficiency_bandwidth = m->achieved_bandwidth / m->peak_bandwidth * 100.0f;
  m->is_compute_bound = m->arithmetic_intensity > m->peak_flops / m->peak_bandwidth;
  m->is_memory_bound = !m->is_compute_bound;
  return TENSORFUSE_SUCCESS;
}

}  // extern "C"
