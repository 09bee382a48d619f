/* tensorfuse/profiler.h -- timing and accounting helpers of the TensorFuse C
 * interface.  Same symbols and struct layouts as the reference header
 * src/tensorfuse/profiler.h (definitions: src/tensorfuse_c_api.cpp:462-643,
 * where every one of them is a constant-returning placeholder).  Here the
 * timers measure real time, the counters count the library's own launches and
 * the roofline helper uses B200 peaks; nothing in this header is on the hot path.
 */
#ifndef TENSORFUSE_B200_PROFILER_H_
#define TENSORFUSE_B200_PROFILER_H_

#include "types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Launch geometry as passed by value to tensorfuse_profiler_record_kernel
 * (binary layout of CUDA's dim3). */
#if defined(__CUDACC__) || defined(__CUDA_RUNTIME_H__) || defined(TENSORFUSE_WITH_CUDA_RUNTIME)
typedef dim3 TensorFuseDim3;
typedef cudaEvent_t TensorFuseCudaEvent;
#else
typedef struct { unsigned int x, y, z; } TensorFuseDim3;
typedef struct CUevent_st* TensorFuseCudaEvent;
#endif

/* reference profiler.h:28-102 */
TensorFuseStatus tensorfuse_profiler_init(const TensorFuseProfileConfig* config);
TensorFuseStatus tensorfuse_profiler_shutdown(void);
int tensorfuse_profiler_start_region(const char* name, const char* category);      /* returns a region id >= 1 */
TensorFuseStatus tensorfuse_profiler_end_region(int region_id);
TensorFuseStatus tensorfuse_profiler_record_kernel(const char* kernel_name, TensorFuseDim3 grid_dim,
                                                   TensorFuseDim3 block_dim, size_t shared_mem_bytes,
                                                   cudaStream_t stream);
TensorFuseStatus tensorfuse_profiler_record_memcpy(const char* src_type, const char* dst_type,
                                                   size_t size_bytes, cudaStream_t stream);
/* num_kernel_launches = kernels launched by this library since the last reset,
 * cpu_time_ms / total_time_ms = time spent inside closed regions. */
TensorFuseStatus tensorfuse_profiler_get_metrics(TensorFuseMetrics* metrics);
TensorFuseStatus tensorfuse_profiler_reset(void);
TensorFuseStatus tensorfuse_profiler_save(const char* filename, const char* format);   /* format "json" or "csv" */

/* reference profiler.h:113-137 (the variant compiled when profiling is enabled) */
typedef struct {
  unsigned long long range_id;
  bool active;
} TensorFuseNvtxRange;
TensorFuseNvtxRange tensorfuse_nvtx_range_start(const char* name, uint32_t color);
void tensorfuse_nvtx_range_end(TensorFuseNvtxRange* range);
void tensorfuse_nvtx_mark(const char* name, uint32_t color);

/* reference profiler.h:217-240: host wall-clock timer, milliseconds */
typedef struct {
  double start_time;
  double end_time;
  bool running;
} TensorFuseTimer;
void tensorfuse_timer_start(TensorFuseTimer* timer);
void tensorfuse_timer_stop(TensorFuseTimer* timer);
double tensorfuse_timer_elapsed_ms(const TensorFuseTimer* timer);

/* reference profiler.h:245-288: CUDA-event timer on a stream */
typedef struct {
  TensorFuseCudaEvent start_event;
  TensorFuseCudaEvent stop_event;
  bool events_created;
  bool timing_started;
} TensorFuseCudaTimer;
TensorFuseStatus tensorfuse_cuda_timer_create(TensorFuseCudaTimer* timer);
TensorFuseStatus tensorfuse_cuda_timer_destroy(TensorFuseCudaTimer* timer);
TensorFuseStatus tensorfuse_cuda_timer_start(TensorFuseCudaTimer* timer, cudaStream_t stream);
TensorFuseStatus tensorfuse_cuda_timer_stop(TensorFuseCudaTimer* timer, cudaStream_t stream);
/* synchronises on the stop event */
TensorFuseStatus tensorfuse_cuda_timer_elapsed_ms(TensorFuseCudaTimer* timer, float* elapsed_ms);

/* reference profiler.h:297-322.  Peaks are the B200's nominal dense FP16 tensor
 * rate (2.25e15 op/s) and HBM3e bandwidth (8e12 B/s); an operation is compute
 * bound when its arithmetic intensity exceeds their ratio. */
typedef struct {
  float peak_flops;
  float peak_bandwidth;
  float arithmetic_intensity;
  float achieved_flops;
  float achieved_bandwidth;
  float efficiency_flops;
  float efficiency_bandwidth;
  bool is_compute_bound;
  bool is_memory_bound;
} TensorFuseRooflineModel;
TensorFuseStatus tensorfuse_calculate_roofline(size_t ops_count, size_t bytes_transferred, float time_ms,
                                               TensorFuseRooflineModel* model);

#ifdef __cplusplus
}
#endif
#endif /* TENSORFUSE_B200_PROFILER_H_ */
