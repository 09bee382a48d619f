// host_ops.cpp -- operators on HOST buffers: the staging the reference performs
// in its Python binding (reference src/python/core_bindings.cpp:402-461 and
// 667-696: cudaMalloc per call, synchronous copies, one device, default stream,
// cudaFree) rebuilt as a cached, pipelined, multi-device path.
//
// Rows are split over the devices chosen at tensorfuse_init (weights and bias
// replicated, no exchange between devices).  On each device the shard is cut
// into chunks that flow through three streams:
//   s_in      host -> device copy of chunk i
//   s_compute kernel on chunk i           (waits for the copy)
//   s_out     device -> host copy of chunk i (waits for the kernel)
// so that the copies in both directions overlap each other and the kernels.
// Staging buffers are grow-only and live until tensorfuse_shutdown.
//
// Concurrency: a call holds the mutex of every device context it uses from its
// first reservation to its final synchronisation, so host-buffer calls from
// several threads are serialised per device (they share the staging buffers,
// streams and events).  On any failure the three streams are drained before
// the call returns, so the caller's buffers are never written afterwards.
//
// Weights: B and bias are uploaded on every call unless the caller has
// registered the host range as immutable (tensorfuse_b200_register_weights);
// then each device keeps one copy until tensorfuse_b200_invalidate_weights.
#include <algorithm>
#include <thread>
#include <utility>
#include <vector>

#include "kernels.h"
#include "runtime.h"
#include "tensorfuse_b200.h"

using namespace tfb;

namespace {

size_t dtype_size(int dt) {
  switch (dt) {
    case kF32: case kI32: return 4;
    case kF16: case kBF16: return 2;
    case kI8: case kU8: return 1;
    default: return 0;
  }
}

TensorFuseStatus from_cuda(cudaError_t e) {
  if (e == cudaSuccess) return TENSORFUSE_SUCCESS;
  cudaGetLastError();
  return e == cudaErrorMemoryAllocation ? TENSORFUSE_ERROR_OUT_OF_MEMORY : TENSORFUSE_ERROR_CUDA_ERROR;
}

TensorFuseStatus from_launch(LaunchResult r) {
  switch (r) {
    case kOk: return TENSORFUSE_SUCCESS;
    case kInvalidArgument: return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    case kCudaError: return TENSORFUSE_ERROR_CUDA_ERROR;
    case kLaunchFailed: return TENSORFUSE_ERROR_KERNEL_LAUNCH_FAILED;
    case kUnsupported: return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  }
  return TENSORFUSE_ERROR_UNKNOWN;
}

// Rows per chunk such that a chunk moves about `target` bytes, a multiple of
// `align` rows, at least one aligned block.
long long rows_per_chunk(size_t bytes_per_row, size_t target, int align) {
  long long r = (long long)(target / (bytes_per_row ? bytes_per_row : 1));
  r = (r / align) * align;
  return r < align ? align : r;
}

#define CK(expr)                                        \
  do {                                                  \
    cudaError_t e__ = (expr);                           \
    if (e__ != cudaSuccess) return from_cuda(e__);      \
  } while (0)

struct GemmHostJob {
  const char* A; const char* B; const char* bias; char* C;
  int N, K, in_dtype, bias_dtype, out_dtype, epilogue;
  float scale;
  bool b_static, bias_static;   // registered as immutable: one cached device copy per device
};

// Drains the three streams of a context: after a failure nothing may still be
// writing the caller's buffers when the (blocking) operator returns.
void drain(DeviceCtx* cx) {
  if (!cx->ready) return;
  cudaStreamSynchronize(cx->s_in);
  cudaStreamSynchronize(cx->s_compute);
  cudaStreamSynchronize(cx->s_out);
  cudaGetLastError();
}

// Device copy of a registered host range, uploaded on s_in the first time it is seen.
TensorFuseStatus cached_weight(DeviceCtx* cx, const void* host, size_t bytes, void** dev) {
  DevBuffer& buf = cx->weights[host];
  if (buf.ptr == nullptr || buf.cap < bytes) {
    CK(buf.reserve(bytes));
    CK(cudaMemcpyAsync(buf.ptr, host, bytes, cudaMemcpyHostToDevice, cx->s_in));
  }
  *dev = buf.ptr;
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus gemm_shard_locked(DeviceCtx* cx, const GemmHostJob& j, long long row0, long long rows);

TensorFuseStatus gemm_shard(DeviceCtx* cx, const GemmHostJob& j, long long row0, long long rows) {
  if (rows <= 0) return TENSORFUSE_SUCCESS;
  std::lock_guard<std::mutex> lk(cx->mu);
  DeviceGuard dg(cx->id);
  const TensorFuseStatus st = gemm_shard_locked(cx, j, row0, rows);
  if (st != TENSORFUSE_SUCCESS) drain(cx);
  return st;
}

TensorFuseStatus gemm_shard_locked(DeviceCtx* cx, const GemmHostJob& j, long long row0, long long rows) {
  const size_t es = dtype_size(j.in_dtype), bs = dtype_size(j.bias_dtype), os = dtype_size(j.out_dtype);
  const size_t a_row = (size_t)j.K * es, c_row = (size_t)j.N * os;
  // Chunks of about 16 MB of traffic, but the first ones are small (256 rows, doubling): the
  // device -> host copy, which dominates, starts as soon as a sliver of the output exists.
  const long long chunk = rows_per_chunk(a_row + c_row, size_t(16) << 20, 128);
  std::vector<std::pair<long long, long long>> chunks;
  for (long long r0 = 0, step = std::min<long long>(256, chunk); r0 < rows;) {
    const long long nr = std::min<long long>(step, rows - r0);
    chunks.emplace_back(r0, nr);
    r0 += nr;
    step = std::min<long long>(step * 2, chunk);
  }
  const size_t nchunks = chunks.size();
  CK(cx->ensure(nchunks));
  CK(cx->a.reserve((size_t)rows * a_row));
  CK(cx->c.reserve((size_t)rows * c_row));
  void* dB = nullptr;
  void* dBias = nullptr;
  if (j.b_static) {
    const TensorFuseStatus st = cached_weight(cx, j.B, (size_t)j.K * j.N * es, &dB);
    if (st != TENSORFUSE_SUCCESS) return st;
  } else {
    CK(cx->b.reserve((size_t)j.K * j.N * es));
    CK(cudaMemcpyAsync(cx->b.ptr, j.B, (size_t)j.K * j.N * es, cudaMemcpyHostToDevice, cx->s_in));
    dB = cx->b.ptr;
  }
  if (j.bias && j.bias_static) {
    const TensorFuseStatus st = cached_weight(cx, j.bias, (size_t)j.N * bs, &dBias);
    if (st != TENSORFUSE_SUCCESS) return st;
  } else {
    CK(cx->bias.reserve(std::max<size_t>((size_t)j.N * bs, 16)));
    if (j.bias) CK(cudaMemcpyAsync(cx->bias.ptr, j.bias, (size_t)j.N * bs, cudaMemcpyHostToDevice, cx->s_in));
    dBias = cx->bias.ptr;
  }
  CK(cudaEventRecord(cx->ev_weights, cx->s_in));
  CK(cudaStreamWaitEvent(cx->s_compute, cx->ev_weights, 0));

  for (size_t i = 0; i < nchunks; ++i) {
    const long long r0 = chunks[i].first;
    const long long nr = chunks[i].second;
    char* dA = static_cast<char*>(cx->a.ptr) + (size_t)r0 * a_row;
    char* dC = static_cast<char*>(cx->c.ptr) + (size_t)r0 * c_row;
    CK(cudaMemcpyAsync(dA, j.A + (size_t)(row0 + r0) * a_row, (size_t)nr * a_row,
                       cudaMemcpyHostToDevice, cx->s_in));
    CK(cudaEventRecord(cx->ev_in[i], cx->s_in));
    CK(cudaStreamWaitEvent(cx->s_compute, cx->ev_in[i], 0));
    GemmArgs g{};
    g.A = dA; g.B = dB; g.bias = dBias; g.C = dC;
    g.M = (int)nr; g.N = j.N; g.K = j.K;
    g.in_dtype = j.in_dtype; g.bias_dtype = j.bias_dtype; g.out_dtype = j.out_dtype;
    g.epilogue = j.epilogue;
    g.alpha = 1.0f; g.beta = 1.0f; g.scale = j.scale;
    const LaunchResult lr = launch_gemm(g, cx->s_compute);
    if (lr != kOk) return from_launch(lr);
    CK(cudaEventRecord(cx->ev_done[i], cx->s_compute));
    CK(cudaStreamWaitEvent(cx->s_out, cx->ev_done[i], 0));
    CK(cudaMemcpyAsync(j.C + (size_t)(row0 + r0) * c_row, dC, (size_t)nr * c_row,
                       cudaMemcpyDeviceToHost, cx->s_out));
  }
  CK(cudaStreamSynchronize(cx->s_out));
  return TENSORFUSE_SUCCESS;
}

struct SoftmaxHostJob {
  const char* in; char* out; unsigned char* mask;
  int L, dtype; float p; unsigned long long seed;
};

TensorFuseStatus softmax_shard_locked(DeviceCtx* cx, const SoftmaxHostJob& j, long long row0, long long rows);

TensorFuseStatus softmax_shard(DeviceCtx* cx, const SoftmaxHostJob& j, long long row0, long long rows) {
  if (rows <= 0) return TENSORFUSE_SUCCESS;
  std::lock_guard<std::mutex> lk(cx->mu);
  DeviceGuard dg(cx->id);
  const TensorFuseStatus st = softmax_shard_locked(cx, j, row0, rows);
  if (st != TENSORFUSE_SUCCESS) drain(cx);
  return st;
}

TensorFuseStatus softmax_shard_locked(DeviceCtx* cx, const SoftmaxHostJob& j, long long row0, long long rows) {
  const size_t es = dtype_size(j.dtype);
  const size_t row_b = (size_t)j.L * es;
  const long long chunk = rows_per_chunk(2 * row_b + (size_t)j.L, size_t(16) << 20, 16);
  const size_t nchunks = (size_t)((rows + chunk - 1) / chunk);
  CK(cx->ensure(nchunks));
  CK(cx->a.reserve((size_t)rows * row_b));
  CK(cx->c.reserve((size_t)rows * row_b));
  CK(cx->mask.reserve((size_t)rows * j.L));
  for (size_t i = 0; i < nchunks; ++i) {
    const long long r0 = (long long)i * chunk;
    const long long nr = std::min<long long>(chunk, rows - r0);
    char* dI = static_cast<char*>(cx->a.ptr) + (size_t)r0 * row_b;
    char* dO = static_cast<char*>(cx->c.ptr) + (size_t)r0 * row_b;
    unsigned char* dM = static_cast<unsigned char*>(cx->mask.ptr) + (size_t)r0 * j.L;
    CK(cudaMemcpyAsync(dI, j.in + (size_t)(row0 + r0) * row_b, (size_t)nr * row_b,
                       cudaMemcpyHostToDevice, cx->s_in));
    CK(cudaEventRecord(cx->ev_in[i], cx->s_in));
    CK(cudaStreamWaitEvent(cx->s_compute, cx->ev_in[i], 0));
    const LaunchResult lr = launch_softmax_dropout(dI, dO, dM, nr, j.L, j.dtype, j.p, j.seed,
                                                   (unsigned long long)(row0 + r0), cx->s_compute);
    if (lr != kOk) return from_launch(lr);
    CK(cudaEventRecord(cx->ev_done[i], cx->s_compute));
    CK(cudaStreamWaitEvent(cx->s_out, cx->ev_done[i], 0));
    CK(cudaMemcpyAsync(j.out + (size_t)(row0 + r0) * row_b, dO, (size_t)nr * row_b,
                       cudaMemcpyDeviceToHost, cx->s_out));
    CK(cudaMemcpyAsync(j.mask + (size_t)(row0 + r0) * j.L, dM, (size_t)nr * j.L,
                       cudaMemcpyDeviceToHost, cx->s_out));
  }
  CK(cudaStreamSynchronize(cx->s_out));
  return TENSORFUSE_SUCCESS;
}

// Runs fn(ctx, begin, count) for every selected device, one host thread per
// device when there is more than one; returns the first failure.
template <typename Fn>
TensorFuseStatus for_each_shard(long long rows, int align, Fn fn) {
  Runtime& rt = Runtime::get();
  const std::vector<int> devs = rt.devices();
  const int n = (int)devs.size();
  if (n < 1) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  std::vector<long long> begins(n), counts(n);
  plan_shards(rows, n, align, begins.data(), counts.data());
  if (n == 1) return fn(rt.ctx(0), begins[0], counts[0]);
  std::vector<TensorFuseStatus> st(n, TENSORFUSE_SUCCESS);
  std::vector<std::thread> th;
  for (int i = 0; i < n; ++i)
    th.emplace_back([&, i] {
      try {
        st[i] = fn(rt.ctx(i), begins[i], counts[i]);
      } catch (...) {
        st[i] = TENSORFUSE_ERROR_UNKNOWN;
      }
    });
  for (std::thread& t : th) t.join();
  for (TensorFuseStatus s : st)
    if (s != TENSORFUSE_SUCCESS) return s;
  return TENSORFUSE_SUCCESS;
}

}  // namespace

extern "C" {

TensorFuseStatus tensorfuse_b200_gemm_bias_gelu_host(const void* A, const void* B, const void* bias,
                                                     void* C, int M, int N, int K, int in_dtype,
                                                     int bias_dtype, int out_dtype, int epilogue,
                                                     float scale_A, float scale_B) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!A || !B || !C) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (M <= 0 || N <= 0 || K <= 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  GemmHostJob j{};
  j.A = static_cast<const char*>(A); j.B = static_cast<const char*>(B);
  j.bias = static_cast<const char*>(bias); j.C = static_cast<char*>(C);
  j.N = N; j.K = K; j.in_dtype = in_dtype; j.bias_dtype = bias_dtype; j.out_dtype = out_dtype;
  if (in_dtype == kI8) {
    if (epilogue != kEpiI8Dequant && epilogue != kEpiI8Legacy && epilogue != kEpiI8Raw)
      return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    j.epilogue = epilogue;
    j.scale = scale_A * scale_B;
    if (epilogue == kEpiI8Raw) j.bias_dtype = kF32;
  } else if (in_dtype == kF16 || in_dtype == kF32) {
    if (bias_dtype != in_dtype || out_dtype != in_dtype) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
    j.epilogue = kEpiGelu;
    j.scale = 1.0f;
  } else {
    return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  }
  if (!bias && j.epilogue != kEpiI8Raw) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  // looked up before any device context is locked (lock order: runtime, then context)
  j.b_static = Runtime::get().registered_bytes(B) >= (size_t)K * N * dtype_size(in_dtype);
  j.bias_static = bias && Runtime::get().registered_bytes(bias) >= (size_t)N * dtype_size(j.bias_dtype);
  return for_each_shard(M, 128, [&](DeviceCtx* cx, long long b, long long c) {
    return gemm_shard(cx, j, b, c);
  });
}

TensorFuseStatus tensorfuse_b200_softmax_dropout_host(const void* input, void* output,
                                                      unsigned char* dropout_mask, long long rows,
                                                      int row_len, int dtype, float dropout_prob,
                                                      unsigned long long seed) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!input || !output || !dropout_mask) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (!(dropout_prob >= 0.0f && dropout_prob <= 1.0f)) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (rows < 0 || row_len < 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (dtype != kF16 && dtype != kF32) return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (rows == 0 || row_len == 0) return TENSORFUSE_SUCCESS;
  SoftmaxHostJob j{static_cast<const char*>(input), static_cast<char*>(output), dropout_mask,
                   row_len, dtype, dropout_prob, seed};
  return for_each_shard(rows, 16, [&](DeviceCtx* cx, long long b, long long c) {
    return softmax_shard(cx, j, b, c);
  });
}

TensorFuseStatus tensorfuse_b200_register_weights(const void* host_ptr, size_t bytes) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!host_ptr || bytes == 0) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  Runtime::get().register_weights(host_ptr, bytes);
  return TENSORFUSE_SUCCESS;
}

TensorFuseStatus tensorfuse_b200_invalidate_weights(const void* host_ptr) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  Runtime::get().invalidate_weights(host_ptr);
  return TENSORFUSE_SUCCESS;
}

void* tensorfuse_b200_alloc_pinned(size_t bytes) {
  void* p = nullptr;
  if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
void tensorfuse_b200_free_pinned(void* p) {
  if (p) cudaFreeHost(p);
}

}  // extern "C"
