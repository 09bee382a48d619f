// quantize.cu -- per-tensor symmetric INT8 quantisation on the device, the
// producer side of the INT8 GEMM:
//     scale = max|x| / 127          (1 when the tensor is all zero)
//     q     = clip(rint(x / scale), -127, 127)      round-half-even, IEEE divide
// The scale stays in device memory, where the GEMM's scale pointers read it
// (TensorFuseTensor.scale), so quantise -> GEMM needs no host round trip.
//
// The reference has no quantiser: its Python binding scans the already
// quantised INT8 operands on the host for their maximum and guesses a scale
// from it on every call (reference src/python/core_bindings.cpp:467-491).
// Two HBM-bound passes: 4 (or 2) bytes read per element for the maximum, the
// same again plus 1 byte written for the conversion; the scale word holds
// max|x| between them.
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels.h"

namespace tfb {
namespace {

template <typename T> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&x)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      x[2 * k] = f.x; x[2 * k + 1] = f.y;
    }
  }
};
template <typename T> __device__ __forceinline__ float widen(T v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }

// max |x| as the bit pattern of a non-negative float (such patterns order like
// unsigned integers; NaN inputs are ignored by fmaxf).
template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T* __restrict__ x, long long n, bool vec, unsigned* out) {
  float m = 0.0f;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long n8 = vec ? n / 8 : 0;
  long long u = tid;
  for (; u + 3 * nthreads < n8; u += 4 * nthreads) {      // four independent 16/32-byte loads in flight
    float v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) Vec8<T>::load(x + (u + j * nthreads) * 8, v[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[j][i]));
  }
  for (; u < n8; u += nthreads) {
    float v[8];
    Vec8<T>::load(x + u * 8, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  }
  for (long long i = n8 * 8 + tid; i < n; i += nthreads) m = fmaxf(m, fabsf(widen<T>(x[i])));
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wm[w]);
    atomicMax(out, __float_as_uint(m));
  }
}

__device__ __forceinline__ int quant1(float x, float s) {
  const float r = rintf(__fdiv_rn(x, s));
  return (int)fminf(fmaxf(r, -127.0f), 127.0f);
}

// The word that held max|x| becomes the scale (one thread; the conversion pass
// that follows on the stream reads it).
__global__ void scale_from_absmax_kernel(float* word) {
  const float amax = *word;
  *word = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ x, long long n, bool vec,
                                                       const float* __restrict__ scale, int8_t* __restrict__ q) {
  const float s = *scale;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long n8 = vec ? n / 8 : 0;
  auto convert = [&](const float (&v)[8], long long unit) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= (uint32_t)(quant1(v[i], s) & 0xFF) << (8 * i);
      hi |= (uint32_t)(quant1(v[4 + i], s) & 0xFF) << (8 * i);
    }
    *reinterpret_cast<uint2*>(q + unit * 8) = make_uint2(lo, hi);
  };
  long long u = tid;
  for (; u + 3 * nthreads < n8; u += 4 * nthreads) {
    float v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) Vec8<T>::load(x + (u + j * nthreads) * 8, v[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) convert(v[j], u + j * nthreads);
  }
  for (; u < n8; u += nthreads) {
    float v[8];
    Vec8<T>::load(x + u * 8, v);
    convert(v, u);
  }
  for (long long i = n8 * 8 + tid; i < n; i += nthreads) q[i] = (int8_t)quant1(widen<T>(x[i]), s);
}

// Column-wise: one thread per column walks the K rows (neighbouring threads read
// neighbouring columns, so every row segment is one coalesced access); rows are
// split over blockIdx.y and merged with an atomic maximum on the bit patterns.
template <typename T>
__global__ void __launch_bounds__(256) absmax_columns_kernel(const T* __restrict__ w, int K, int N, unsigned* out) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n >= N) return;
  const int rows_per = (K + gridDim.y - 1) / gridDim.y;
  const int k0 = blockIdx.y * rows_per, k1 = min(K, k0 + rows_per);
  float m = 0.0f;
  for (int k = k0; k < k1; ++k) m = fmaxf(m, fabsf(widen<T>(w[(size_t)k * N + n])));
  atomicMax(out + n, __float_as_uint(m));
}
__global__ void __launch_bounds__(256) scales_from_absmax_kernel(float* words, int N) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n >= N) return;
  const float amax = words[n];
  words[n] = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
}
template <typename T>
__global__ void __launch_bounds__(256) quantize_columns_kernel(const T* __restrict__ w, int K, int N,
                                                               const float* __restrict__ scales,
                                                               int8_t* __restrict__ q) {
  const int n = blockIdx.x * 256 + threadIdx.x;
  if (n >= N) return;
  const float s = scales[n];
  const int rows_per = (K + gridDim.y - 1) / gridDim.y;
  const int k0 = blockIdx.y * rows_per, k1 = min(K, k0 + rows_per);
  for (int k = k0; k < k1; ++k) q[(size_t)k * N + n] = (int8_t)quant1(widen<T>(w[(size_t)k * N + n]), s);
}

template <typename T>
LaunchResult run_columns(const void* w, int K, int N, int8_t* q, float* scales, cudaStream_t stream) {
  const unsigned gx = (unsigned)((N + 255) / 256);
  unsigned gy = (unsigned)((8 * 148 + gx - 1) / gx);       // enough CTAs to fill the device
  if (gy > (unsigned)K) gy = (unsigned)K;
  if (gy < 1) gy = 1;
  if (gy > 65535u) gy = 65535u;
  if (cudaMemsetAsync(scales, 0, sizeof(float) * (size_t)N, stream) != cudaSuccess) return kCudaError;
  absmax_columns_kernel<T><<<dim3(gx, gy), 256, 0, stream>>>(static_cast<const T*>(w), K, N,
                                                            reinterpret_cast<unsigned*>(scales));
  scales_from_absmax_kernel<<<gx, 256, 0, stream>>>(scales, N);
  quantize_columns_kernel<T><<<dim3(gx, gy), 256, 0, stream>>>(static_cast<const T*>(w), K, N, scales, q);
  count_launch(3);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int sm_count_now() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

template <typename T>
LaunchResult run(const void* x, long long n, int8_t* q, float* scale_dev, cudaStream_t stream) {
  const bool vec = (((uintptr_t)x & 15u) == 0) && (((uintptr_t)q & 7u) == 0);
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = 16ll * sm_count_now();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (cudaMemsetAsync(scale_dev, 0, sizeof(float), stream) != cudaSuccess) return kCudaError;
  absmax_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const T*>(x), n, vec,
                                                         reinterpret_cast<unsigned*>(scale_dev));
  scale_from_absmax_kernel<<<1, 1, 0, stream>>>(scale_dev);
  quantize_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const T*>(x), n, vec, scale_dev, q);
  count_launch(3);
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace

LaunchResult launch_quantize_int8(const void* x, int dtype, long long n, signed char* q, float* scale_dev,
                                  cudaStream_t stream) {
  if (!x || !q || !scale_dev || n < 0) return kInvalidArgument;
  if (dtype != kF16 && dtype != kF32) return kUnsupported;
  if (n == 0) return kOk;
  if (dtype == kF16) return run<__half>(x, n, reinterpret_cast<int8_t*>(q), scale_dev, stream);
  return run<float>(x, n, reinterpret_cast<int8_t*>(q), scale_dev, stream);
}

LaunchResult launch_quantize_int8_columns(const void* w, int dtype, int K, int N, signed char* q, float* scales_dev,
                                          cudaStream_t stream) {
  if (!w || !q || !scales_dev || K < 0 || N < 0) return kInvalidArgument;
  if (dtype != kF16 && dtype != kF32) return kUnsupported;
  if (K == 0 || N == 0) return kOk;
  if (dtype == kF16) return run_columns<__half>(w, K, N, reinterpret_cast<int8_t*>(q), scales_dev, stream);
  return run_columns<float>(w, K, N, reinterpret_cast<int8_t*>(q), scales_dev, stream);
}

}  // namespace tfb
