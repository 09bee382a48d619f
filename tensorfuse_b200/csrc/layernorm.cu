// layernorm.cu -- out = LayerNorm(x + residual) * gamma + beta over the last
// dimension, the glue between the fused operators inside a transformer layer
// (the reference's TensorFuseTransformerParams carries ln1/ln2 weights and an
// epsilon, src/tensorfuse/types.h:153-185, but no kernel uses them).
//
// HBM-bound: 2 reads + 1 write per element, everything else stays in
// registers.  One warp per row; the row (x + residual, FP32) is held in
// registers between the mean, the variance (second pass over the registers,
// not E[x^2] - mean^2) and the normalisation.  Rows up to 2048 elements with
// 16-byte aligned pitches take this path; anything else takes a block-per-row
// kernel that re-reads the row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels.h"

namespace tfb {
namespace {

template <typename T> struct Io8;
template <> struct Io8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&x)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      x[2 * k] = f.x; x[2 * k + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2 h = __floats2half2_rn(x[2 * k], x[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Io8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {          // a BF16 value is the upper half of the FP32 with the same value
      x[2 * k] = __uint_as_float(w[k] << 16);
      x[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * k], x[2 * k + 1]);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Io8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *(reinterpret_cast<const float4*>(p) + 1);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&x)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    *(reinterpret_cast<float4*>(p) + 1) = make_float4(x[4], x[5], x[6], x[7]);
  }
};
template <typename T> __device__ __forceinline__ float ld1(const T* p);
template <> __device__ __forceinline__ float ld1<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld1<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st1(T* p, float v);
template <> __device__ __forceinline__ void st1<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st1<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <> __device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// CH = 8-element units per lane: rows of up to 256 * CH elements.
template <typename T, int CH>
__global__ void __launch_bounds__(256) add_layernorm_warp_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                                 const T* __restrict__ gamma, const T* __restrict__ beta,
                                                                 T* __restrict__ out, long long rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * 8;
  const float inv_h = 1.0f / (float)H;
  for (long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += stride) {
    float v[CH][8];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = (lane + 32 * c) * 8;
      if (col < H) {
        Io8<T>::load(x + row * H + col, v[c]);
        if (res != nullptr) {
          float r[8];
          Io8<T>::load(res + row * H + col, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c][i] += r[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += v[c][i];
      }
    }
    const float mean = warp_sum(sum) * inv_h;
    float sq = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c)
      if ((lane + 32 * c) * 8 < H) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float d = v[c][i] - mean; sq = fmaf(d, d, sq); }
      }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) * inv_h + eps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int col = (lane + 32 * c) * 8;
      if (col < H) {
        float g[8], b[8], o[8];
        Io8<T>::load(gamma + col, g);
        Io8<T>::load(beta + col, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = fmaf((v[c][i] - mean) * rstd, g[i], b[i]);
        Io8<T>::store(out + row * H + col, o);
      }
    }
  }
}

// Any row length / alignment: one CTA per row, three passes over the row.
template <typename T>
__global__ void __launch_bounds__(256) add_layernorm_block_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                                  const T* __restrict__ gamma, const T* __restrict__ beta,
                                                                  T* __restrict__ out, long long rows, int H, float eps) {
  __shared__ float red[8];
  __shared__ float bcast;
  auto block_sum = [&](float v) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.0f;
      for (int w = 0; w < 8; ++w) t += red[w];
      bcast = t;
    }
    __syncthreads();
    const float r = bcast;
    __syncthreads();
    return r;
  };
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * H;
    const T* rr = res ? res + row * H : nullptr;
    float s = 0.0f;
    for (int c = threadIdx.x; c < H; c += 256) s += ld1<T>(xr + c) + (rr ? ld1<T>(rr + c) : 0.0f);
    const float mean = block_sum(s) / (float)H;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < H; c += 256) {
      const float d = ld1<T>(xr + c) + (rr ? ld1<T>(rr + c) : 0.0f) - mean;
      sq = fmaf(d, d, sq);
    }
    const float rstd = 1.0f / sqrtf(block_sum(sq) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += 256) {
      const float val = ld1<T>(xr + c) + (rr ? ld1<T>(rr + c) : 0.0f);
      st1<T>(out + row * H + c, fmaf((val - mean) * rstd, ld1<T>(gamma + c), ld1<T>(beta + c)));
    }
  }
}

template <typename T>
LaunchResult run(const void* x, const void* res, const void* gamma, const void* beta, void* out, long long rows, int H,
                 float eps, cudaStream_t stream) {
  const T* xp = static_cast<const T*>(x); const T* rp = static_cast<const T*>(res);
  const T* gp = static_cast<const T*>(gamma); const T* bp = static_cast<const T*>(beta);
  T* op = static_cast<T*>(out);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const uintptr_t bits = (uintptr_t)x | (uintptr_t)res | (uintptr_t)gamma | (uintptr_t)beta | (uintptr_t)out;
  const bool vec = (bits & 15u) == 0 && H % 8 == 0 && ((size_t)H * sizeof(T)) % 16 == 0 && H <= 2048;
  if (vec) {
    long long blocks = (rows + 7) / 8;
    if (blocks > 8ll * sms) blocks = 8ll * sms;
    const unsigned g = (unsigned)blocks;
    if (H <= 256) add_layernorm_warp_kernel<T, 1><<<g, 256, 0, stream>>>(xp, rp, gp, bp, op, rows, H, eps);
    else if (H <= 512) add_layernorm_warp_kernel<T, 2><<<g, 256, 0, stream>>>(xp, rp, gp, bp, op, rows, H, eps);
    else if (H <= 1024) add_layernorm_warp_kernel<T, 4><<<g, 256, 0, stream>>>(xp, rp, gp, bp, op, rows, H, eps);
    else add_layernorm_warp_kernel<T, 8><<<g, 256, 0, stream>>>(xp, rp, gp, bp, op, rows, H, eps);
  } else {
    const long long blocks = rows < 16ll * sms ? rows : 16ll * sms;
    add_layernorm_block_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(xp, rp, gp, bp, op, rows, H, eps);
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace

LaunchResult launch_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                                  long long rows, int hidden, int dtype, float eps, cudaStream_t stream) {
  if (!x || !gamma || !beta || !out || rows < 0 || hidden <= 0) return kInvalidArgument;
  if (dtype != kF16 && dtype != kBF16 && dtype != kF32) return kUnsupported;
  if (rows == 0) return kOk;
  if (dtype == kF16) return run<__half>(x, residual, gamma, beta, out, rows, hidden, eps, stream);
  if (dtype == kBF16) return run<__nv_bfloat16>(x, residual, gamma, beta, out, rows, hidden, eps, stream);
  return run<float>(x, residual, gamma, beta, out, rows, hidden, eps, stream);
}

}  // namespace tfb
