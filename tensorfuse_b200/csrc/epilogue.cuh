// epilogue.cuh -- the element-wise tail of GEMM+bias+GELU, shared by the
// tensor-core and the CUDA-core kernels.  Everything here runs on accumulators
// that are still in registers; the pre-activation never goes to memory.
//
// GELU is the tanh form the reference uses
// (reference src/kernels/fused_gemm_bias_gelu_optimized.cu:42-51):
//   gelu(x) = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
// Two evaluations:
//   gelu_accurate : tanhf, used when the output is FP32 (reference tolerance 1e-4 abs)
//   gelu_fast     : the algebraically equal x * sigmoid(2u) with ex2.approx and an
//                   approximate reciprocal (relative error ~1e-6, far below one FP16
//                   ulp, and accurate in the negative tail where 1 + tanh cancels)
#pragma once
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

#include "kernels.h"

namespace tfb {

// scale_a / scale_b: optional device pointers to one float each (the `scale`
// field of an INT8 TensorFuseTensor).  Reading them on the device keeps the call
// asynchronous; the reference copies them to the host with a blocking memcpy
// (reference src/tensorfuse_c_api.cpp:200-208).
struct EpiParams {
  float alpha, beta, scale;
  const float* scale_a;
  const float* scale_b;
  const float* scale_cols = nullptr;   // optional: one dequantisation factor per output column (device, N floats)
};

__device__ __forceinline__ EpiParams resolve_scales(EpiParams ep) {
  if (ep.scale_a) ep.scale *= __ldg(ep.scale_a);
  if (ep.scale_b) ep.scale *= __ldg(ep.scale_b);
  return ep;
}

__device__ __forceinline__ float gelu_accurate(float x) {
  const float a = 0.7978845608028654f, b = 0.044715f;
  return x * 0.5f * (1.0f + tanhf(a * (x + b * x * x * x)));
}

__device__ __forceinline__ float gelu_fast(float x) {
  // 2u*log2(e) = x * (k1 + k2 x^2)
  const float k1 = 2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float k2 = k1 * 0.044715f;
  const float z = x * fmaf(k2, x * x, k1);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z));
  return __fdividef(x, 1.0f + e);
}

__device__ __forceinline__ float gelu_clamped(float v) {
  const float a = 0.7978845608028654f, b = 0.044715f;
  float arg = a * (v + b * v * v * v);
  arg = fmaxf(-10.0f, fminf(10.0f, arg));
  return v * 0.5f * (1.0f + tanhf(arg));
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

// acc: accumulator as produced by the MMA (float, or int32 for INT8 operands).
// Returns the value to store, still in FP32 (or the raw integer through a bit cast).
template <int EPI, bool FP32_OUT, typename AccT>
__device__ __forceinline__ float epilogue_value(AccT acc, float bias, const EpiParams& ep) {
  if constexpr (EPI == kEpiLinear) {
    return ep.alpha * (float)acc + ep.beta * bias;
  } else if constexpr (EPI == kEpiGelu) {
    const float x = ep.alpha * (float)acc + ep.beta * bias;
    return FP32_OUT ? gelu_accurate(x) : gelu_fast(x);
  } else if constexpr (EPI == kEpiI8Dequant) {
    const float x = fmaf((float)acc, ep.scale, bias);
    return FP32_OUT ? gelu_accurate(x) : gelu_fast(x);
  } else if constexpr (EPI == kEpiI8Legacy) {
    const float v = __fdiv_rn((float)acc, ep.scale) + bias;
    const float r = gelu_clamped(v) * ep.scale;
    return isfinite(r) ? r : 0.0f;
  } else {
    return __int_as_float((int)acc);
  }
}

}  // namespace tfb
