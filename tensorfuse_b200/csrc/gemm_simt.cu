// gemm_simt.cu -- CUDA-core GEMM + bias + GELU with the epilogue fused in.
//
// Serves the FP32 entry points (reference src/kernels/fused_gemm_bias_gelu.cu:306-326,
// which run a SIMT CUTLASS GEMM followed by a second element-wise kernel) and
// any FP16/INT8 problem whose pointers or row pitches are not 16-byte aligned
// and therefore cannot be described to TMA.  Any M, N, K >= 1.
//
// 128x128 output tile per CTA, K step 8, 256 threads, 8x8 accumulators per
// thread held in registers; bias, activation and the conversion to the output
// type are applied to those registers and stored once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "epilogue.cuh"
#include "kernels.h"

namespace tfb {
namespace {

constexpr int BM = 128, BN = 128, BK = 8;

template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<int8_t> { using type = int; };

template <typename TAcc> __device__ __forceinline__ TAcc widen(float v) { return (TAcc)v; }
template <typename TAcc> __device__ __forceinline__ TAcc widen(int8_t v) { return (TAcc)v; }
template <typename TAcc> __device__ __forceinline__ TAcc widen(__half v) { return (TAcc)__half2float(v); }
template <typename TAcc> __device__ __forceinline__ TAcc widen(__nv_bfloat16 v) { return (TAcc)__bfloat162float(v); }
template <typename TAcc> __device__ __forceinline__ TAcc widen(__nv_fp8_e4m3 v) { return (TAcc)float(v); }

__device__ __forceinline__ float load_bias(const void* bias, int bias_dtype, int n) {
  if (bias_dtype == kF16) return __half2float(static_cast<const __half*>(bias)[n]);
  if (bias_dtype == kBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
  return static_cast<const float*>(bias)[n];
}
__device__ __forceinline__ void store_out(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_out(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_out(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void store_out(int* p, float v) { *p = __float_as_int(v); }

template <typename TIn, typename TOut, int EPI>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TIn* __restrict__ A,
                                                         const TIn* __restrict__ B,
                                                         const void* __restrict__ bias,
                                                         int bias_dtype, TOut* __restrict__ C, int M,
                                                         int N, int K, EpiParams ep_in) {
  const EpiParams ep = resolve_scales(ep_in);
  using TAcc = typename AccOf<TIn>::type;
  __shared__ TAcc As[BK][BM + 4];
  __shared__ TAcc Bs[BK][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  TAcc acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0;

  const int a_row = tid >> 1, a_k = (tid & 1) * 4;  // A tile: 128 rows x 8 k
  const int b_k = tid >> 5, b_n = (tid & 31) * 4;    // B tile: 8 k x 128 n

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int gm = m0 + a_row, gk = k0 + a_k + i;
      As[a_k + i][a_row] = (gm < M && gk < K) ? widen<TAcc>(A[(size_t)gm * K + gk]) : (TAcc)0;
      const int gkb = k0 + b_k, gn = n0 + b_n + i;
      Bs[b_k][b_n + i] = (gkb < K && gn < N) ? widen<TAcc>(B[(size_t)gkb * N + gn]) : (TAcc)0;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      TAcc a[8], b[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = As[k][ty * 4 + i];
        a[4 + i] = As[k][64 + ty * 4 + i];
        b[i] = Bs[k][tx * 4 + i];
        b[4 + i] = Bs[k][64 + tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }

  constexpr bool kFp32Out = sizeof(TOut) == 4;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
    if (gn >= N) continue;
    const float bv = (EPI == kEpiI8Raw) ? 0.0f : load_bias(bias, bias_dtype, gn);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
      if (gm >= M) continue;
      EpiParams epn = ep;
      if (EPI == kEpiI8Dequant && ep.scale_cols != nullptr) epn.scale = ep.scale * ep.scale_cols[gn];
      const float v = epilogue_value<EPI, kFp32Out>(acc[i][j], bv, epn);
      if constexpr (EPI == kEpiI8Raw) C[(size_t)gm * N + gn] = (TOut)acc[i][j];
      else store_out(C + (size_t)gm * N + gn, v);
    }
  }
}

template <typename TIn, typename TOut, int EPI>
LaunchResult run(const GemmArgs& a, cudaStream_t stream) {
  dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
  if (grid.y > 65535u) return kUnsupported;
  EpiParams ep{a.alpha, a.beta, a.scale, a.scale_a_dev, a.scale_b_dev, a.scale_b_cols};
  gemm_simt_kernel<TIn, TOut, EPI><<<grid, 256, 0, stream>>>(
      static_cast<const TIn*>(a.A), static_cast<const TIn*>(a.B), a.bias, a.bias_dtype,
      static_cast<TOut*>(a.C), a.M, a.N, a.K, ep);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace

LaunchResult launch_gemm_simt(const GemmArgs& a, cudaStream_t stream) {
  if (!a.A || !a.B || !a.C || (!a.bias && a.epilogue != kEpiI8Raw)) return kInvalidArgument;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return kInvalidArgument;
  if (a.bias_dtype != kF32 && a.bias_dtype != kF16 && a.bias_dtype != kBF16) return kUnsupported;
  if (a.in_dtype == kF32 && a.out_dtype == kF32 && a.epilogue == kEpiGelu)
    return run<float, float, kEpiGelu>(a, stream);
  if (a.in_dtype == kF16 && a.out_dtype == kF16 && a.epilogue == kEpiGelu)
    return run<__half, __half, kEpiGelu>(a, stream);
  if (a.in_dtype == kF32 && a.out_dtype == kF32 && a.epilogue == kEpiLinear)
    return run<float, float, kEpiLinear>(a, stream);
  if (a.in_dtype == kF16 && a.out_dtype == kF16 && a.epilogue == kEpiLinear)
    return run<__half, __half, kEpiLinear>(a, stream);
  if (a.in_dtype == kBF16 && a.out_dtype == kBF16 && a.epilogue == kEpiGelu)
    return run<__nv_bfloat16, __nv_bfloat16, kEpiGelu>(a, stream);
  if (a.in_dtype == kBF16 && a.out_dtype == kBF16 && a.epilogue == kEpiLinear)
    return run<__nv_bfloat16, __nv_bfloat16, kEpiLinear>(a, stream);
  if (a.in_dtype == kFp8E4M3 && a.epilogue == kEpiI8Dequant) {
    if (a.out_dtype == kF16) return run<__nv_fp8_e4m3, __half, kEpiI8Dequant>(a, stream);
    if (a.out_dtype == kF32) return run<__nv_fp8_e4m3, float, kEpiI8Dequant>(a, stream);
  }
  if (a.in_dtype == kI8) {
    if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF16) return run<int8_t, __half, kEpiI8Dequant>(a, stream);
    if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF32) return run<int8_t, float, kEpiI8Dequant>(a, stream);
    if (a.epilogue == kEpiI8Legacy && a.out_dtype == kF32) return run<int8_t, float, kEpiI8Legacy>(a, stream);
    if (a.epilogue == kEpiI8Raw && a.out_dtype == kI32) return run<int8_t, int, kEpiI8Raw>(a, stream);
  }
  return kUnsupported;
}

}  // namespace tfb
