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
#include "ptx.cuh"

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


// ------------------------------------------------------ FP32 fast path
// The FP32 entry points are what the reference itself benchmarks
// (benchmarks/bert_baseline.cu), so they get a tuned CUDA-core kernel of their
// own: 128 x 128 x 8 tiles, 256 threads with 8 x 8 accumulators each, 16-byte
// global loads (A along K, B along N), the next K slice fetched into registers
// while the current one is multiplied out of double-buffered shared memory, and
// 16-byte shared-memory reads for both fragments.  Needs 16-byte aligned
// pointers, K % 4 == 0 and N % 4 == 0; everything else takes the generic kernel.
template <int EPI>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       const float* __restrict__ bias, float* __restrict__ C, int M,
                                                       int N, int K, EpiParams ep) {
  __shared__ __align__(16) float As[2][BK][BM];
  __shared__ __align__(16) float Bs[2][BK][BN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int a_row = tid >> 1, a_k = (tid & 1) * 4;   // A slice: 128 rows x 8 k, one float4 along k per thread
  const int b_k = tid >> 5, b_n = (tid & 31) * 4;    // B slice: 8 k x 128 n, one float4 along n per thread
  const bool a_ok = m0 + a_row < M, b_ok = n0 + b_n < N;
  const float* ap = A + (size_t)(m0 + a_row) * K + a_k;
  const float* bp = B + (size_t)b_k * N + n0 + b_n;
  const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);

  // accumulators as packed pairs (columns 2j, 2j+1): one fma.rn.f32x2 per pair halves the
  // instructions of the inner product; each lane of it is an ordinary FP32 FMA
  uint64_t acc2[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc2[i][j] = pack2(0.0f, 0.0f);

  auto fetch = [&](int k0, float4& a4, float4& b4) {
    a4 = (a_ok && k0 + a_k < K) ? __ldg(reinterpret_cast<const float4*>(ap + k0)) : zero4;
    b4 = (b_ok && k0 + b_k < K) ? __ldg(reinterpret_cast<const float4*>(bp + (size_t)k0 * N)) : zero4;
  };
  auto stash = [&](int buf, const float4& a4, const float4& b4) {
    As[buf][a_k + 0][a_row] = a4.x; As[buf][a_k + 1][a_row] = a4.y;
    As[buf][a_k + 2][a_row] = a4.z; As[buf][a_k + 3][a_row] = a4.w;
    *reinterpret_cast<float4*>(&Bs[buf][b_k][b_n]) = b4;
  };
  float4 a4, b4;
  fetch(0, a4, b4);
  stash(0, a4, b4);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += BK) {
    const bool more = k0 + BK < K;
    if (more) fetch(k0 + BK, a4, b4);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a_lo = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a_hi = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 b_lo = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b_hi = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      const uint64_t b2[4] = {pack2(b_lo.x, b_lo.y), pack2(b_lo.z, b_lo.w), pack2(b_hi.x, b_hi.y), pack2(b_hi.z, b_hi.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint64_t aa = pack2(a[i], a[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[i][j] = fma2(aa, b2[j], acc2[i][j]);
      }
    }
    if (more) {
      stash(buf ^ 1, a4, b4);       // the other buffer was last read one trip ago, before the barrier below
      __syncthreads();
      buf ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gn = n0 + h * 64 + tx * 4;
      if (gn >= N) continue;
      const float4 bv = __ldg(reinterpret_cast<const float4*>(bias + gn));
      const float2 p0 = unpack2(acc2[i][h * 2]), p1 = unpack2(acc2[i][h * 2 + 1]);
      float4 o;
      o.x = epilogue_value<EPI, true>(p0.x, bv.x, ep);
      o.y = epilogue_value<EPI, true>(p0.y, bv.y, ep);
      o.z = epilogue_value<EPI, true>(p1.x, bv.z, ep);
      o.w = epilogue_value<EPI, true>(p1.y, bv.w, ep);
      *reinterpret_cast<float4*>(C + (size_t)gm * N + gn) = o;
    }
  }
}

template <int EPI>
LaunchResult run_f32(const GemmArgs& a, cudaStream_t stream) {
  dim3 grid((a.N + BN - 1) / BN, (a.M + BM - 1) / BM);
  if (grid.y > 65535u) return kUnsupported;
  EpiParams ep{a.alpha, a.beta, a.scale, nullptr, nullptr};
  gemm_f32_kernel<EPI><<<grid, 256, 0, stream>>>(static_cast<const float*>(a.A), static_cast<const float*>(a.B),
                                                 static_cast<const float*>(a.bias), static_cast<float*>(a.C), a.M, a.N,
                                                 a.K, ep);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

bool f32_fast_path(const GemmArgs& a) {
  if (a.in_dtype != kF32 || a.out_dtype != kF32 || a.bias_dtype != kF32) return false;
  const uintptr_t ptrs = (uintptr_t)a.A | (uintptr_t)a.B | (uintptr_t)a.C | (uintptr_t)a.bias;
  return (ptrs & 15u) == 0 && a.K % 4 == 0 && a.N % 4 == 0;
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
  if (f32_fast_path(a) && a.epilogue == kEpiGelu) return run_f32<kEpiGelu>(a, stream);
  if (f32_fast_path(a) && a.epilogue == kEpiLinear) return run_f32<kEpiLinear>(a, stream);
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
