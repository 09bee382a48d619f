// gemm_tc.cu -- host side of the tensor-core GEMM + bias + GELU (the kernel is
// in gemm_tc_kernel.cuh): TMA tensor maps, launch geometry, dispatch.
//
// Replaces the reference's two-kernel FP16 path (CUTLASS mma.sync GEMM writing
// the pre-activation, then optimized_add_bias_gelu_kernel re-reading it:
// reference src/kernels/fused_gemm_bias_gelu_optimized.cu:115-259) and its
// three-kernel INT8 path (per-call transpose of B, GEMM, apply_scaled_gelu_kernel:
// reference src/kernels/fused_gemm_bias_gelu_int8.cu:156-344) with one launch.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include <cstdlib>
#include <cstring>

#include "gemm_tc_kernel.cuh"
#include "gemm_tc_pair_kernel.cuh"
#include "gemm_tf32x3_kernel.cuh"
#include "runtime.h"
#include "tma_host.h"

namespace tfb {
namespace {

using namespace tc;

// 2-D row-major matrix [rows, cols] of 1-, 2- or 4-byte elements; box = 128
// bytes of the contiguous dimension x box_rows rows, 128-byte swizzle, zero fill
// outside on loads, clipping on stores.
bool make_map(CUtensorMap* m, const void* base, int es, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * es};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = es == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                               : es == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                         : CU_TENSOR_MAP_DATA_TYPE_INT32;
  const CUresult r = fn(m, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct MapKey {
  const void* base; int es, rows, cols, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && es == o.es && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
// Small per-thread cache: encoding a tensor map costs a few microseconds and the
// same weight / activation buffers come back call after call.  The map is
// copied out, so a later insertion that recycles the slot cannot change it.
bool cached_map(const MapKey& k, CUtensorMap* out) {
  constexpr int kSlots = 24;
  thread_local MapKey keys[kSlots];
  thread_local CUtensorMap maps[kSlots];
  thread_local bool used[kSlots] = {};
  thread_local int next = 0;
  for (int i = 0; i < kSlots; ++i)
    if (used[i] && keys[i] == k) { *out = maps[i]; return true; }
  const int slot = next;
  next = (next + 1) % kSlots;
  used[slot] = false;
  if (!make_map(&maps[slot], k.base, k.es, k.rows, k.cols, k.box_rows)) return false;
  keys[slot] = k;
  used[slot] = true;
  *out = maps[slot];
  return true;
}

int sm_count(int dev) {
  static int cached[64] = {0};
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

template <int KIND, int EPI, typename TOut>
LaunchResult run(const GemmArgs& a, cudaStream_t stream) {
  constexpr int ES = KindTraits<KIND>::ES;
  auto kernel = gemm_tc_kernel<KIND, EPI, TOut>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kCudaError;
  // Once per instantiation and device: opt in to the large dynamic shared-memory carve-out.
  static bool ready[64] = {};
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!ready[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return kCudaError;
      }
      ready[dev] = true;
    }
  }
  CUtensorMap ma, mb, mc;
  if (!cached_map(MapKey{a.A, ES, a.M, a.K, TBM}, &ma) ||
      !cached_map(MapKey{a.B, ES, a.K, a.N, 128 / ES}, &mb) ||
      !cached_map(MapKey{a.C, (int)sizeof(TOut), a.M, a.N, 32}, &mc))
    return kLaunchFailed;
  const int tiles = ((a.M + TBM - 1) / TBM) * ((a.N + TBN - 1) / TBN);
  const int sms = sm_count(dev);
  const int grid = tiles < sms ? tiles : sms;
  EpiParams ep{a.alpha, a.beta, a.scale, a.scale_a_dev, a.scale_b_dev, a.scale_b_cols};
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, mc, a.bias, a.bias_dtype, a.M, a.N, a.K, ep,
                                                    watchdog_word());
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
  return kOk;
}

// The CTA-pair form of the same kernel (gemm_tc_pair_kernel.cuh).
template <int KIND, int EPI, typename TOut>
LaunchResult run_pair(const GemmArgs& a, cudaStream_t stream) {
  using namespace tc2;
  constexpr int ES = KindTraits<KIND>::ES;
  auto kernel = gemm_tc_pair_kernel<KIND, EPI, TOut>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kCudaError;
  static bool ready[64] = {};
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!ready[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return kCudaError;
      }
      ready[dev] = true;
    }
  }
  CUtensorMap ma, mb, mc;
  if (!cached_map(MapKey{a.A, ES, a.M, a.K, TBM}, &ma) ||
      !cached_map(MapKey{a.B, ES, a.K, a.N, 128 / ES}, &mb) ||
      !cached_map(MapKey{a.C, (int)sizeof(TOut), a.M, a.N, 32}, &mc))
    return kLaunchFailed;
  const int tiles = ((a.M + 2 * TBM - 1) / (2 * TBM)) * ((a.N + TBN - 1) / TBN);
  // one resident cluster per SM pair the device can actually co-schedule
  static int max_clusters[64] = {};
  if (max_clusters[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)(sm_count(dev) / 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count(dev) / 2; }
    max_clusters[dev] = n;
  }
  const int pairs_max = max_clusters[dev];
  const int pairs = tiles < pairs_max ? tiles : pairs_max;
  EpiParams ep{a.alpha, a.beta, a.scale, a.scale_a_dev, a.scale_b_dev, a.scale_b_cols};
  kernel<<<2 * pairs, NUM_THREADS, P_SMEM_BYTES, stream>>>(ma, mb, mc, a.bias, a.bias_dtype, a.M, a.N, a.K, ep,
                                                          watchdog_word());
  count_launch();
  if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
  return kOk;
}

// Kernel form: the CTA-pair kernel whenever the problem has more than one
// 128-row band (a pair tile is 256 rows), the single-CTA kernel otherwise.
// TENSORFUSE_B200_GEMM_FORM = single | pair overrides the choice (for measurements).
bool use_pair_form(const GemmArgs& a) {
  static const int mode = [] {
    const char* e = std::getenv("TENSORFUSE_B200_GEMM_FORM");
    if (e && std::strcmp(e, "pair") == 0) return 1;
    if (e && std::strcmp(e, "single") == 0) return 2;
    return 0;
  }();
  if (mode == 1) return true;
  if (mode == 2) return false;
  return a.M > tc::TBM;
}

// FP32 on the tensor cores: split A and B into TF32 hi/lo planes (stream-ordered
// scratch from the library's workspace pool), then the three-product kernel.
template <int EPI>
LaunchResult run_tf32x3(const GemmArgs& a, cudaStream_t stream) {
  using namespace tf32x3;
  auto kernel = gemm_tf32x3_kernel<EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kCudaError;
  static bool ready[64] = {};
  static int max_clusters[64] = {};
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!ready[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, X_SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return kCudaError;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (unsigned)(sm_count(dev) / 2));
      cfg.blockDim = dim3(NUM_THREADS);
      cfg.dynamicSmemBytes = X_SMEM_BYTES;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      cfg.attrs = &attr; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 0; }
      max_clusters[dev] = n;
      ready[dev] = true;
    }
  }
  if (max_clusters[dev] <= 0) return kLaunchFailed;      // cannot co-schedule CTA pairs here
  cudaMemPool_t pool = Runtime::get().workspace_pool(dev);
  if (pool == nullptr) return kLaunchFailed;
  const size_t a_elems = (size_t)a.M * a.K, b_elems = (size_t)a.K * a.N;
  auto round_up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t a_bytes = round_up(a_elems * 4), b_bytes = round_up(b_elems * 4);
  char* ws = nullptr;
  if (cudaMallocFromPoolAsync(reinterpret_cast<void**>(&ws), 2 * a_bytes + 2 * b_bytes, pool, stream) != cudaSuccess) {
    cudaGetLastError();
    return kLaunchFailed;
  }
  float* ah = reinterpret_cast<float*>(ws);
  float* al = reinterpret_cast<float*>(ws + a_bytes);
  float* bh = reinterpret_cast<float*>(ws + 2 * a_bytes);
  float* bl = reinterpret_cast<float*>(ws + 2 * a_bytes + b_bytes);
  const int sms = sm_count(dev);
  {
    const long long n4 = (long long)(a_elems / 4);
    const long long want_a = (n4 + 255) / 256;
    const int blocks_a = (int)(want_a < (long long)sms * 6 ? (want_a > 0 ? want_a : 1) : (long long)sms * 6);
    const long long tiles = (long long)((a.N + 31) / 32) * ((a.K + 31) / 32);
    const int blocks_b = (int)(tiles < (long long)sms * 6 ? (tiles > 0 ? tiles : 1) : (long long)sms * 6);
    split_operands_kernel<<<blocks_a + blocks_b, 256, 0, stream>>>(static_cast<const float4*>(a.A), reinterpret_cast<float4*>(ah),
                                                                   reinterpret_cast<float4*>(al), n4, blocks_a,
                                                                   static_cast<const float*>(a.B), bh, bl, a.K, a.N);
  }
  count_launch(1);
  LaunchResult res = kOk;
  CUtensorMap mah, mal, mbh, mbl, mc;
  if (!cached_map(MapKey{ah, 4, a.M, a.K, TBM}, &mah) || !cached_map(MapKey{al, 4, a.M, a.K, TBM}, &mal) ||
      !cached_map(MapKey{bh, 4, a.N, a.K, 128}, &mbh) || !cached_map(MapKey{bl, 4, a.N, a.K, 128}, &mbl) ||
      !cached_map(MapKey{a.C, 4, a.M, a.N, 32}, &mc)) {
    res = kLaunchFailed;
  } else {
    const int tiles = ((a.M + 2 * TBM - 1) / (2 * TBM)) * ((a.N + TBN - 1) / TBN);
    const int pairs = tiles < max_clusters[dev] ? tiles : max_clusters[dev];
    EpiParams ep{a.alpha, a.beta, a.scale, a.scale_a_dev, a.scale_b_dev, nullptr};
    // programmatic dependent launch: the GEMM's set-up overlaps the tail of the split kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)pairs);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = X_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    const void* bias_p = a.bias;
    int bias_dt = a.bias_dtype, M_ = a.M, N_ = a.N, K_ = a.K;
    int* wd = watchdog_word();
    if (cudaLaunchKernelEx(&cfg, kernel, mah, mal, mbh, mbl, mc, bias_p, bias_dt, M_, N_, K_, ep, wd) != cudaSuccess) {
      cudaGetLastError();
      res = kLaunchFailed;
    }
    count_launch();
  }
  cudaFreeAsync(ws, stream);
  return res;
}

// 0 = by size, 1 = CUDA cores only, 2 = tensor cores wherever eligible
// (TENSORFUSE_B200_FP32_FORM = simt | tf32x3, read once; for measurements and tests).
int fp32_form_override() {
  static const int mode = [] {
    const char* e = std::getenv("TENSORFUSE_B200_FP32_FORM");
    if (e && std::strcmp(e, "simt") == 0) return 1;
    if (e && std::strcmp(e, "tf32x3") == 0) return 2;
    return 0;
  }();
  return mode;
}

template <int KIND, int EPI, typename TOut>
LaunchResult run_any(const GemmArgs& a, cudaStream_t stream) {
  if (use_pair_form(a)) {
    const LaunchResult r = run_pair<KIND, EPI, TOut>(a, stream);
    if (r != kLaunchFailed) return r;
    cudaGetLastError();   // e.g. a partition that cannot co-schedule two CTAs: the single-CTA form still can run
  }
  return run<KIND, EPI, TOut>(a, stream);
}

}  // namespace

bool gemm_tc_eligible(const GemmArgs& a) {
  if (a.in_dtype != kF16 && a.in_dtype != kBF16 && a.in_dtype != kI8 && a.in_dtype != kFp8E4M3) return false;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return false;
  const int es = (a.in_dtype == kF16 || a.in_dtype == kBF16) ? 2 : 1;
  const int out_es = (a.out_dtype == kF16 || a.out_dtype == kBF16) ? 2 : 4;
  const uintptr_t ptrs = (uintptr_t)a.A | (uintptr_t)a.B | (uintptr_t)a.C;
  if (ptrs & 15u) return false;
  if (a.scale_b_cols != nullptr && (((uintptr_t)a.scale_b_cols & 15u) || a.epilogue != kEpiI8Dequant)) return false;
  if (((size_t)a.K * es) % 16 || ((size_t)a.N * es) % 16 || ((size_t)a.N * out_es) % 16) return false;
  if (a.in_dtype == kF16) return a.out_dtype == kF16 && (a.epilogue == kEpiGelu || a.epilogue == kEpiLinear);
  if (a.in_dtype == kBF16) return a.out_dtype == kBF16 && (a.epilogue == kEpiGelu || a.epilogue == kEpiLinear);
  if (a.in_dtype == kFp8E4M3) return a.epilogue == kEpiI8Dequant && (a.out_dtype == kF16 || a.out_dtype == kF32);
  return (a.epilogue == kEpiI8Dequant && (a.out_dtype == kF16 || a.out_dtype == kF32)) ||
         (a.epilogue == kEpiI8Legacy && a.out_dtype == kF32) ||
         (a.epilogue == kEpiI8Raw && a.out_dtype == kI32);
}

LaunchResult launch_gemm_tc(const GemmArgs& a, cudaStream_t stream) {
  if (!gemm_tc_eligible(a)) return kUnsupported;
  if (!a.bias && a.epilogue != kEpiI8Raw) return kInvalidArgument;
  if (a.in_dtype == kF16 && a.epilogue == kEpiLinear) return run_any<0, kEpiLinear, __half>(a, stream);
  if (a.in_dtype == kF16) return run_any<0, kEpiGelu, __half>(a, stream);
  if (a.in_dtype == kBF16 && a.epilogue == kEpiLinear) return run_any<2, kEpiLinear, __nv_bfloat16>(a, stream);
  if (a.in_dtype == kBF16) return run_any<2, kEpiGelu, __nv_bfloat16>(a, stream);
  if (a.in_dtype == kFp8E4M3 && a.out_dtype == kF16) return run_any<3, kEpiI8Dequant, __half>(a, stream);
  if (a.in_dtype == kFp8E4M3) return run_any<3, kEpiI8Dequant, float>(a, stream);
  if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF16) return run_any<1, kEpiI8Dequant, __half>(a, stream);
  if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF32) return run_any<1, kEpiI8Dequant, float>(a, stream);
  if (a.epilogue == kEpiI8Legacy) return run_any<1, kEpiI8Legacy, float>(a, stream);
  return run_any<1, kEpiI8Raw, int>(a, stream);
}

bool gemm_tf32x3_eligible(const GemmArgs& a) {
  if (a.in_dtype != kF32 || a.out_dtype != kF32) return false;
  if (a.epilogue != kEpiGelu && a.epilogue != kEpiLinear) return false;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || !a.bias) return false;
  if (((uintptr_t)a.A | (uintptr_t)a.B | (uintptr_t)a.C) & 15u) return false;
  if (a.K % 4 != 0 || a.N % 4 != 0) return false;                  // 16-byte row pitches for the tensor maps
  const int mode = fp32_form_override();
  if (mode == 1) return false;
  if (mode == 2) return true;
  // small problems stay on the CUDA-core kernel: the split pass and a cluster launch cost more than they save
  return (double)a.M * a.N * a.K >= 16777216.0;
}

LaunchResult launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  // the epilogues read the bias as FP32, FP16 or BF16 and nothing else
  if (a.epilogue != kEpiI8Raw && a.bias_dtype != kF32 && a.bias_dtype != kF16 && a.bias_dtype != kBF16)
    return kUnsupported;
  if (gemm_tf32x3_eligible(a)) {
    const LaunchResult r = a.epilogue == kEpiGelu ? run_tf32x3<kEpiGelu>(a, stream) : run_tf32x3<kEpiLinear>(a, stream);
    if (r != kLaunchFailed) return r;
    cudaGetLastError();     // no CTA pairs / no workspace: the CUDA-core kernel still runs
  }
  if (gemm_tc_eligible(a)) return launch_gemm_tc(a, stream);
  return launch_gemm_simt(a, stream);
}

}  // namespace tfb
