// gemm_tc.cu -- GEMM + bias + GELU on the sm_100a tensor cores, one kernel.
//
// Replaces the reference's two-kernel FP16 path (CUTLASS mma.sync GEMM writing
// the pre-activation, then optimized_add_bias_gelu_kernel re-reading it:
// reference src/kernels/fused_gemm_bias_gelu_optimized.cu:115-259) and its
// three-kernel INT8 path (per-call transpose of B, GEMM, apply_scaled_gelu_kernel:
// reference src/kernels/fused_gemm_bias_gelu_int8.cu:156-344).
//
// Shape of the kernel
//   * persistent: one CTA per SM walks output tiles of 128 x 256 in row-major
//     tile order (all N tiles of one M band are in flight together, so the A band
//     is read from HBM once and then served by L2; B is small and L2 resident).
//   * warp 0 (one elected lane)  : TMA producer.  Per K step (128 bytes of K) it
//     loads a 128-row A box and the 256-column B slab into a 4-deep ring of
//     128-byte-swizzled shared-memory stages and signals an mbarrier with the
//     byte count.
//   * warp 1 (one elected lane)  : issues tcgen05.mma (M=128, N=256, K=32 bytes)
//     straight from shared memory into a TMEM accumulator; tcgen05.commit frees
//     the stage and, at the end of a tile, publishes the accumulator.
//   * warps 2-5                  : epilogue.  tcgen05.ld pulls 32 columns of the
//     thread's accumulator row into registers, applies dequant scale, bias and
//     GELU there, converts and stores 16-byte vectors.  TMEM holds two 256-column
//     accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.
//   A is [M,K] row-major -> K-major operand.  B is [K,N] row-major -> the
//   "MN-major" operand form, consumed as stored: no transpose pass, no copy.
//
// Every mbarrier wait is bounded (ptx.cuh); a wait that expires raises a CTA
// abort flag, records a code in the watchdog word and all roles fall through to
// the tear-down that frees TMEM.
#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "epilogue.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tfb {
namespace {

constexpr int TBM = 128, TBN = 256, STAGES = 4;
constexpr int A_STAGE_BYTES = TBM * 128;  // 128 rows x 128 bytes of K
constexpr int B_STAGE_BYTES = TBN * 128;  // 256 columns x 128 bytes-worth of K rows
constexpr int STAGE_TX_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;

constexpr int OFF_A = 0;
constexpr int OFF_B = OFF_A + STAGES * A_STAGE_BYTES;
constexpr int OFF_BIAS = OFF_B + STAGES * B_STAGE_BYTES;  // 2 x 256 floats
constexpr int OFF_BAR = OFF_BIAS + 2 * TBN * 4;
// barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], bias_ready[2]
constexpr int NUM_BARS = 2 * STAGES + 6;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;  // tmem base address, abort flag
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;  // + slack for 1024-byte alignment

// watchdog codes (first wait that expired)
enum : int { kWdEmpty = 101, kWdFull = 102, kWdTmemEmpty = 103, kWdTmemFull = 104, kWdBias = 105 };

template <int KIND> struct KindTraits;
template <> struct KindTraits<0> {  // FP16 operands, FP32 accumulate
  static constexpr int ES = 2;
  static constexpr uint32_t IDESC = make_idesc(1u, 0u, TBM, TBN);
  using Acc = float;
};
template <> struct KindTraits<1> {  // INT8 operands, INT32 accumulate
  static constexpr int ES = 1;
  static constexpr uint32_t IDESC = make_idesc(2u, 1u, TBM, TBN);
  using Acc = int;
};

template <int KIND, int EPI, typename TOut>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const void* __restrict__ bias, int bias_dtype, TOut* __restrict__ C, int M, int N,
               int K, EpiParams ep_in, int* status) {
  using KT = KindTraits<KIND>;
  using Acc = typename KT::Acc;
  constexpr int ES = KT::ES;
  constexpr int BKE = 128 / ES;              // K elements per stage
  constexpr int MMA_PER_STAGE = 4;           // 32 bytes of K per MMA
  constexpr int B_BOX_COLS = 128 / ES;       // N elements per B box (128 bytes wide)
  constexpr int B_BOXES = TBN / B_BOX_COLS;
  constexpr int B_BOX_BYTES = 128 * BKE;     // BKE rows of 128 bytes
  constexpr int B_K_STEP_BYTES = (32 / ES) * 128;  // K rows per MMA x 128 bytes

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sA = smem_u32(smem + OFF_A);
  const uint32_t sB = smem_u32(smem + OFF_B);
  float* bias_s = reinterpret_cast<float*>(smem + OFF_BIAS);
  const uint32_t bars = smem_u32(smem + OFF_BAR);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  auto bias_bar = [&](int b) { return bars + 8u * (2 * STAGES + 4 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + TBN - 1) / TBN;
  const int tiles_m = (M + TBM - 1) / TBM;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), EPI_THREADS);
      mbar_init(bias_bar(b), EPI_THREADS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * TBM, n0 = (tile % tiles_n) * TBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, kWdEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(full_bar(stage), STAGE_TX_BYTES);
          tma_load_2d(sA + stage * A_STAGE_BYTES, &tmA, full_bar(stage), kb * BKE, m0);
#pragma unroll
          for (int j = 0; j < B_BOXES; ++j)
            tma_load_2d(sB + stage * B_STAGE_BYTES + j * B_BOX_BYTES, &tmB, full_bar(stage),
                        n0 + j * B_BOX_COLS, kb * BKE);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0, t_local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t_local) {
        const uint32_t buf = t_local & 1u, use = t_local >> 1;
        if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, status, kWdTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * TBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, status, kWdFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a0 = sA + stage * A_STAGE_BYTES, b0 = sB + stage * B_STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < MMA_PER_STAGE; ++j) {
            const uint64_t adesc = make_smem_desc(a0 + j * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc(b0 + j * B_K_STEP_BYTES, B_BOX_BYTES, 1024);
            const uint32_t accumulate = (kb | j) != 0 ? 1u : 0u;
            if (KIND == 0) tc_mma_f16(d, adesc, bdesc, KT::IDESC, accumulate);
            else tc_mma_i8(d, adesc, bdesc, KT::IDESC, accumulate);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int e = threadIdx.x - 64;      // 0..127
    const EpiParams ep = resolve_scales(ep_in);
    uint32_t t_local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t_local) {
      const uint32_t buf = t_local & 1u, use = t_local >> 1;
      const int m0 = (tile / tiles_n) * TBM, n0 = (tile % tiles_n) * TBN;
      float* bs = bias_s + buf * TBN;
      if (EPI != kEpiI8Raw) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int n = n0 + e + h * EPI_THREADS;
          float bv = 0.0f;
          if (n < N) bv = bias_dtype == kF16 ? __half2float(static_cast<const __half*>(bias)[n])
                                             : static_cast<const float*>(bias)[n];
          bs[e + h * EPI_THREADS] = bv;
        }
      }
      mbar_arrive(bias_bar(buf));
      if (!mbar_wait(bias_bar(buf), use & 1u, abort_flag, status, kWdBias)) break;
      if (!mbar_wait(tfull_bar(buf), use & 1u, abort_flag, status, kWdTmemFull)) break;
      tc_fence_after();

      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * TBN;
#pragma unroll 1
      for (int c = 0; c < TBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int ncol = n0 + c * 32;
        if (ncol >= N) continue;
        constexpr bool kFp32Out = sizeof(TOut) == 4;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(bs + c * 32 + i);
          const float bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            Acc a;
            if constexpr (KIND == 0) a = __uint_as_float(r[i + t]);
            else a = static_cast<int>(r[i + t]);
            v[i + t] = epilogue_value<EPI, kFp32Out>(a, bb[t], ep);
          }
        }
        if (row_ok) {
          TOut* crow = C + static_cast<size_t>(row) * N + ncol;
          if constexpr (sizeof(TOut) == 2) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if (ncol + g * 8 < N) {
                uint32_t w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                  const __half2 h = __floats2half2_rn(v[g * 8 + 2 * t], v[g * 8 + 2 * t + 1]);
                  w[t] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(crow + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            }
          } else {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (ncol + g * 4 < N) {
                *reinterpret_cast<uint4*>(crow + g * 4) =
                    make_uint4(__float_as_uint(v[g * 4]), __float_as_uint(v[g * 4 + 1]),
                               __float_as_uint(v[g * 4 + 2]), __float_as_uint(v[g * 4 + 3]));
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(buf));
    }
  }

  // ------------------------------------------------------------------ tear-down
  __syncwarp();
  if (*abort_flag) {
    // Give copies and MMAs that are still in flight time to land before the
    // shared memory and TMEM of this CTA are released.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major matrix [rows, cols] of 1- or 2-byte elements, box = 128 bytes of
// the contiguous dimension x box_rows rows, 128-byte swizzle, zero fill outside.
bool make_map(CUtensorMap* m, const void* base, int es, int rows, int cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * es};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(m, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                        const_cast<void*>(base), gdim, gstride, box, estr,
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
  constexpr int kSlots = 16;
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

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
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
  // Opt in to the large dynamic shared-memory carve-out once per device.
  static bool attr_set[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kCudaError;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!attr_set[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
        return kCudaError;
      attr_set[dev] = true;
    }
  }
  CUtensorMap ma, mb;
  if (!cached_map(MapKey{a.A, ES, a.M, a.K, TBM}, &ma) ||
      !cached_map(MapKey{a.B, ES, a.K, a.N, 128 / ES}, &mb))
    return kLaunchFailed;
  const int tiles = ((a.M + TBM - 1) / TBM) * ((a.N + TBN - 1) / TBN);
  const int sms = sm_count();
  const int grid = tiles < sms ? tiles : sms;
  EpiParams ep{a.alpha, a.beta, a.scale, a.scale_a_dev, a.scale_b_dev};
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, a.bias, a.bias_dtype,
                                                    static_cast<TOut*>(a.C), a.M, a.N, a.K, ep,
                                                    watchdog_word());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace

bool gemm_tc_eligible(const GemmArgs& a) {
  if (a.in_dtype != kF16 && a.in_dtype != kI8) return false;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return false;
  const int es = a.in_dtype == kF16 ? 2 : 1;
  const int out_es = a.out_dtype == kF16 ? 2 : 4;
  const uintptr_t ptrs = (uintptr_t)a.A | (uintptr_t)a.B | (uintptr_t)a.C;
  if (ptrs & 15u) return false;
  if (((size_t)a.K * es) % 16 || ((size_t)a.N * es) % 16 || ((size_t)a.N * out_es) % 16) return false;
  if (a.in_dtype == kF16) return a.out_dtype == kF16 && a.epilogue == kEpiGelu;
  return (a.epilogue == kEpiI8Dequant && (a.out_dtype == kF16 || a.out_dtype == kF32)) ||
         (a.epilogue == kEpiI8Legacy && a.out_dtype == kF32) ||
         (a.epilogue == kEpiI8Raw && a.out_dtype == kI32);
}

LaunchResult launch_gemm_tc(const GemmArgs& a, cudaStream_t stream) {
  if (!gemm_tc_eligible(a)) return kUnsupported;
  if (!a.bias && a.epilogue != kEpiI8Raw) return kInvalidArgument;
  if (a.in_dtype == kF16) return run<0, kEpiGelu, __half>(a, stream);
  if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF16) return run<1, kEpiI8Dequant, __half>(a, stream);
  if (a.epilogue == kEpiI8Dequant && a.out_dtype == kF32) return run<1, kEpiI8Dequant, float>(a, stream);
  if (a.epilogue == kEpiI8Legacy) return run<1, kEpiI8Legacy, float>(a, stream);
  return run<1, kEpiI8Raw, int>(a, stream);
}

LaunchResult launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (gemm_tc_eligible(a)) return launch_gemm_tc(a, stream);
  return launch_gemm_simt(a, stream);
}

}  // namespace tfb
