// gemm_tc_kernel.cuh -- device side of the tensor-core GEMM + bias + GELU.
//
// Shape of the kernel
//   * persistent: one CTA per SM walks output tiles of 128 x 256 in a
//     column-panel order (panels of 16 tile columns, column index fastest inside
//     a panel) so that the B panel and the A bands of the tiles in flight stay
//     L2-resident.
//   * warp 0 (one elected lane): TMA producer.  Per K step (128 bytes of K) it
//     loads a 128-row A box and the 256-column slab of B into a 4-deep ring of
//     128-byte-swizzled shared-memory stages; completion is counted in bytes on
//     an mbarrier.  Plain per-CTA loads.
//   * warp 1 (one elected lane): issues tcgen05.mma (M 128, N 256, 32 bytes of K
//     per instruction) from shared-memory descriptors into TMEM; tcgen05.commit
//     frees the stage and, after the last K step, publishes the accumulator.
//   * warps 2-9: epilogue.  Warp w may read TMEM lanes 32*(w%4)..; two warps share
//     a lane quarter and split the 256 columns.  tcgen05.ld pulls 32 columns of
//     the thread's accumulator row into registers (the next chunk is in flight
//     while the current one is processed); dequant scale, bias and GELU are
//     applied there with packed f32x2 arithmetic; the converted values go to a
//     per-warp 4 KB staging box in shared memory (128-byte swizzle, conflict
//     free) and leave through a TMA tensor store, which writes whole 128-byte
//     lines and clips the M and N tails.  TMEM holds two 256-column
//     accumulators, so the epilogue of tile i overlaps the main loop of tile i+1.
//   A is [M,K] row-major -> K-major operand.  B is [K,N] row-major -> the
//   "MN-major" operand form, consumed as stored: no transpose pass, no copy.
//
// This single-CTA form serves problems with one 128-row band; larger ones take
// the CTA-pair form (gemm_tc_pair_kernel.cuh), which moves a third less through
// each SM's shared memory: 1330 against 1215 TFLOPS on the 16384 x 4096 x 1024
// FP16 problem, 3090 against 2780 TOPS on the INT8 one.  Measured alternatives
// that are not kept: TMA prefetches of the next tile's operands into L2 cost
// 10-25 %; an evict-first hint on the output stores and narrower rasterisation
// panels changed nothing; register-to-global stores instead of the staged TMA
// stores were slower (1083 TFLOPS in the pair form).
//
// Every mbarrier wait is bounded (ptx.cuh); a wait that expires raises a CTA
// abort flag, records a code in the watchdog word and all roles fall through to
// the tear-down that frees TMEM.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tfb {
namespace tc {

constexpr int TBM = 128;   // accumulator rows per tile
constexpr int TBN = 256;   // accumulator columns per tile
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = TBM * 128;  // 128 rows x 128 bytes of K
constexpr int B_STAGE_BYTES = TBN * 128;  // 256 columns x 128 bytes-worth of K rows
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int NUM_THREADS = 64 + EPI_THREADS;
constexpr int TMEM_COLS = 512;
constexpr int PANEL_TILES_N = 16;    // tile columns per rasterisation panel
constexpr int STAGING_BYTES = 4096;  // per epilogue warp: 32 rows x 128 bytes

constexpr int OFF_A = 0;
constexpr int OFF_B = OFF_A + STAGES * A_STAGE_BYTES;
constexpr int OFF_STAGING = OFF_B + STAGES * B_STAGE_BYTES;
constexpr int OFF_BIAS = OFF_STAGING + EPI_WARPS * STAGING_BYTES;  // 2 x 256 floats
constexpr int OFF_BAR = OFF_BIAS + 2 * TBN * 4;
// barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], bias_ready[2]
constexpr int NUM_BARS = 2 * STAGES + 6;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;  // tmem base address, abort flag
constexpr int SMEM_BYTES = OFF_MISC + 16;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");

// watchdog codes (first wait that expired; 106 = shared memory window not 1024-byte aligned)
enum : int { kWdEmpty = 101, kWdFull = 102, kWdTmemEmpty = 103, kWdTmemFull = 104, kWdBias = 105, kWdAlign = 106 };

template <int KIND> struct KindTraits;
template <> struct KindTraits<0> {  // FP16 operands, FP32 accumulate
  static constexpr int ES = 2;
  static constexpr uint32_t C_FORMAT = 1u, AB_FORMAT = 0u;
  static constexpr bool kIntAcc = false;
};
template <> struct KindTraits<1> {  // INT8 operands, INT32 accumulate
  static constexpr int ES = 1;
  static constexpr uint32_t C_FORMAT = 2u, AB_FORMAT = 1u;
  static constexpr bool kIntAcc = true;
};
template <> struct KindTraits<2> {  // BF16 operands, FP32 accumulate (kind::f16, format 1)
  static constexpr int ES = 2;
  static constexpr uint32_t C_FORMAT = 1u, AB_FORMAT = 1u;
  static constexpr bool kIntAcc = false;
};
template <> struct KindTraits<3> {  // FP8 E4M3 operands, FP32 accumulate (kind::f8f6f4, format 0)
  static constexpr int ES = 1;
  static constexpr uint32_t C_FORMAT = 1u, AB_FORMAT = 0u;
  static constexpr bool kIntAcc = false;
};
template <typename T> struct IsBf16 { static constexpr bool value = false; };
template <> struct IsBf16<__nv_bfloat16> { static constexpr bool value = true; };

// Tile index -> (row tile, column tile): panels of PANEL_TILES_N tile columns,
// inside a panel the column index runs fastest.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_panel = tiles_m * PANEL_TILES_N;
  const int panel = t / per_panel;
  const int r = t - panel * per_panel;
  const int n_first = panel * PANEL_TILES_N;
  const int width = min(PANEL_TILES_N, tiles_n - n_first);
  tm = r / width;
  tn = n_first + (r - tm * width);
}

// ------------------------------------------------------------ TMA store side
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the staging box may be overwritten once every committed store has read it
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// 16-byte chunk j (0..7) of staging row r lives at chunk j ^ (r & 7): the
// 128-byte swizzle the tensor map of C uses, and conflict-free for a warp in
// which lane = row.
__device__ __forceinline__ void staging_store16(uint32_t base, int row, int j, uint4 v) {
  const uint32_t addr = base + row * 128 + ((j ^ (row & 7)) << 4);
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ------------------------------------------------------------ epilogue maths
// Two neighbouring accumulators at once.  Fast path (FP16 output): packed
// f32x2 arithmetic around the special-function operations (three per pair) of
// gelu(x) = x / (1 + 2^(-x (k1 + k2 x^2))).
template <int EPI, bool FP32_OUT, bool INT_ACC>
__device__ __forceinline__ float2 epilogue_pair(uint32_t r0, uint32_t r1, float b0, float b1, const EpiParams& ep) {
  if constexpr (!FP32_OUT && (EPI == kEpiGelu || EPI == kEpiI8Dequant || EPI == kEpiLinear)) {
    float a0, a1;
    if constexpr (INT_ACC) { a0 = (float)(int)r0; a1 = (float)(int)r1; }
    else { a0 = __uint_as_float(r0); a1 = __uint_as_float(r1); }
    uint64_t x2;
    if constexpr (EPI == kEpiGelu || EPI == kEpiLinear) x2 = fma2(pack2(a0, a1), pack2(ep.alpha, ep.alpha), pack2(ep.beta * b0, ep.beta * b1));
    else x2 = fma2(pack2(a0, a1), pack2(ep.scale, ep.scale), pack2(b0, b1));
    if constexpr (EPI == kEpiLinear) return unpack2(x2);
    const float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
    const float k2 = k1 * 0.044715f;
    const uint64_t w2 = fma2(mul2(x2, x2), pack2(k2, k2), pack2(k1, k1));
    float2 nz = unpack2(mul2(x2, w2));     // -2u*log2(e)
    // One reciprocal serves the pair: 1/a = b/(ab), 1/b = a/(ab).  The special-function
    // unit is what the epilogue is short of (three operations per pair instead of four);
    // the exponent is capped at 60 so that the product of the two denominators stays
    // finite (beyond it x * 2^-60 and the exact value both round to zero in 16 bits).
    nz.x = fminf(nz.x, 60.0f);
    nz.y = fminf(nz.y, 60.0f);
    float e0, e1;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(nz.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(nz.y));
    const float2 d = unpack2(add2(pack2(e0, e1), pack2(1.0f, 1.0f)));
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d.x * d.y));
    return unpack2(mul2(x2, mul2(pack2(r, r), pack2(d.y, d.x))));
  } else {
    float2 o;
    if constexpr (INT_ACC) {
      o.x = epilogue_value<EPI, FP32_OUT>((int)r0, b0, ep);
      o.y = epilogue_value<EPI, FP32_OUT>((int)r1, b1, ep);
    } else {
      o.x = epilogue_value<EPI, FP32_OUT>(__uint_as_float(r0), b0, ep);
      o.y = epilogue_value<EPI, FP32_OUT>(__uint_as_float(r1), b1, ep);
    }
    return o;
  }
}

// 32 accumulator columns of one row -> output bits: 16 words (FP16 output) or
// 32 words (4-byte output) in w[].
template <int EPI, typename TOut, bool INT_ACC>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], const float* bs, const EpiParams& ep,
                                               uint32_t (&w)[32]) {
  constexpr bool kFp32Out = sizeof(TOut) == 4;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 b4 = *reinterpret_cast<const float4*>(bs + i);
    const float2 v0 = epilogue_pair<EPI, kFp32Out, INT_ACC>(r[i], r[i + 1], b4.x, b4.y, ep);
    const float2 v1 = epilogue_pair<EPI, kFp32Out, INT_ACC>(r[i + 2], r[i + 3], b4.z, b4.w, ep);
    if constexpr (IsBf16<TOut>::value) {
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(v0.x, v0.y), h1 = __floats2bfloat162_rn(v1.x, v1.y);
      w[i / 2] = *reinterpret_cast<const uint32_t*>(&h0);
      w[i / 2 + 1] = *reinterpret_cast<const uint32_t*>(&h1);
    } else if constexpr (sizeof(TOut) == 2) {
      const __half2 h0 = __floats2half2_rn(v0.x, v0.y), h1 = __floats2half2_rn(v1.x, v1.y);
      w[i / 2] = *reinterpret_cast<const uint32_t*>(&h0);
      w[i / 2 + 1] = *reinterpret_cast<const uint32_t*>(&h1);
    } else {
      w[i] = __float_as_uint(v0.x); w[i + 1] = __float_as_uint(v0.y);
      w[i + 2] = __float_as_uint(v1.x); w[i + 3] = __float_as_uint(v1.y);
    }
  }
}

// Per-column dequantisation (weights quantised channel by channel): the factor of
// column n is ep.scale * scale_cols[n], read through the read-only cache (the
// same 32 values for every lane of the warp).  col0 is a multiple of 32 and N a
// multiple of 16 on this path, so a float4 of factors is entirely inside or
// outside the matrix.
template <typename TOut, bool INT_ACC>
__device__ __forceinline__ void epilogue_chunk_cols(const uint32_t (&r)[32], const float* bs, const EpiParams& ep,
                                                    int col0, int N, uint32_t (&w)[32]) {
  constexpr bool kFp32Out = sizeof(TOut) == 4;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float4 b4 = *reinterpret_cast<const float4*>(bs + i);
    float4 s4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (col0 + i < N) s4 = __ldg(reinterpret_cast<const float4*>(ep.scale_cols + col0 + i));
    const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float a = INT_ACC ? (float)(int)r[i + u] : __uint_as_float(r[i + u]);
      const float x = fmaf(a, ep.scale * ss[u], bb[u]);
      v[u] = kFp32Out ? gelu_accurate(x) : gelu_fast(x);
    }
    if constexpr (sizeof(TOut) == 2) {
      const __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
      w[i / 2] = *reinterpret_cast<const uint32_t*>(&h0);
      w[i / 2 + 1] = *reinterpret_cast<const uint32_t*>(&h1);
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) w[i + u] = __float_as_uint(v[u]);
    }
  }
}

// The epilogue of one 128 x 256 accumulator, shared by the single-CTA and the
// CTA-pair kernel: stage the bias slice, wait for the accumulator, then per 32
// columns TMEM -> registers -> scale/bias/activation -> staging box -> TMA
// store.  `release` hands the accumulator back to the MMA issuer (a local or a
// shared::cluster mbarrier arrive).  Returns false when a bounded wait expired.
template <int EPI, typename TOut, bool INT_ACC, typename ReleaseFn>
__device__ __forceinline__ bool epilogue_tile(const CUtensorMap* tmC, const void* bias, int bias_dtype, int M, int N,
                                              int m0, int n0, uint32_t buf, uint32_t use, float* bias_s,
                                              uint32_t staging, uint32_t bias_bar, uint32_t tfull_bar,
                                              uint32_t tmem_base, const EpiParams& ep, volatile int* abort_flag,
                                              int* status, ReleaseFn release) {
  constexpr int CHUNKS_PER_BOX = sizeof(TOut) == 2 ? 2 : 1;   // a staging row is 128 bytes
  constexpr int VEC_PER_CHUNK = sizeof(TOut) == 2 ? 4 : 8;    // 16-byte vectors per 32 columns
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3;                  // TMEM lane quarter this warp may read
  const int half = (warp - 2) >> 2;        // which 128 of the 256 columns
  const int e = threadIdx.x - 64;          // 0..255
  float* bs = bias_s + buf * TBN;
  if (EPI != kEpiI8Raw) {
    const int n = n0 + e;
    float bv = 0.0f;
    if (n < N) bv = bias_dtype == kF16    ? __half2float(static_cast<const __half*>(bias)[n])
                    : bias_dtype == kBF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n])
                                          : static_cast<const float*>(bias)[n];
    bs[e] = bv;
  }
  mbar_arrive(bias_bar);
  if (!mbar_wait(bias_bar, use & 1u, abort_flag, status, kWdBias)) return false;
  if (!mbar_wait(tfull_bar, use & 1u, abort_flag, status, kWdTmemFull)) return false;
  tc_fence_after();

  const int row0 = m0 + q * 32;            // first row of this warp's 32-row band
  const int nc = n0 + half * 128;          // first of this warp's 128 columns
  const float* bsh = bs + half * 128;
  const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * TBN + half * 128;
  uint32_t acc[2][32];
  tmem_ld_32x32(t_row, acc[0]);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    tmem_ld_wait();
    if (c < 3) tmem_ld_32x32(t_row + (c + 1) * 32, acc[(c + 1) & 1]);
    else {
      // every TMEM read of this accumulator is done: hand it back to the
      // MMA issuer before the last chunk's arithmetic
      tc_fence_before();
      release();
    }
    uint32_t w[32];
    if (EPI == kEpiI8Dequant && ep.scale_cols != nullptr)
      epilogue_chunk_cols<TOut, INT_ACC>(acc[c & 1], bsh + c * 32, ep, nc + c * 32, N, w);
    else
      epilogue_chunk<EPI, TOut, INT_ACC>(acc[c & 1], bsh + c * 32, ep, w);
    if (c % CHUNKS_PER_BOX == 0) {
      if (lane == 0) bulk_wait_read_all();   // the previous box has left the staging buffer
      __syncwarp();
    }
#pragma unroll
    for (int g = 0; g < VEC_PER_CHUNK; ++g)
      staging_store16(staging, lane, (c % CHUNKS_PER_BOX) * VEC_PER_CHUNK + g,
                      make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]));
    if (c % CHUNKS_PER_BOX == CHUNKS_PER_BOX - 1) {
      fence_async_smem();
      __syncwarp();
      const int x = nc + (c / CHUNKS_PER_BOX) * (128 / (int)sizeof(TOut));
      if (lane == 0 && x < N && row0 < M) {
        tma_store_2d(tmC, staging, x, row0);
        bulk_commit();
      }
    }
  }
  return true;
}

template <int KIND, int EPI, typename TOut>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const void* __restrict__ bias, int bias_dtype,
               int M, int N, int K, EpiParams ep_in, int* status) {
  using KT = KindTraits<KIND>;
  constexpr int ES = KT::ES;
  constexpr int BKE = 128 / ES;                    // K elements per stage
  constexpr int MMA_PER_STAGE = 4;                 // 32 bytes of K per MMA
  constexpr int B_BOX_COLS = 128 / ES;             // N elements per B box (128 bytes wide)
  constexpr int B_BOXES = TBN / B_BOX_COLS;
  constexpr int B_BOX_BYTES = 128 * BKE;           // BKE rows of 128 bytes
  constexpr int B_K_STEP_BYTES = (32 / ES) * 128;  // K rows per MMA x 128 bytes
  constexpr uint32_t IDESC = make_idesc(KT::C_FORMAT, KT::AB_FORMAT, TBM, TBN);

  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {   // the swizzled stages need 1024-byte alignment
    if (threadIdx.x == 0 && status != nullptr) *reinterpret_cast<volatile int*>(status) = kWdAlign;
    return;
  }
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
    tma_prefetch_desc(&tmC);
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
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * TBM, n0 = tn * TBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, kWdEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
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
            if (KIND == 0 || KIND == 2) tc_mma_f16(d, adesc, bdesc, IDESC, accumulate);
            else if (KIND == 1) tc_mma_i8(d, adesc, bdesc, IDESC, accumulate);
            else tc_mma_f8(d, adesc, bdesc, IDESC, accumulate);
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tc_commit(tfull_bar(buf));
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const uint32_t staging = smem_u32(smem + OFF_STAGING) + (warp - 2) * STAGING_BYTES;
    const EpiParams ep = resolve_scales(ep_in);
    uint32_t t_local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t_local) {
      const uint32_t buf = t_local & 1u, use = t_local >> 1;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const uint32_t tempty = tempty_bar(buf);
      if (!epilogue_tile<EPI, TOut, KT::kIntAcc>(&tmC, bias, bias_dtype, M, N, tm * TBM, tn * TBN, buf, use, bias_s,
                                                 staging, bias_bar(buf), tfull_bar(buf), tmem_base, ep, abort_flag,
                                                 status, [&] { mbar_arrive(tempty); }))
        break;
    }
    if (lane == 0) bulk_wait_all();
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

}  // namespace tc
}  // namespace tfb
