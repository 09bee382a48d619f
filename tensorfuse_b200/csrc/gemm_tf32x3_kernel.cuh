// gemm_tf32x3_kernel.cuh -- FP32 GEMM + bias + GELU on the tensor cores.
//
// An FP32 product is rebuilt from three TF32 tensor-core products: every operand
// x is split into hi = tf32(x) and lo = tf32(x - hi) (split_operands_kernel, one
// launch, one pass over A and B into scratch planes) and
//     A*B  ~=  A_hi*B_hi + A_lo*B_hi + A_hi*B_lo          (FP32 accumulation in TMEM)
// which leaves a relative error of about 2^-21 per product (the lo*lo term and
// the rounding of lo), an order of magnitude inside the 1e-4 absolute bound the
// reference's FP32 tests use (reference src/tests/test_kernels.cu:139,
// test_gemm_edge_cases.cu:155,249).  Replaces the reference's CUDA-core FP32 GEMM
// + separate bias/GELU kernel (reference
// src/kernels/fused_gemm_bias_gelu_optimized.cu:58-112,192-250).
//
// The tensor cores add into their FP32 accumulator with truncation, so a long
// chain of accumulations drifts by about half an ulp of the running sum per
// update (measured: 2.9e-4 absolute at K = 2048 with one accumulator per tile).
// The K loop is therefore cut into chunks of CHUNK_K elements: every chunk is
// accumulated from zero in one of the two TMEM buffers, and the epilogue warps
// add the finished chunk into FP32 partial sums that they keep in registers
// (round-to-nearest adds on the CUDA cores) while the tensor cores work on the
// next chunk in the other buffer.
//
// The kernel is the CTA-pair form of gemm_tc_pair_kernel.cuh with two planes
// per operand in every stage and three tcgen05.mma.cta_group::2.kind::tf32 per
// 32-byte slice of K; roles, barriers, bounded waits, the two TMEM accumulators
// and the epilogue (epilogue_tile with FP32 output) are the same.  Both operands
// are K-major here: the split pass writes the planes of B transposed ([N, K]),
// which costs nothing extra (B is rewritten anyway) and keeps the 32-bit
// operands on the plain 128-byte swizzle.
#pragma once
#include "gemm_tc_pair_kernel.cuh"

namespace tfb {
namespace tf32x3 {

using namespace tc;

constexpr int X_STAGES = 3;
constexpr int CHUNK_STAGES = 2;                   // K chunk accumulated inside the tensor cores: 2 stages = 64 elements
constexpr int X_PLANE_A = TBM * 128;              // 128 rows x 128 bytes (32 K elements)
constexpr int X_PLANE_B = 128 * 128;              // this CTA's 128 columns of B^T: 128 rows x 128 bytes of K
constexpr int X_STAGE_BYTES = 2 * X_PLANE_A + 2 * X_PLANE_B;   // hi and lo of both operands
constexpr int X_OFF_STAGES = 0;
constexpr int X_OFF_STAGING = X_OFF_STAGES + X_STAGES * X_STAGE_BYTES;
constexpr int X_OFF_BIAS = X_OFF_STAGING + EPI_WARPS * STAGING_BYTES;
constexpr int X_OFF_BAR = X_OFF_BIAS + 2 * TBN * 4;
constexpr int X_NUM_BARS = 2 * X_STAGES + 6;
constexpr int X_OFF_MISC = X_OFF_BAR + X_NUM_BARS * 8;
constexpr int X_SMEM_BYTES = X_OFF_MISC + 16;
static_assert(X_SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");

__device__ __forceinline__ void tc_mma_tf32_pair(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// x -> (tf32(x), tf32(x - tf32(x))), both stored as FP32 words whose low 13
// mantissa bits are zero.  Inf/NaN stay in the hi plane only (x - hi would be NaN).
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t hb, lb;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(x));
  hi = __uint_as_float(hb);
  const float d = isfinite(x) ? __fsub_rn(x, hi) : 0.0f;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(d));
  lo = __uint_as_float(lb);
}

// One launch splits both operands.  Blocks [0, blocks_a): A as it is stored, in
// float4 groups (n4 of them) into the planes a_hi / a_lo.  The other blocks:
// B[K, N] row-major into the two planes of B^T, each [N, K] row-major (K
// contiguous), 32 x 32 tiles through shared memory.  256 threads per block.
__global__ void __launch_bounds__(256) split_operands_kernel(const float4* __restrict__ a, float4* __restrict__ a_hi,
                                                             float4* __restrict__ a_lo, long long n4, int blocks_a,
                                                             const float* __restrict__ b, float* __restrict__ b_hi_t,
                                                             float* __restrict__ b_lo_t, int K, int N) {
  // the GEMM that consumes the planes may be scheduled as soon as SMs free up; it
  // waits (griddepcontrol.wait) for this whole grid before its first load
  asm volatile("griddepcontrol.launch_dependents;");
  if ((int)blockIdx.x < blocks_a) {
    const long long stride = (long long)blocks_a * 256;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n4; i += stride) {
      const float4 v = __ldg(a + i);
      float4 h, l;
      split_tf32(v.x, h.x, l.x); split_tf32(v.y, h.y, l.y); split_tf32(v.z, h.z, l.z); split_tf32(v.w, h.w, l.w);
      a_hi[i] = h;
      a_lo[i] = l;
    }
    return;
  }
  __shared__ float th[32][33], tl[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
  const int tiles_n = (N + 31) / 32, tiles_k = (K + 31) / 32;
  const int blocks_b = (int)gridDim.x - blocks_a;
  for (int t = (int)blockIdx.x - blocks_a; t < tiles_n * tiles_k; t += blocks_b) {
    const int k0 = (t / tiles_n) * 32, n0 = (t % tiles_n) * 32;
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
      const int k = k0 + r, n = n0 + tx;
      float x = 0.0f;
      if (k < K && n < N) x = __ldg(b + (size_t)k * N + n);
      split_tf32(x, th[r][tx], tl[r][tx]);
    }
    __syncthreads();
#pragma unroll
    for (int r = ty; r < 32; r += 8) {
      const int n = n0 + r, k = k0 + tx;
      if (n < N && k < K) {
        b_hi_t[(size_t)n * K + k] = th[tx][r];
        b_lo_t[(size_t)n * K + k] = tl[tx][r];
      }
    }
    __syncthreads();
  }
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                   const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                   const __grid_constant__ CUtensorMap tmC, const void* __restrict__ bias, int bias_dtype,
                   int M, int N, int K, EpiParams ep_in, int* status) {
  constexpr int BKE = 32;                          // K elements per stage (128 bytes)
  constexpr int MMA_PER_STAGE = 4;                 // 8 K elements (32 bytes) per MMA
  // c = F32 (1), a = b = TF32 (2), both operands K-major, M 256 over the pair, N 256
  constexpr uint32_t IDESC = make_idesc_major(1u, 2u, 0u, 0u, 2 * TBM, TBN);

  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const bool aligned = (smem_u32(smem) & 1023u) == 0u;
  const uint32_t s0 = smem_u32(smem + X_OFF_STAGES);
  float* bias_s = reinterpret_cast<float*>(smem + X_OFF_BIAS);
  const uint32_t bars = smem_u32(smem + X_OFF_BAR);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (X_STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * X_STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * X_STAGES + 2 + b); };
  auto bias_bar = [&](int b) { return bars + 8u * (2 * X_STAGES + 4 + b); };
  // planes of stage s: A_hi, A_lo, B_hi, B_lo
  auto plane = [&](int s, int which) {
    return s0 + s * X_STAGE_BYTES + (which < 2 ? which * X_PLANE_A : 2 * X_PLANE_A + (which - 2) * X_PLANE_B);
  };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + X_OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + X_OFF_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + TBN - 1) / TBN;
  const int tiles_m2 = (M + 2 * TBM - 1) / (2 * TBM);
  const int num_tiles = tiles_m2 * tiles_n;
  const int kblocks = (K + BKE - 1) / BKE;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < X_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * EPI_THREADS);
      mbar_init(bias_bar(b), EPI_THREADS);
    }
    *abort_flag = aligned ? 0 : 1;
    if (!aligned && status != nullptr) *reinterpret_cast<volatile int*>(status) = kWdAlign;
    mbar_fence_init();
    tma_prefetch_desc(&tmAh); tma_prefetch_desc(&tmAl);
    tma_prefetch_desc(&tmBh); tma_prefetch_desc(&tmBl);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = !*abort_flag;
      // Launched as a programmatic dependent of the split kernel: everything above
      // (barriers, TMEM, descriptor fetches) overlapped that kernel's tail; the
      // planes it writes are read from here on.  Without the launch attribute this
      // returns at once.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m2, tiles_n, tm, tn);
        const int m0 = tm * 2 * TBM + (int)rank * TBM, n0 = tn * TBN + (int)rank * 128;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, kWdEmpty)) { ok = false; break; }
          const uint32_t full_leader = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * X_STAGE_BYTES);
          tma_load_2d_pair(plane(stage, 0), &tmAh, full_leader, kb * BKE, m0);
          tma_load_2d_pair(plane(stage, 1), &tmAl, full_leader, kb * BKE, m0);
          tma_load_2d_pair(plane(stage, 2), &tmBh, full_leader, kb * BKE, n0);    // rows of B^T = columns of B
          tma_load_2d_pair(plane(stage, 3), &tmBl, full_leader, kb * BKE, n0);
          if (++stage == X_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------- MMA issuer (leader CTA)
    if (leader && elect_one()) {
      uint32_t stage = 0, phase = 0, c_local = 0;      // c_local counts chunks: buffer = c_local & 1
      bool ok = !*abort_flag;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        for (int kb0 = 0; kb0 < kblocks && ok; kb0 += CHUNK_STAGES, ++c_local) {
          const uint32_t buf = c_local & 1u, use = c_local >> 1;
          if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, status, kWdTmemEmpty)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + buf * TBN;
          const int kb1 = min(kblocks, kb0 + CHUNK_STAGES);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag, status, kWdFull)) { ok = false; break; }
            tc_fence_after();
            const uint32_t ah = plane(stage, 0), al = plane(stage, 1), bh = plane(stage, 2), bl = plane(stage, 3);
#pragma unroll
            for (int j = 0; j < MMA_PER_STAGE; ++j) {
              const uint64_t ahd = make_smem_desc(ah + j * 32, 16, 1024), ald = make_smem_desc(al + j * 32, 16, 1024);
              const uint64_t bhd = make_smem_desc(bh + j * 32, 16, 1024), bld = make_smem_desc(bl + j * 32, 16, 1024);
              // the two small cross terms first, the large term last; a chunk starts from zero
              tc_mma_tf32_pair(d, ald, bhd, IDESC, (kb != kb0 || j != 0) ? 1u : 0u);
              tc_mma_tf32_pair(d, ahd, bld, IDESC, 1u);
              tc_mma_tf32_pair(d, ahd, bhd, IDESC, 1u);
            }
            tc_commit_pair(map_to_cta(empty_bar(stage), 0));
            tc_commit_pair(map_to_cta(empty_bar(stage), 1));
            if (++stage == X_STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) {
            tc_commit_pair(map_to_cta(tfull_bar(buf), 0));
            tc_commit_pair(map_to_cta(tfull_bar(buf), 1));
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const uint32_t staging = smem_u32(smem + X_OFF_STAGING) + (warp - 2) * STAGING_BYTES;
    const EpiParams ep = resolve_scales(ep_in);
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;        // which 128 of the 256 columns
    const int e = threadIdx.x - 64;          // 0..255
    const int nchunks = (kblocks + CHUNK_STAGES - 1) / CHUNK_STAGES;
    uint32_t c_local = 0, t_local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++t_local) {
      int tm, tn;
      tile_coords(tile, tiles_m2, tiles_n, tm, tn);
      const int m0 = tm * 2 * TBM + (int)rank * TBM, n0 = tn * TBN;
      // bias slice of this tile (one buffer per tile parity; the barrier also orders its reuse)
      const uint32_t bbuf = t_local & 1u;
      float* bs = bias_s + bbuf * TBN;
      {
        const int n = n0 + e;
        float bv = 0.0f;
        if (n < N) bv = bias_dtype == kF16    ? __half2float(static_cast<const __half*>(bias)[n])
                        : bias_dtype == kBF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n])
                                              : static_cast<const float*>(bias)[n];
        bs[e] = bv;
      }
      mbar_arrive(bias_bar(bbuf));
      if (!mbar_wait(bias_bar(bbuf), (t_local >> 1) & 1u, abort_flag, status, kWdBias)) break;

      float part[128];                       // this thread's row, 128 columns: FP32 sums over the chunks
#pragma unroll
      for (int i = 0; i < 128; ++i) part[i] = 0.0f;
      for (int ch = 0; ch < nchunks; ++ch, ++c_local) {
        const uint32_t buf = c_local & 1u, use = c_local >> 1;
        if (!mbar_wait(tfull_bar(buf), use & 1u, abort_flag, status, kWdTmemFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * TBN + half * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(t_row + c * 32, acc);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) part[c * 32 + i] = __fadd_rn(part[c * 32 + i], __uint_as_float(acc[i]));
        }
        tc_fence_before();
        mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));      // the chunk buffer goes back to the MMA issuer
      }
      if (!ok) break;

      const int row0 = m0 + q * 32;
      const int nc = n0 + half * 128;
      const float* bsh = bs + half * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32], w[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(part[c * 32 + i]);
        epilogue_chunk<EPI, float, false>(r, bsh + c * 32, ep, w);
        if (lane == 0) bulk_wait_read_all();   // the previous box has left the staging buffer
        __syncwarp();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          staging_store16(staging, lane, g, make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]));
        fence_async_smem();
        __syncwarp();
        const int x = nc + c * 32;
        if (lane == 0 && x < N && row0 < M) {
          tma_store_2d(&tmC, staging, x, row0);
          bulk_commit();
        }
      }
    }
    if (lane == 0) bulk_wait_all();
  }

  // ------------------------------------------------------------------ tear-down
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace tf32x3
}  // namespace tfb
