// gemm_tc_pair_kernel.cuh -- the CTA-pair (tcgen05 cta_group::2) form of the
// tensor-core GEMM + bias + GELU.
//
// Two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 output
// tile.  Each CTA loads its own 128 rows of A and its own 128 of the tile's 256
// columns of B per K step; the leader's one tcgen05.mma.cta_group::2
// instruction drives both tensor cores, each of which accumulates its 128 rows
// x 256 columns in its own TMEM while the hardware feeds the two B halves to
// both.  Per SM and K step that is 32 KB through shared memory instead of the
// 48 KB of the single-CTA 128 x 256 form, which is what bounds that form (its
// shared-memory port carries operand reads and TMA writes together).
//   * both CTAs : warp 0 (one lane) TMA producer for its own operand halves,
//                 byte counts signalled on the LEADER's "full" barrier
//                 (the cta_group::2 form of the tensor load; every load is
//                 addressed to one CTA's shared memory only);
//                 warps 2-9 epilogue of their own 128 x 256 accumulator, as in
//                 the single-CTA kernel (same code).
//   * leader    : warp 1 (one lane) issues the MMAs and commits to the "empty"
//                 barrier of each CTA (two plain commits, one per CTA) and to
//                 both "accumulator ready" barriers; it waits on one
//                 "accumulator drained" barrier that both CTAs' epilogue threads
//                 arrive on (the peer's through a shared::cluster arrive).
// Every wait is bounded as in the single-CTA kernel; the two CTAs rendezvous on
// the cluster barrier after set-up and before tear-down, so neither touches the
// other's shared memory or barriers outside that window.
#pragma once
#include "gemm_tc_kernel.cuh"

namespace tfb {
namespace tc2 {

using namespace tc;

constexpr int P_STAGES = 6;
constexpr int P_A_STAGE_BYTES = TBM * 128;        // 128 rows x 128 bytes of K
constexpr int P_B_STAGE_BYTES = 128 * 128;        // this CTA's 128 columns x 128 bytes-worth of K rows
constexpr int P_STAGE_BYTES = P_A_STAGE_BYTES + P_B_STAGE_BYTES;
constexpr int P_OFF_A = 0;
constexpr int P_OFF_B = P_OFF_A + P_STAGES * P_A_STAGE_BYTES;
constexpr int P_OFF_STAGING = P_OFF_B + P_STAGES * P_B_STAGE_BYTES;
constexpr int P_OFF_BIAS = P_OFF_STAGING + EPI_WARPS * STAGING_BYTES;
constexpr int P_OFF_BAR = P_OFF_BIAS + 2 * TBN * 4;
// barriers: full[S], empty[S], tmem_full[2], tmem_empty[2], bias_ready[2]
constexpr int P_NUM_BARS = 2 * P_STAGES + 6;
constexpr int P_OFF_MISC = P_OFF_BAR + P_NUM_BARS * 8;
constexpr int P_SMEM_BYTES = P_OFF_MISC + 16;
static_assert(P_SMEM_BYTES <= 232448, "exceeds the 227 KB a CTA may use");

template <int KIND, int EPI, typename TOut>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const void* __restrict__ bias, int bias_dtype,
                    int M, int N, int K, EpiParams ep_in, int* status) {
  using KT = KindTraits<KIND>;
  constexpr int ES = KT::ES;
  constexpr int BKE = 128 / ES;                    // K elements per stage
  constexpr int MMA_PER_STAGE = 4;                 // 32 bytes of K per MMA
  constexpr int B_BOX_COLS = 128 / ES;             // N elements per B box (128 bytes wide)
  constexpr int B_BOXES = 128 / B_BOX_COLS;        // boxes of this CTA's 128 columns
  constexpr int B_BOX_BYTES = 128 * BKE;           // BKE rows of 128 bytes
  constexpr int B_K_STEP_BYTES = (32 / ES) * 128;  // K rows per MMA x 128 bytes
  constexpr uint32_t IDESC = make_idesc(KT::C_FORMAT, KT::AB_FORMAT, 2 * TBM, TBN);   // M 256 over the pair

  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const bool aligned = (smem_u32(smem) & 1023u) == 0u;
  const uint32_t sA = smem_u32(smem + P_OFF_A);
  const uint32_t sB = smem_u32(smem + P_OFF_B);
  float* bias_s = reinterpret_cast<float*>(smem + P_OFF_BIAS);
  const uint32_t bars = smem_u32(smem + P_OFF_BAR);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (P_STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * P_STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * P_STAGES + 2 + b); };
  auto bias_bar = [&](int b) { return bars + 8u * (2 * P_STAGES + 4 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + P_OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + P_OFF_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + TBN - 1) / TBN;
  const int tiles_m2 = (M + 2 * TBM - 1) / (2 * TBM);       // 256-row pair tiles
  const int num_tiles = tiles_m2 * tiles_n;
  const int kblocks = (K + BKE - 1) / BKE;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * EPI_THREADS);     // both CTAs' epilogue threads (only the leader's copy is used)
      mbar_init(bias_bar(b), EPI_THREADS);
    }
    *abort_flag = aligned ? 0 : 1;
    if (!aligned && status != nullptr) *reinterpret_cast<volatile int*>(status) = kWdAlign;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = !*abort_flag;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, tiles_m2, tiles_n, tm, tn);
        const int m0 = tm * 2 * TBM + (int)rank * TBM, n0 = tn * TBN + (int)rank * 128;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, kWdEmpty)) { ok = false; break; }
          const uint32_t full_leader = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);
          tma_load_2d_pair(sA + stage * P_A_STAGE_BYTES, &tmA, full_leader, kb * BKE, m0);
#pragma unroll
          for (int j = 0; j < B_BOXES; ++j)
            tma_load_2d_pair(sB + stage * P_B_STAGE_BYTES + j * B_BOX_BYTES, &tmB, full_leader,
                             n0 + j * B_BOX_COLS, kb * BKE);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------- MMA issuer (leader CTA)
    if (leader && elect_one()) {
      uint32_t stage = 0, phase = 0, t_local = 0;
      bool ok = !*abort_flag;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++t_local) {
        const uint32_t buf = t_local & 1u, use = t_local >> 1;
        if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u, abort_flag, status, kWdTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * TBN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, status, kWdFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a0 = sA + stage * P_A_STAGE_BYTES, b0 = sB + stage * P_B_STAGE_BYTES;
#pragma unroll
          for (int j = 0; j < MMA_PER_STAGE; ++j) {
            const uint64_t adesc = make_smem_desc(a0 + j * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc(b0 + j * B_K_STEP_BYTES, B_BOX_BYTES, 1024);
            const uint32_t accumulate = (kb | j) != 0 ? 1u : 0u;
            if (KIND == 0 || KIND == 2) tc_mma_f16_pair(d, adesc, bdesc, IDESC, accumulate);
            else if (KIND == 1) tc_mma_i8_pair(d, adesc, bdesc, IDESC, accumulate);
            else tc_mma_f8_pair(d, adesc, bdesc, IDESC, accumulate);
          }
          tc_commit_pair(map_to_cta(empty_bar(stage), 0));
          tc_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          tc_commit_pair(map_to_cta(tfull_bar(buf), 0));
          tc_commit_pair(map_to_cta(tfull_bar(buf), 1));
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const uint32_t staging = smem_u32(smem + P_OFF_STAGING) + (warp - 2) * STAGING_BYTES;
    const EpiParams ep = resolve_scales(ep_in);
    uint32_t t_local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++t_local) {
      const uint32_t buf = t_local & 1u, use = t_local >> 1;
      int tm, tn;
      tile_coords(tile, tiles_m2, tiles_n, tm, tn);
      const uint32_t tempty_leader = map_to_cta(tempty_bar(buf), 0);
      if (!epilogue_tile<EPI, TOut, KT::kIntAcc>(&tmC, bias, bias_dtype, M, N, tm * 2 * TBM + (int)rank * TBM, tn * TBN,
                                                 buf, use, bias_s, staging, bias_bar(buf), tfull_bar(buf), tmem_base, ep,
                                                 abort_flag, status, [&] { mbar_arrive_cluster(tempty_leader); }))
        break;
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
  cluster_sync_all();          // the peer is done with this CTA's shared memory, barriers and TMEM
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace tc2
}  // namespace tfb
