// attention_tc_kernel.cuh -- device side of the fused multi-head attention
// forward for FP16 tensors with 64-wide heads:
//     out = dropout(softmax(scale * Q K^T)) V     per (batch item, head)
// The probabilities never reach device memory.  (The reference declares this
// operator and leaves it empty: reference src/tensorfuse_c_api.cpp:288-311.)
//
// A work item is 128 query rows of one head; its keys are walked in blocks of
// 128.  The kernel is persistent: two CTAs per SM (112 KB of shared memory, 256
// TMEM columns each) take work items round-robin, so TMEM allocation, barrier
// set-up and descriptor fetches happen once, the next item's Q, K, V arrive and
// its first scores are computed while the current item's output rows are
// normalised and stored, and one CTA's softmax arithmetic overlaps the other's
// tensor-core work.
//   warp 0, one lane : TMA producer.  Q of this and of the next item (two stages); K and V blocks into a 2-deep ring
//                      of 128-byte-swizzled boxes (4-D tensor maps: any batch /
//                      sequence / head strides, zero fill past the sequence end).
//   warp 1, one lane : tcgen05.mma issuer.  S = Q K_j^T (M 128, N 128, K 64: both
//                      operands K-major) into TMEM columns 0..127; O += P_j V_j
//                      (M 128, N 64, K 128: P read from TMEM columns 192..255,
//                      V as stored, i.e. MN-major) into columns 128..191.  S_{j+1} is
//                      issued as soon as the softmax warps have read S_j.
//   warps 2-5        : softmax.  Thread = query row = TMEM lane, so row maxima
//                      and sums need no shuffles.  Pass 1 reads the 128 scores
//                      of the row for the block maximum; pass 2 reads them again,
//                      exponentiates in the base-2 domain (scale * log2 e folded
//                      into one FMA), applies the dropout decisions, and writes
//                      the FP16 probabilities back to TMEM (tcgen05.st), from
//                      where the second product reads them as its A operand:
//                      they never touch shared memory.  When the
//                      running maximum moves, the same thread rescales its O row
//                      in TMEM (tcgen05.ld / st) before releasing P to the MMA
//                      issuer.  The final O row is divided by the row sum, scaled
//                      by 1/(1-p), converted and staged; each warp stores its own 32
//                      rows through TMA, so the warps never wait for one another.
// Every mbarrier wait is bounded (ptx.cuh): an expired wait raises the CTA abort
// flag, records a code in the watchdog word, and all roles fall through to the
// tear-down that frees TMEM.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "philox.cuh"
#include "ptx.cuh"

namespace tfb {
namespace attn {

constexpr int BQ = 128;    // query rows per CTA
constexpr int BKV = 128;   // keys per block
constexpr int HD = 64;     // head width
constexpr int KV_STAGES = 2;
constexpr float kRescaleSlack = 8.0f;   // log2 of the largest unnormalised probability kept without rescaling
constexpr int TILE_BYTES = 128 * 128;          // 128 rows of 64 FP16
constexpr int NUM_THREADS = 192;
constexpr int SOFTMAX_THREADS = 128;
constexpr int TMEM_COLS = 256;                 // S: 0..127, O: 128..191, P (FP16 pairs): 192..255
constexpr int Q_STAGES = 2;                    // the next item's query rows arrive during the current item
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_STAGES * TILE_BYTES;
constexpr int OFF_V = OFF_K + KV_STAGES * TILE_BYTES;
constexpr int OFF_P = OFF_V + KV_STAGES * TILE_BYTES;   // staging box of the output rows
constexpr int OFF_BAR = OFF_P + TILE_BYTES;
// barriers: q_full[2], q_empty[2], k_full[2], v_full[2], k_empty[2], v_empty[2], s_full, s_free, p_full, o_done
constexpr int NUM_BARS = 2 * Q_STAGES + 4 * KV_STAGES + 4;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16;
static_assert(2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs per SM");

// watchdog codes of this kernel
enum : int { kWdQ = 201, kWdKFull = 202, kWdVFull = 203, kWdKEmpty = 204, kWdVEmpty = 205, kWdSFull = 206,
             kWdSFree = 207, kWdPFull = 208, kWdODone = 209, kWdAlign = 210 };

struct Params {
  int batch, heads, seq_q, seq_kv;
  int q_tiles, n_tiles;  // query tiles per (batch item, head); work items in all
  float scale_log2;      // scale * log2(e)
  float keep_scale;      // 1/(1-p)
  uint32_t thr, thr_h2;  // dropout threshold (see philox.cuh); thr_h2 = thr in both halves
  int hcmp;              // thr <= 0x7C00: compare two fields with one packed FP16 compare
  const int* kv_lengths;
  uint32_t key[20];
};

struct TrueT { static constexpr bool value = true; };
struct FalseT { static constexpr bool value = false; };
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^t for t <= 0 without the exponent unit: round-to-nearest range reduction
// through the 1.5 * 2^23 constant, a degree-3 polynomial for 2^f on [-0.5, 0.5]
// (maximum relative error 7.5e-5, a quarter of an FP16 half-ulp), the integer
// part added to the exponent bits.  A quarter of the exponentials of the
// dropout-free kernel go this way: the exponent unit (16 results per clock
// and SM) is what bounds that kernel, the FMA pipe has room.
__device__ __forceinline__ float exp2_poly3(float t) {
  t = fmaxf(t, -125.0f);
  const float y = t + 12582912.0f;
  const float f = t - (y - 12582912.0f);
  float q = fmaf(f, 0x1.c3f6fp-5f, 0x1.f0ddf6p-3f);
  q = fmaf(q, f, 0x1.62f31ap-1f);
  q = fmaf(q, f, 0x1.fff694p-1f);
  return __int_as_float(__float_as_int(q) + (__float_as_int(y) << 23));
}

// Two FP32 values -> one word of two 16-bit values of the tensor's type.
template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// BF16 = false: FP16 tensors; true: BF16 tensors (same layouts, the MMAs take the
// other 16-bit format, probabilities and output are rounded to BF16).
template <bool DROP, bool BF16>
__global__ void __launch_bounds__(NUM_THREADS, 2)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO32,
                    const __grid_constant__ Params p, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0u) {
    if (threadIdx.x == 0 && status != nullptr) *reinterpret_cast<volatile int*>(status) = kWdAlign;
    return;
  }
  const uint32_t sQ = smem_u32(smem + OFF_Q), sK = smem_u32(smem + OFF_K), sV = smem_u32(smem + OFF_V),
                 sP = smem_u32(smem + OFF_P);
  const uint32_t bars = smem_u32(smem + OFF_BAR);
  auto q_full = [&](uint32_t s) { return bars + 8u * s; };
  auto q_empty = [&](uint32_t s) { return bars + 8u * (Q_STAGES + s); };
  constexpr int KB = 2 * Q_STAGES;
  auto k_full = [&](int s) { return bars + 8u * (KB + s); };
  auto v_full = [&](int s) { return bars + 8u * (KB + KV_STAGES + s); };
  auto k_empty = [&](int s) { return bars + 8u * (KB + 2 * KV_STAGES + s); };
  auto v_empty = [&](int s) { return bars + 8u * (KB + 3 * KV_STAGES + s); };
  const uint32_t bar_s_full = bars + 8u * (KB + 4 * KV_STAGES);
  const uint32_t bar_s_free = bar_s_full + 8u, bar_p_full = bar_s_full + 16u, bar_o_done = bar_s_full + 24u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Work item t -> (query tile, head, batch item); the query tile runs fastest so
  // that CTAs working side by side read the same K and V from L2.
  auto tile_coords = [&](int t, int& q0, int& h, int& b, int& kv_len) {
    const int qt = t % p.q_tiles;
    const int rest = t / p.q_tiles;
    h = rest % p.heads;
    b = rest / p.heads;
    q0 = qt * BQ;
    kv_len = p.seq_kv;
    if (p.kv_lengths != nullptr) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < Q_STAGES; ++s) { mbar_init(q_full(s), 1); mbar_init(q_empty(s), 1); }
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1); mbar_init(v_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_empty(s), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_s_free, SOFTMAX_THREADS);
    mbar_init(bar_p_full, SOFTMAX_THREADS);
    mbar_init(bar_o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmO32);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Counters that run across the work items of this CTA: `wt` counts items with
  // at least one key block (phases of the Q barriers), `g` counts key blocks
  // (ring stage and phases of the per-block barriers).
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t wt = 0, g = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
        int q0, h, b, kv_len;
        tile_coords(t, q0, h, b, kv_len);
        const int nblk = (kv_len + BKV - 1) / BKV;
        if (nblk == 0) continue;
        const uint32_t qs = wt % Q_STAGES, qph = (wt / Q_STAGES) & 1u;
        if (!mbar_wait(q_empty(qs), qph ^ 1u, abort_flag, status, kWdQ)) break;
        mbar_arrive_expect_tx(q_full(qs), TILE_BYTES);
        tma_load_4d(sQ + qs * TILE_BYTES, &tmQ, q_full(qs), 0, q0, h, b);
        ++wt;
        for (int j = 0; j < nblk; ++j, ++g) {
          const int s = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1u;
          if (!mbar_wait(k_empty(s), ph ^ 1u, abort_flag, status, kWdKEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(k_full(s), TILE_BYTES);
          tma_load_4d(sK + s * TILE_BYTES, &tmK, k_full(s), 0, j * BKV, h, b);
          if (!mbar_wait(v_empty(s), ph ^ 1u, abort_flag, status, kWdVEmpty)) { ok = false; break; }
          mbar_arrive_expect_tx(v_full(s), TILE_BYTES);
          tma_load_4d(sV + s * TILE_BYTES, &tmV, v_full(s), 0, j * BKV, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t FMT = BF16 ? 1u : 0u;
      constexpr uint32_t IDESC_S = make_idesc_major(1u, FMT, 0u, 0u, BQ, BKV);   // Q, K: K-major
      constexpr uint32_t IDESC_O = make_idesc_major(1u, FMT, 0u, 1u, BQ, HD);    // P K-major, V MN-major
      const uint32_t tS = tmem_base, tO = tmem_base + 128, tP = tmem_base + 192;
      // S = Q K^T of key block number gi (counted over the whole CTA)
      // `qi` = number of the item (with key blocks) the block belongs to: selects the Q stage
      auto issue_s = [&](uint32_t gi, uint32_t qi, bool last_of_item) -> bool {
        const uint32_t qs = qi % Q_STAGES;
        const int s = gi % KV_STAGES;
        const uint32_t ph = (gi / KV_STAGES) & 1u;
        if (!mbar_wait(k_full(s), ph, abort_flag, status, kWdKFull)) return false;
        if (gi > 0 && !mbar_wait(bar_s_free, (gi - 1) & 1u, abort_flag, status, kWdSFree)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          tc_mma_f16(tS, make_smem_desc(sQ + qs * TILE_BYTES + kk * 32, 16, 1024),
                     make_smem_desc(sK + s * TILE_BYTES + kk * 32, 16, 1024), IDESC_S, kk != 0 ? 1u : 0u);
        tc_commit(bar_s_full);
        tc_commit(k_empty(s));
        if (last_of_item) tc_commit(q_empty(qs));     // this Q stage may take another item's rows
        return true;
      };
      uint32_t wt = 0, g = 0;
      bool ok = true;
      // first scores of the first item with work
      int t = blockIdx.x, nblk = 0;
      auto next_item = [&]() {        // advance t to the next item that has key blocks; sets nblk
        for (; t < p.n_tiles; t += gridDim.x) {
          int q0, h, b, kv_len;
          tile_coords(t, q0, h, b, kv_len);
          nblk = (kv_len + BKV - 1) / BKV;
          if (nblk > 0) return true;
        }
        return false;
      };
      bool have = next_item();
      // wt = items started so far; the current item is number wt - 1
      if (have) {
        ok = mbar_wait(q_full(wt % Q_STAGES), (wt / Q_STAGES) & 1u, abort_flag, status, kWdQ);
        ++wt;
        ok = ok && issue_s(g, wt - 1, nblk == 1);
      }
      while (have && ok) {
        const int nb = nblk;
        for (int j = 0; j < nb && ok; ++j, ++g) {
          if (j + 1 < nb) {
            if (!issue_s(g + 1, wt - 1, j + 2 == nb)) { ok = false; break; }
          } else {
            // the scores of the next item's first block go out before this item's last P V
            t += gridDim.x;
            have = next_item();
            if (have) {
              if (!mbar_wait(q_full(wt % Q_STAGES), (wt / Q_STAGES) & 1u, abort_flag, status, kWdQ)) { ok = false; break; }
              ++wt;
              if (!issue_s(g + 1, wt - 1, nblk == 1)) { ok = false; break; }
            }
          }
          const int s = g % KV_STAGES;
          const uint32_t ph = (g / KV_STAGES) & 1u;
          if (!mbar_wait(bar_p_full, g & 1u, abort_flag, status, kWdPFull)) { ok = false; break; }
          if (!mbar_wait(v_full(s), ph, abort_flag, status, kWdVFull)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk)
            tc_mma_f16_ts(tO, tP + kk * 8, make_smem_desc(sV + s * TILE_BYTES + kk * 2048, TILE_BYTES, 1024),
                          IDESC_O, (j | kk) != 0 ? 1u : 0u);
          tc_commit(bar_o_done);
          tc_commit(v_empty(s));
        }
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    const int qtr = warp & 3;                 // TMEM lane quarter this warp may touch
    const int row = qtr * 32 + lane;          // tile row = TMEM lane
    const uint32_t tS = tmem_base + (static_cast<uint32_t>(qtr * 32) << 16);
    const uint32_t tO = tS + 128, tP = tS + 192;
    const float sl2 = p.scale_log2;
    bool ok = true;
    bool store_pending = false;               // a TMA store may still be reading the staging box
    uint32_t g = 0;                           // key blocks processed by this CTA so far
    uint32_t r[2][32];
    unsigned long long blk_row = 0;           // Philox block index of element (b, h, q0 + row, 0)
    // the warp leaves a wait together, so the .aligned TMEM instructions stay convergent
    auto wait_warp = [&](uint32_t bar, uint32_t parity, int code) {
      return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, abort_flag, status, code)) != 0;
    };
    // Each warp stages and stores its own 32 output rows (a 4 KB slice of the
    // box): the slice is written again only after the warp's previous store has read it.
    const uint32_t sPw = sP + qtr * (32 * 128);
    auto staging_ready = [&]() {
      if (store_pending) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        store_pending = false;
        __syncwarp();
      }
    };
    // Pass 1: maximum of the 128 scores of the row.  TAIL: the block holds fewer
    // than 128 real keys (columns >= valid are zero-filled, not scores).
    auto pass1 = [&](auto tail_c, int valid) -> float {
      constexpr bool TAIL = decltype(tail_c)::value;
      float mx0 = -INFINITY, mx1 = -INFINITY;
      tmem_ld_32x32(tS, r[0]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld_wait();
        if (c < 3) tmem_ld_32x32(tS + (c + 1) * 32, r[(c + 1) & 1]);
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            x[u] = __uint_as_float(r[c & 1][i + u]);
            if (TAIL && c * 32 + i + u >= valid) x[u] = -INFINITY;
          }
          mx0 = max3(mx0, x[0], x[1]);
          mx1 = max3(mx1, x[2], x[3]);
        }
      }
      return fmaxf(mx0, mx1);
    };
    // Pass 2: unnormalised probabilities 2^(s*scale*log2e - m), their FP32 sum,
    // dropout, FP16 tile P (K-major, 128-byte swizzle).  Returns the row sum.
    auto pass2 = [&](auto tail_c, int valid, int j, float m_new) -> float {
      constexpr bool TAIL = decltype(tail_c)::value;
      uint64_t ls2 = pack2(0.0f, 0.0f);
      const uint64_t sl2_2 = pack2(sl2, sl2), nm_2 = pack2(-m_new, -m_new);
      tmem_ld_32x32(tS, r[0]);
      // Two chunks per trip (the two register buffers alternate), the trip itself not
      // unrolled: half the code of a fully unrolled sweep, which matters for the
      // instruction cache with two CTAs' warps at different places of this kernel.
      auto chunk = [&](int c, const uint32_t (&rc)[32]) {
        // dropout decisions of the 32 keys of this chunk: four Philox blocks at once
        uint32_t km[4][4];
        if (DROP) {
          const unsigned long long blk = blk_row + (unsigned)(j * (BKV / 8) + c * 4);
          uint32_t o[4][4];
          philox_block_x4(blk, p.key, o);
          const __half2 thr2 = *reinterpret_cast<const __half2*>(&p.thr_h2);
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (p.hcmp) {
                const uint32_t f = o[gq][k] & 0x7FFF7FFFu;
                km[gq][k] = __hgeu2_mask(*reinterpret_cast<const __half2*>(&f), thr2);
              } else {
                km[gq][k] = ((o[gq][k] & 0x7FFFu) >= p.thr ? 0x0000FFFFu : 0u) |
                            (((o[gq][k] >> 16) & 0x7FFFu) >= p.thr ? 0xFFFF0000u : 0u);
              }
            }
        }
        uint32_t w[16];                       // 32 probabilities as FP16 pairs
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const int i = 2 * k;
          // one packed FMA for the pair (the two scores sit in an aligned register pair)
          const float2 t = unpack2(fma2(pack2(__uint_as_float(rc[i]), __uint_as_float(rc[i + 1])), sl2_2, nm_2));
          float e0, e1;
          if (!DROP && (k & 3) == 3) { e0 = exp2_poly3(t.x); e1 = exp2_poly3(t.y); }
          else { e0 = ex2_approx(t.x); e1 = ex2_approx(t.y); }
          if (TAIL) {
            if (c * 32 + i >= valid) e0 = 0.0f;
            if (c * 32 + i + 1 >= valid) e1 = 0.0f;
          }
          ls2 = add2(ls2, pack2(e0, e1));
          w[k] = pack16<BF16>(e0, e1);
          if (DROP) w[k] &= km[k >> 2][k & 3];
        }
        tmem_st_32x16(tP + c * 16, w);
      };
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_wait();
        tmem_ld_32x32(tS + (2 * cc + 1) * 32, r[1]);
        chunk(2 * cc, r[0]);
        tmem_ld_wait();
        if (cc == 0) tmem_ld_32x32(tS + 64, r[0]);
        else {
          tc_fence_before();
          mbar_arrive(bar_s_free);            // S may be overwritten by the next block's scores
        }
        chunk(2 * cc + 1, r[1]);
      }
      tmem_st_wait();
      const float2 ls = unpack2(ls2);
      return ls.x + ls.y;
    };

    for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
      int q0, h, b, kv_len;
      tile_coords(t, q0, h, b, kv_len);
      const int nblk = (kv_len + BKV - 1) / BKV;
      blk_row = ((((unsigned long long)b * p.heads + h) * p.seq_q + (unsigned long long)(q0 + row)) *
                 (unsigned long long)p.seq_kv) >> 3;
      float m_run = -INFINITY, l_run = 0.0f;
      for (int j = 0; j < nblk && ok; ++j, ++g) {
        if (!wait_warp(bar_s_full, g & 1u, kWdSFull)) { ok = false; break; }
        tc_fence_after();
        const int valid = kv_len - j * BKV;     // columns of this block that are real keys
        const bool tail = valid < BKV;
        const float mx = tail ? pass1(TrueT{}, valid) : pass1(FalseT{}, valid);
        // The reference point of the exponentials moves only when the block maximum
        // exceeds it by more than 2^8: probabilities up to 256 are as exact in 16 bits
        // as probabilities up to 1, the row sum is taken against the same reference,
        // and the O row is then rescaled for the first block of an item and almost
        // never again.
        const float mb = mx * sl2;
        const float m_new = mb > m_run + kRescaleSlack ? mb : m_run;
        const float alpha = m_new == m_run ? 1.0f : ex2_approx(m_run - m_new);     // 0 on the first block
        // P and O are still in use by the previous block's second MMA
        if (j > 0 && !wait_warp(bar_o_done, (g - 1) & 1u, kWdODone)) { ok = false; break; }
        tc_fence_after();
        const float ls = tail ? pass2(TrueT{}, valid, j, m_new) : pass2(FalseT{}, valid, j, m_new);
        l_run = fmaf(l_run, alpha, ls);
        m_run = m_new;
        // rescale the O row when the maximum of any row of this warp moved
        if (j > 0 && __any_sync(0xFFFFFFFFu, alpha != 1.0f)) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tmem_ld_32x32(tO + c * 32, r[0]);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[0][i] = __float_as_uint(__uint_as_float(r[0][i]) * alpha);
            tmem_st_32x32(tO + c * 32, r[0]);
          }
          tmem_st_wait();
        }
        tc_fence_before();
        mbar_arrive(bar_p_full);
      }
      // ---------------------------------------------------------- final O rows
      if (ok && nblk > 0) ok = wait_warp(bar_o_done, (g - 1) & 1u, kWdODone);
      if (!ok) break;
      tc_fence_after();
      staging_ready();
      const float inv = nblk > 0 && l_run > 0.0f ? p.keep_scale / l_run : 0.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (nblk > 0) { tmem_ld_32x32(tO + c * 32, r[0]); tmem_ld_wait(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[0][i] = 0u;
        }
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = gq * 8 + 2 * k;
            w[k] = pack16<BF16>(__uint_as_float(r[0][i]) * inv, __uint_as_float(r[0][i + 1]) * inv);
          }
          const uint32_t addr = sP + row * 128 + (((c * 4 + gq) ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();                       // the O reads above precede the next item's first P V
      __syncwarp();
      if (lane == 0 && q0 + qtr * 32 < p.seq_q) {
        tma_store_4d(&tmO32, sPw, 0, q0 + qtr * 32, h, b);
        bulk_commit_group();
      }
      store_pending = true;
    }
    if (lane == 0) bulk_wait_group0();
  }

  // ------------------------------------------------------------------ tear-down
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace attn
}  // namespace tfb
