// softmax_dropout.cu -- fused row softmax + dropout for sm_100a.
//
// Replaces the reference kernels fused_softmax_dropout_warp_kernel /
// fused_softmax_dropout_kernel (reference src/kernels/fused_softmax_dropout.cu:39-233):
//   m = max_j x_j;  e_j = exp(x_j - m);  y_j = e_j / sum_j e_j;
//   keep_j = (p == 0) or (u_j > p);  out_j = keep_j ? y_j / (1-p) : 0;  mask_j = keep_j
// with FP32 arithmetic on FP16 or FP32 storage.
//
// Memory-bound by construction (2 B read + 2 B write + 1 B mask per FP16
// element), so the kernels are organised around 16-byte accesses and a row that
// stays in registers between the reductions and the store:
//   * warp-per-row kernel for rows up to 2048 elements: lane l owns the 8-element
//     units l, l+32, ...; one 128-bit load per unit, shuffle reductions, one
//     128-bit store plus one 64-bit mask store per unit; the next row's loads are
//     issued before the current row is processed.
//   * CTA-per-row kernel for longer or unaligned rows: three passes over a row
//     that is L2-resident after the first.
//
// Arithmetic is written so that a CPU can reproduce every bit: the exponential
// is a round-to-nearest range reduction plus a degree-5 FMA polynomial (no
// MUFU), sums follow a fixed schedule (two accumulators per thread, xor
// butterfly per warp, warps in ascending order), the reciprocal is IEEE.  The
// packed fma/add/mul.f32x2 instructions of sm_100 keep the instruction count of
// that polynomial close to a MUFU-based one.
//
// Dropout uses Philox4x32 with 7 rounds (philox.cuh): eight consecutive elements share one block
// (counter = global element index / 8, key = seed), each element takes a 16-bit
// field and is kept when its low 15 bits are >= round(p * 32768).  The counter depends only on
// the element's position in the whole tensor, so any row-sharding across GPUs
// reproduces the same mask.
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "kernels.h"
#include "philox.cuh"
#include "ptx.cuh"

namespace tfb {
namespace {

struct SmParams {
  const void* in;
  void* out;
  unsigned char* mask;
  long long rows;
  int L;
  float keep_scale;              // 1/(1-p), 0 when p >= 1
  uint32_t thr;                  // drop when the 15-bit field < thr (thr = round(p * 32768))
  uint32_t thr_h2;               // thr in both halves of a word, for the packed FP16 compare
  int hcmp;                      // thr <= 0x7C00: 15-bit fields order like positive FP16 numbers
  unsigned long long first_row;  // row offset of this shard inside the whole tensor
  uint32_t key[20];              // Philox round keys
  // extended form (scores scaled and key-length masked on load); unused otherwise
  float scale;                   // softmax(scale * x)
  const int* lengths;            // valid row length per batch item, or null
  long long rows_per_item;       // rows that share one entry of `lengths`
};

// Extended form: x <- scale * x for columns below the valid length, -inf from
// there on.  The arithmetic that follows is the FP32-storage one whatever the
// storage type, so that one CPU restatement covers both.
template <bool EXT>
__device__ __forceinline__ void adjust8(float (&x)[8], int col0, int len, float scale) {
  if constexpr (EXT) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = (col0 + i < len) ? __fmul_rn(x[i], scale) : -INFINITY;
  }
}
template <bool EXT>
__device__ __forceinline__ float adjust1(float x, int col, int len, float scale) {
  if constexpr (EXT) return col < len ? __fmul_rn(x, scale) : -INFINITY;
  return x;
}
template <bool EXT>
__device__ __forceinline__ int valid_length(const SmParams& p, long long row) {
  if constexpr (EXT) {
    if (p.lengths == nullptr) return p.L;
    const long long b = (long long)((p.first_row + (unsigned long long)row) / (unsigned long long)p.rows_per_item);
    return max(0, min(p.L, p.lengths[b]));
  }
  return p.L;
}

constexpr float kLog2e = 0x1.715476p+0f;
constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
constexpr float kC0 = 0x1.000002p+0f, kC1 = 0x1.62e428p-1f, kC2 = 0x1.ebf918p-3f,
                kC3 = 0x1.c6b6e4p-5f, kC4 = 0x1.3d0c52p-7f, kC5 = 0x1.5c08e6p-10f;

// 2^t for two values t in [-127, ~0] at once; t = -127 yields exactly 0.
__device__ __forceinline__ uint64_t exp2_pair(uint64_t t2) {
  const uint64_t magic2 = pack2(kMagic, kMagic);
  const uint64_t r2 = add2(t2, magic2);
  const uint64_t nf2 = sub2(r2, magic2);
  const uint64_t f2 = sub2(t2, nf2);
  uint64_t p2 = pack2(kC5, kC5);
  p2 = fma2(p2, f2, pack2(kC4, kC4));
  p2 = fma2(p2, f2, pack2(kC3, kC3));
  p2 = fma2(p2, f2, pack2(kC2, kC2));
  p2 = fma2(p2, f2, pack2(kC1, kC1));
  p2 = fma2(p2, f2, pack2(kC0, kC0));
  const float2 r = unpack2(r2);
  const uint32_t s0 = (__float_as_uint(r.x) << 23) + 0x3f800000u;
  const uint32_t s1 = (__float_as_uint(r.y) << 23) + 0x3f800000u;
  return mul2(p2, pack2(__uint_as_float(s0), __uint_as_float(s1)));
}

// FP16-storage form: the inputs have been clamped from below at lo ~ max - 64,
// so t lies in about [-116, 0] and 2^n can be added into the exponent field
// directly; degree-4 polynomial (max relative error 2.7e-6, two orders below an
// FP16 ulp).
constexpr float kD0 = 0x1.ffffe8p-1f, kD1 = 0x1.62e0dcp-1f, kD2 = 0x1.ec06dap-3f,
                kD3 = 0x1.ca144p-5f, kD4 = 0x1.3997d6p-7f;
__device__ __forceinline__ uint64_t exp2_pair_h(uint64_t t2) {
  const uint64_t magic2 = pack2(kMagic, kMagic);
  const uint64_t r2 = add2(t2, magic2);
  const uint64_t nf2 = sub2(r2, magic2);
  const uint64_t f2 = sub2(t2, nf2);
  uint64_t p2 = pack2(kD4, kD4);
  p2 = fma2(p2, f2, pack2(kD3, kD3));
  p2 = fma2(p2, f2, pack2(kD2, kD2));
  p2 = fma2(p2, f2, pack2(kD1, kD1));
  p2 = fma2(p2, f2, pack2(kD0, kD0));
  const float2 r = unpack2(r2), p = unpack2(p2);
  const uint32_t e0 = __float_as_uint(p.x) + (__float_as_uint(r.x) << 23);
  const uint32_t e1 = __float_as_uint(p.y) + (__float_as_uint(r.y) << 23);
  return pack2(__uint_as_float(e0), __uint_as_float(e1));
}

// Row constants of the exponential.  lo is only used by the FP16-storage form.
struct ExpCtx {
  uint64_t log2e2, negc2;
  float lo;
};
// m: row maximum (already 0 for an all -inf row).
template <bool HF>
__device__ __forceinline__ ExpCtx make_exp_ctx(float m) {
  ExpCtx c;
  const float negc = -__fmul_rn(m, kLog2e);
  c.log2e2 = pack2(kLog2e, kLog2e);
  c.negc2 = pack2(negc, negc);
  c.lo = HF ? __half2float(__float2half_rn(__fsub_rn(m, 64.0f))) : 0.0f;
  return c;
}
// FP32 storage: e = 2^(max(x*log2e - c, -127)).
// FP16 storage: e = 2^(max(x, lo)*log2e - c); PRECLAMPED says the caller has
// already applied the max on the packed halves.
template <bool HF, bool PRECLAMPED = false>
__device__ __forceinline__ uint64_t exp_pair(float x0, float x1, const ExpCtx& c) {
  if constexpr (HF) {
    if constexpr (!PRECLAMPED) { x0 = fmaxf(x0, c.lo); x1 = fmaxf(x1, c.lo); }
    return exp2_pair_h(fma2(pack2(x0, x1), c.log2e2, c.negc2));
  } else {
    const float2 t = unpack2(fma2(pack2(x0, x1), c.log2e2, c.negc2));
    return exp2_pair(pack2(fmaxf(t.x, -127.0f), fmaxf(t.y, -127.0f)));
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
__device__ __forceinline__ float warp_sum_butterfly(float v) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// ------------------------------------------------------------ 8-element units
template <typename T> struct Unit;
template <> struct Unit<__half> {
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) { raw = __ldcs(reinterpret_cast<const uint4*>(p)); }
  // default caching: for data that is read again soon (second sweep of a long row, served by L2)
  __device__ __forceinline__ void load_keep(const __half* p) { raw = __ldg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void fill_neg_inf() { raw = make_uint4(0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u, 0xFC00FC00u); }
  __device__ __forceinline__ void widen(float (&x)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
      x[2 * k] = f.x; x[2 * k + 1] = f.y;
    }
  }
};
template <> struct Unit<float> {
  uint4 raw[2];
  __device__ __forceinline__ void load(const float* p) {
    raw[0] = __ldcs(reinterpret_cast<const uint4*>(p));
    raw[1] = __ldcs(reinterpret_cast<const uint4*>(p) + 1);
  }
  __device__ __forceinline__ void load_keep(const float* p) {
    raw[0] = __ldg(reinterpret_cast<const uint4*>(p));
    raw[1] = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  }
  __device__ __forceinline__ void fill_neg_inf() {
    raw[0] = raw[1] = make_uint4(0xFF800000u, 0xFF800000u, 0xFF800000u, 0xFF800000u);
  }
  __device__ __forceinline__ void widen(float (&x)[8]) const {
    x[0] = __uint_as_float(raw[0].x); x[1] = __uint_as_float(raw[0].y);
    x[2] = __uint_as_float(raw[0].z); x[3] = __uint_as_float(raw[0].w);
    x[4] = __uint_as_float(raw[1].x); x[5] = __uint_as_float(raw[1].y);
    x[6] = __uint_as_float(raw[1].z); x[7] = __uint_as_float(raw[1].w);
  }
};

// Keep decisions of one Philox block as four mask words: the low / high half of
// km[k] is 0xFFFF when element 2k / 2k+1 survives.  A decision compares the low
// 15 bits of a 16-bit field with thr; when thr <= 0x7C00 those 15-bit patterns
// order exactly like non-negative FP16 numbers (patterns above 0x7C00 are NaNs,
// for which "greater-or-unordered" is true, as it must be), so one packed FP16
// compare decides two elements.
// Raw Philox words of one block -> the four mask words.
template <bool DROP>
__device__ __forceinline__ void masks_from_words(const SmParams& p, const uint32_t (&o)[4], uint32_t (&km)[4]) {
  if (DROP) {
    if (p.hcmp) {
      const __half2 thr2 = *reinterpret_cast<const __half2*>(&p.thr_h2);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t f = o[k] & 0x7FFF7FFFu;
        km[k] = __hgeu2_mask(*reinterpret_cast<const __half2*>(&f), thr2);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        km[k] = ((o[k] & 0x7FFFu) >= p.thr ? 0x0000FFFFu : 0u) | (((o[k] >> 16) & 0x7FFFu) >= p.thr ? 0xFFFF0000u : 0u);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) km[k] = 0xFFFFFFFFu;
  }
}
template <bool DROP>
__device__ __forceinline__ void keep_masks(const SmParams& p, unsigned long long philox_blk, uint32_t (&km)[4]) {
  if (DROP) {
    uint32_t o[4];
    philox_block((uint32_t)philox_blk, (uint32_t)(philox_blk >> 32), p.key, o);
    if (p.hcmp) {
      const __half2 thr2 = *reinterpret_cast<const __half2*>(&p.thr_h2);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t f = o[k] & 0x7FFF7FFFu;
        km[k] = __hgeu2_mask(*reinterpret_cast<const __half2*>(&f), thr2);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        km[k] = ((o[k] & 0x7FFFu) >= p.thr ? 0x0000FFFFu : 0u) | (((o[k] >> 16) & 0x7FFFu) >= p.thr ? 0xFFFF0000u : 0u);
    }
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) km[k] = 0xFFFFFFFFu;
  }
}

// Scale, drop and store one unit.  e2[k] holds elements 2k, 2k+1.
template <typename T, bool DROP>
__device__ __forceinline__ void finish_unit_masked(const uint64_t (&e2)[4], uint64_t g2, T* out, unsigned char* mask,
                                                   const uint32_t (&km)[4]);
template <typename T, bool DROP>
__device__ __forceinline__ void finish_unit(const uint64_t (&e2)[4], uint64_t g2, T* out,
                                            unsigned char* mask, const SmParams& p,
                                            unsigned long long philox_blk) {
  uint32_t km[4];
  keep_masks<DROP>(p, philox_blk, km);
  finish_unit_masked<T, DROP>(e2, g2, out, mask, km);
}
template <typename T, bool DROP>
__device__ __forceinline__ void finish_unit_masked(const uint64_t (&e2)[4], uint64_t g2, T* out, unsigned char* mask,
                                                   const uint32_t (&km)[4]) {
  uint2 mb;   // one byte per element: byte 0 / 2 of each mask word, reduced to 0 / 1
  mb.x = __byte_perm(km[0], km[1], 0x6420) & 0x01010101u;
  mb.y = __byte_perm(km[2], km[3], 0x6420) & 0x01010101u;
  __stcs(reinterpret_cast<uint2*>(mask), mb);

  float2 y[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) y[k] = unpack2(mul2(e2[k], g2));
  if constexpr (sizeof(T) == 2) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2 h = __floats2half2_rn(y[k].x, y[k].y);
      w[k] = *reinterpret_cast<const uint32_t*>(&h) & km[k];
    }
    __stcs(reinterpret_cast<uint4*>(out), make_uint4(w[0], w[1], w[2], w[3]));
  } else {
    float v[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = (km[k] & 0xFFFFu) ? y[k].x : 0.0f;
      v[2 * k + 1] = (km[k] >> 16) ? y[k].y : 0.0f;
    }
    float4* o4 = reinterpret_cast<float4*>(out);
    __stcs(o4, make_float4(v[0], v[1], v[2], v[3]));
    __stcs(o4 + 1, make_float4(v[4], v[5], v[6], v[7]));
  }
}

// ------------------------------------------------------- warp-per-row kernel
__device__ __forceinline__ uint32_t hmax2_bits(uint32_t a, uint32_t b) {
  const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Dropout decisions of one lane's units of one row.  They depend on positions
// only; up to four Philox blocks are generated with interleaved rounds.
template <int CH, bool DROP>
__device__ __forceinline__ void row_keep_masks(const SmParams& p, long long row, int lane, uint32_t (&km)[CH][4]) {
  const unsigned long long blk0 = ((p.first_row + (unsigned long long)row) * (unsigned long long)p.L) >> 3;
  constexpr int NB = CH < 4 ? CH : 4;
#pragma unroll
  for (int c0 = 0; c0 < CH; c0 += NB) {
    if (DROP) {
      unsigned long long blk[NB];
      uint32_t o[NB][4];
#pragma unroll
      for (int q = 0; q < NB; ++q) blk[q] = blk0 + (unsigned)(lane + 32 * (c0 + q));
      philox_blocks<NB>(blk, p.key, o);
#pragma unroll
      for (int q = 0; q < NB; ++q) masks_from_words<true>(p, o[q], km[c0 + q]);
    } else {
#pragma unroll
      for (int q = 0; q < NB; ++q) masks_from_words<false>(p, km[c0 + q], km[c0 + q]);
    }
  }
}

// One row held by a warp as CH units per lane (unit c of lane l = elements
// (l + 32c)*8 ..): maximum, exponentials e2[c][k] (elements 2k, 2k+1 of unit c)
// and the factor g = keep_scale / sum.  FP16 storage keeps the row packed for
// as long as possible: the maximum and the clamp at lo are taken on half2 words,
// the widening to FP32 happens once.  The order of every operation is fixed
// (it is the order the CPU restatement follows).
template <typename T, int CH, bool EXT>
__device__ __forceinline__ uint64_t row_exponentials(const SmParams& p, const Unit<T> (&cur)[CH], long long row,
                                                     int lane, uint64_t (&e2)[CH][4]) {
  constexpr bool HF = sizeof(T) == 2 && !EXT;
  const int len = valid_length<EXT>(p, row);
  float m;
  if constexpr (HF) {
    uint32_t m2 = 0xFC00FC00u;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const uint4 r = cur[c].raw;
      m2 = hmax2_bits(hmax2_bits(m2, hmax2_bits(r.x, r.y)), hmax2_bits(r.z, r.w));
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) m2 = hmax2_bits(m2, __shfl_xor_sync(0xffffffffu, m2, off));
    const float2 mf = __half22float2(*reinterpret_cast<const __half2*>(&m2));
    m = fmaxf(mf.x, mf.y);
  } else {
    m = -INFINITY;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      float x[8];
      cur[c].widen(x);
      adjust8<EXT>(x, (lane + 32 * c) * 8, len, p.scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, x[i]);
    }
    m = warp_max(m);
  }
  const bool all_masked = m == -INFINITY;   // defined as an all-zero output row
  if (all_masked) m = 0.0f;
  const ExpCtx ctx = make_exp_ctx<HF>(m);

  uint64_t s2 = pack2(0.0f, 0.0f);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    if constexpr (HF) {
      const __half lo_h = __float2half_rn(ctx.lo);
      const __half2 lo2 = __halves2half2(lo_h, lo_h);
      const uint32_t lo_bits = *reinterpret_cast<const uint32_t*>(&lo2);
      const uint32_t w[4] = {cur[c].raw.x, cur[c].raw.y, cur[c].raw.z, cur[c].raw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t xw = hmax2_bits(w[k], lo_bits);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw));
        e2[c][k] = exp_pair<true, true>(f.x, f.y, ctx);
        s2 = add2(s2, e2[c][k]);
      }
    } else {
      float x[8];
      cur[c].widen(x);
      adjust8<EXT>(x, (lane + 32 * c) * 8, len, p.scale);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        e2[c][k] = exp_pair<false>(x[2 * k], x[2 * k + 1], ctx);
        s2 = add2(s2, e2[c][k]);
      }
    }
  }
  const float2 s = unpack2(s2);
  const float total = warp_sum_butterfly(__fadd_rn(s.x, s.y));
  const float inv = (total == 0.0f || all_masked) ? 0.0f : __fdiv_rn(1.0f, total);
  const float g = __fmul_rn(inv, p.keep_scale);
  return pack2(g, g);
}

// The same for NR rows in lockstep: every step is carried out for all rows before
// the next one starts, so that a warp always has NR independent dependency
// chains (shuffle reductions, polynomial evaluations) in flight.  Row for row
// the operations and their order are those of row_exponentials.
template <typename T, int CH, bool EXT, int NR>
__device__ __forceinline__ void rows_exponentials(const SmParams& p, const Unit<T> (&cur)[NR][CH],
                                                  const long long (&row)[NR], int lane, uint64_t (&e2)[NR][CH][4],
                                                  uint64_t (&g2)[NR]) {
  constexpr bool HF = sizeof(T) == 2 && !EXT;
  int len[NR];
  float m[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) len[r] = valid_length<EXT>(p, row[r]);
  if constexpr (HF) {
    uint32_t m2[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      m2[r] = 0xFC00FC00u;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const uint4 v = cur[r][c].raw;
        m2[r] = hmax2_bits(hmax2_bits(m2[r], hmax2_bits(v.x, v.y)), hmax2_bits(v.z, v.w));
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
      for (int r = 0; r < NR; ++r) m2[r] = hmax2_bits(m2[r], __shfl_xor_sync(0xffffffffu, m2[r], off));
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const float2 mf = __half22float2(*reinterpret_cast<const __half2*>(&m2[r]));
      m[r] = fmaxf(mf.x, mf.y);
    }
  } else {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      m[r] = -INFINITY;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        float x[8];
        cur[r][c].widen(x);
        adjust8<EXT>(x, (lane + 32 * c) * 8, len[r], p.scale);
#pragma unroll
        for (int i = 0; i < 8; ++i) m[r] = fmaxf(m[r], x[i]);
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
      for (int r = 0; r < NR; ++r) m[r] = fmaxf(m[r], __shfl_xor_sync(0xffffffffu, m[r], off));
    }
  }
  bool all_masked[NR];
  ExpCtx ctx[NR];
  uint64_t s2[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    all_masked[r] = m[r] == -INFINITY;
    if (all_masked[r]) m[r] = 0.0f;
    ctx[r] = make_exp_ctx<HF>(m[r]);
    s2[r] = pack2(0.0f, 0.0f);
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if constexpr (HF) {
        const __half lo_h = __float2half_rn(ctx[r].lo);
        const __half2 lo2 = __halves2half2(lo_h, lo_h);
        const uint32_t lo_bits = *reinterpret_cast<const uint32_t*>(&lo2);
        const uint32_t w[4] = {cur[r][c].raw.x, cur[r][c].raw.y, cur[r][c].raw.z, cur[r][c].raw.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t xw = hmax2_bits(w[k], lo_bits);
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw));
          e2[r][c][k] = exp_pair<true, true>(f.x, f.y, ctx[r]);
          s2[r] = add2(s2[r], e2[r][c][k]);
        }
      } else {
        float x[8];
        cur[r][c].widen(x);
        adjust8<EXT>(x, (lane + 32 * c) * 8, len[r], p.scale);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          e2[r][c][k] = exp_pair<false>(x[2 * k], x[2 * k + 1], ctx[r]);
          s2[r] = add2(s2[r], e2[r][c][k]);
        }
      }
    }
  }
  float total[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const float2 sp = unpack2(s2[r]);
    total[r] = __fadd_rn(sp.x, sp.y);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
    for (int r = 0; r < NR; ++r) total[r] = __fadd_rn(total[r], __shfl_xor_sync(0xffffffffu, total[r], off));
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const float inv = (total[r] == 0.0f || all_masked[r]) ? 0.0f : __fdiv_rn(1.0f, total[r]);
    const float g = __fmul_rn(inv, p.keep_scale);
    g2[r] = pack2(g, g);
  }
}

// CH = units per lane (row length <= 256*CH).  8 warps per CTA, grid-stride
// over rows, next row's loads in flight while the current row is processed.
template <typename T, int CH, bool DROP, bool EXT>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const SmParams p) {
  const int lane = threadIdx.x & 31;
  const int L = p.L;
  const long long stride = (long long)gridDim.x * 8;
  long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);

  bool valid[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) valid[c] = (lane + 32 * c) * 8 < L;

  Unit<T> cur[CH], nxt[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    if (valid[c]) cur[c].load(in + row * L + (lane + 32 * c) * 8);
    else cur[c].fill_neg_inf();
  }

  for (; row < p.rows; row += stride) {
    const long long next_row = row + stride;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (valid[c] && next_row < p.rows) nxt[c].load(in + next_row * L + (lane + 32 * c) * 8);
      else nxt[c].fill_neg_inf();
    }
    // generated here, where the integer work overlaps the latency of the loads
    // above and of the reductions below
    uint32_t km[CH][4];
    row_keep_masks<CH, DROP>(p, row, lane, km);
    uint64_t e2[CH][4];
    const uint64_t g2 = row_exponentials<T, CH, EXT>(p, cur, row, lane, e2);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      if (valid[c]) {
        const long long off = row * L + (lane + 32 * c) * 8;
        finish_unit_masked<T, DROP>(e2[c], g2, out + off, p.mask + off, km[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) cur[c] = nxt[c];
  }
}

// ----------------------------------------------------- streaming (bulk-copy) kernel
// The dropout-free kernel for large problems: the same per-row arithmetic, fed
// by the copy engine instead of by the warps' own loads.  Rows are dense, so a
// tile of R consecutive rows is one contiguous byte range:
//   * a producer warp streams tiles into a ring of shared-memory stages with
//     cp.async.bulk (completion counted in bytes on an mbarrier);
//   * eight consumer warps take RPW rows each out of a stage, work on them in
//     lockstep, hand the stage back, and write results and mask bytes into
//     their own double-buffered staging area, which leaves through
//     cp.async.bulk stores (one for the values, one for the mask per warp and tile).
// The warps never wait on global memory: several tiles per SM are in flight in
// each direction, whatever the arithmetic is doing.  (With dropout the kernel is
// bound by instruction issue, not by memory: there the warp-per-row kernel,
// which has the fewest instructions per element and the most resident warps, is
// the faster one -- a variant of this kernel with dedicated generator warps
// reached 4.0 TB/s against 5.0 TB/s -- so dropout never takes this path.)
namespace stream {

constexpr int WARPS = 8;            // consumer warps; warp WARPS is the producer
constexpr int THREADS = (WARPS + 1) * 32;
constexpr int STAGES = 3;
enum : int { kWdStreamFull = 301, kWdStreamEmpty = 302 };

template <typename T, int CH> struct Cfg {
  static constexpr int ROW_BYTES_MAX = CH * 256 * (int)sizeof(T);
  // rows per consumer warp and tile: tiles of about 16 KB of input
  static constexpr int RPW = ROW_BYTES_MAX <= 512 ? 4 : ROW_BYTES_MAX <= 1024 ? 2 : 1;
  static constexpr int R = WARPS * RPW;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_wait_read_le1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts16(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts8(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}

template <typename T> __device__ __forceinline__ void unit_from_smem(Unit<T>& u, uint32_t addr);
template <> __device__ __forceinline__ void unit_from_smem<__half>(Unit<__half>& u, uint32_t addr) { u.raw = lds16(addr); }
template <> __device__ __forceinline__ void unit_from_smem<float>(Unit<float>& u, uint32_t addr) {
  u.raw[0] = lds16(addr);
  u.raw[1] = lds16(addr + 16);
}

// One unit of a dropout-free row into the staging area: values, and eight mask bytes of 1.
template <typename T>
__device__ __forceinline__ void finish_unit_smem(const uint64_t (&e2)[4], uint64_t g2, uint32_t out_addr,
                                                 uint32_t mask_addr) {
  sts8(mask_addr, make_uint2(0x01010101u, 0x01010101u));
  float2 y[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) y[k] = unpack2(mul2(e2[k], g2));
  if constexpr (sizeof(T) == 2) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2 h = __floats2half2_rn(y[k].x, y[k].y);
      w[k] = *reinterpret_cast<const uint32_t*>(&h);
    }
    sts16(out_addr, make_uint4(w[0], w[1], w[2], w[3]));
  } else {
    sts16(out_addr, make_uint4(__float_as_uint(y[0].x), __float_as_uint(y[0].y), __float_as_uint(y[1].x),
                               __float_as_uint(y[1].y)));
    sts16(out_addr + 16, make_uint4(__float_as_uint(y[2].x), __float_as_uint(y[2].y), __float_as_uint(y[3].x),
                                    __float_as_uint(y[3].y)));
  }
}

// dynamic shared memory: [STAGES x tile_bytes | WARPS x 2 x (RPW*row_bytes + RPW*L) | barriers | abort flag]
template <typename T, int CH, bool EXT>
__global__ void __launch_bounds__(THREADS) softmax_stream_kernel(const SmParams p, int* status) {
  using C = Cfg<T, CH>;
  constexpr int RPW = C::RPW, R = C::R;
  extern __shared__ __align__(128) uint8_t smem[];
  const int L = p.L;
  const uint32_t row_bytes = (uint32_t)L * (uint32_t)sizeof(T);
  const uint32_t tile_bytes = R * row_bytes;
  const uint32_t wout_bytes = RPW * row_bytes, wmask_bytes = RPW * (uint32_t)L;
  const uint32_t wbuf_bytes = wout_bytes + wmask_bytes;            // one staging buffer of one warp
  const uint32_t s_in = smem_u32(smem);
  const uint32_t s_out = s_in + STAGES * tile_bytes;
  const uint32_t bars = s_out + WARPS * 2 * wbuf_bytes;            // 8-byte aligned: every size is a multiple of 16
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (bars - s_in) + 16 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long num_tiles = (p.rows + R - 1) / R;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == WARPS) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      const char* in = static_cast<const char*>(p.in);
      uint32_t stage = 0, phase = 0;
      for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, status, kWdStreamEmpty)) break;
        const long long row0 = tile * R;
        const long long nrows = min((long long)R, p.rows - row0);
        const uint32_t bytes = (uint32_t)nrows * row_bytes;
        mbar_arrive_expect_tx(full_bar(stage), bytes);
        bulk_load(s_in + stage * tile_bytes, in + row0 * (long long)row_bytes, bytes, full_bar(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // --------------------------------------------------------------- consumers
    bool valid[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) valid[c] = (lane + 32 * c) * 8 < L;
    char* out = static_cast<char*>(p.out);
    const uint32_t my_out = s_out + warp * 2 * wbuf_bytes;
    uint32_t stage = 0, phase = 0, buf = 0;
    for (long long tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const long long row0 = tile * R + warp * RPW;       // first of this warp's rows
      const int nrows = (int)max(0ll, min((long long)RPW, p.rows - row0));
      if (!mbar_wait(full_bar(stage), phase, abort_flag, status, kWdStreamFull)) break;
      Unit<T> cur[RPW][CH];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        const uint32_t base = s_in + stage * tile_bytes + (warp * RPW + r) * row_bytes;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          if (valid[c] && r < nrows) unit_from_smem<T>(cur[r][c], base + (lane + 32 * c) * 8 * (uint32_t)sizeof(T));
          else cur[r][c].fill_neg_inf();
        }
      }
      // the staging buffer about to be written was handed to the copy engine two tiles ago
      if (lane == 0) bulk_wait_read_le1();
      __syncwarp();
      // all RPW rows in lockstep (rows past the end of the tensor are -inf filled and never stored)
      uint64_t e2[RPW][CH][4], g2[RPW];
      long long rws[RPW];
#pragma unroll
      for (int r = 0; r < RPW; ++r) rws[r] = min(row0 + r, p.rows - 1);
      rows_exponentials<T, CH, EXT, RPW>(p, cur, rws, lane, e2, g2);
      // Hand the stage back only now.  The copy engine refills it as soon as the
      // eighth warp has arrived, and an arrive does not wait for shared-memory
      // loads that are still in flight: issued right after the loads it let the
      // refill overtake them (seen with FP32 rows, whose 32-byte lane pitch makes
      // the loads replay).  Here every loaded word has been consumed -- by this
      // lane's arithmetic and, through the reductions, by the whole warp.
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
      if (++stage == STAGES) { stage = 0; phase ^= 1u; }

      const uint32_t ob = my_out + buf * wbuf_bytes, mb = ob + wout_bytes;
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
#pragma unroll
        for (int c = 0; c < CH; ++c)
          if (valid[c])
            finish_unit_smem<T>(e2[r][c], g2[r], ob + r * row_bytes + (lane + 32 * c) * 8 * (uint32_t)sizeof(T),
                                mb + r * L + (lane + 32 * c) * 8);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && nrows > 0) {
        bulk_store(out + row0 * (long long)row_bytes, ob, (uint32_t)nrows * row_bytes);
        bulk_store(p.mask + row0 * (long long)L, mb, (uint32_t)nrows * (uint32_t)L);
        bulk_commit_group();
      }
      buf ^= 1u;
    }
    if (lane == 0) bulk_wait_all();
  }
}

}  // namespace stream

// -------------------------------------------------------- CTA-per-row kernel
// Three passes over the row (the second and third are served by L2).  VEC = 8
// needs 16-byte aligned rows and L % 8 == 0; VEC = 1 takes anything.
template <typename T, int VEC, bool DROP, bool EXT>
__global__ void __launch_bounds__(256) softmax_block_kernel(const SmParams p) {
  constexpr bool HF = sizeof(T) == 2 && !EXT;
  __shared__ float red[32];
  const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = nthr >> 5;
  const int L = p.L;
  const int units = (L + VEC - 1) / VEC;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);

  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = in + row * L;
    const int len = valid_length<EXT>(p, row);
    // pass 1: maximum
    float m = -INFINITY;
    for (int u = tid; u < units; u += nthr) {
      if constexpr (VEC == 8) {
        Unit<T> un; un.load(xr + u * 8);
        float x[8]; un.widen(x);
        adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, x[i]);
      } else {
        m = fmaxf(m, adjust1<EXT>((float)xr[u], u, len, p.scale));
      }
    }
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (int w = 1; w < nwarps; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    const bool all_masked = m == -INFINITY;
    if (all_masked) m = 0.0f;
    const ExpCtx ctx = make_exp_ctx<HF>(m);

    // pass 2: sum of exponentials
    float lane_sum;
    if constexpr (VEC == 8) {
      uint64_t s2 = pack2(0.0f, 0.0f);
      for (int u = tid; u < units; u += nthr) {
        Unit<T> un; un.load(xr + u * 8);
        float x[8]; un.widen(x);
        adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
        for (int k = 0; k < 4; ++k) s2 = add2(s2, exp_pair<HF>(x[2 * k], x[2 * k + 1], ctx));
      }
      const float2 s = unpack2(s2);
      lane_sum = __fadd_rn(s.x, s.y);
    } else {
      float s0 = 0.0f;
      for (int u = tid; u < units; u += nthr) {
        const float xv = adjust1<EXT>((float)xr[u], u, len, p.scale);
        s0 = __fadd_rn(s0, unpack2(exp_pair<HF>(xv, xv, ctx)).x);
      }
      lane_sum = __fadd_rn(s0, 0.0f);
    }
    lane_sum = warp_sum_butterfly(lane_sum);
    if (lane == 0) red[warp] = lane_sum;
    __syncthreads();
    float total = red[0];
    for (int w = 1; w < nwarps; ++w) total = __fadd_rn(total, red[w]);
    __syncthreads();
    const float inv = (total == 0.0f || all_masked) ? 0.0f : __fdiv_rn(1.0f, total);
    const float g = __fmul_rn(inv, p.keep_scale);
    const uint64_t g2 = pack2(g, g);

    // pass 3: normalise, drop, store
    const unsigned long long idx0 = (p.first_row + (unsigned long long)row) * (unsigned long long)L;
    for (int u = tid; u < units; u += nthr) {
      if constexpr (VEC == 8) {
        Unit<T> un; un.load(xr + u * 8);
        float x[8]; un.widen(x);
        adjust8<EXT>(x, u * 8, len, p.scale);
        uint64_t e2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) e2[k] = exp_pair<HF>(x[2 * k], x[2 * k + 1], ctx);
        const long long off = row * L + (long long)u * 8;
        finish_unit<T, DROP>(e2, g2, out + off, p.mask + off, p, (idx0 >> 3) + (unsigned)u);
      } else {
        const float xv = adjust1<EXT>((float)xr[u], u, len, p.scale);
        const float e = unpack2(exp_pair<HF>(xv, xv, ctx)).x;
        float y = __fmul_rn(e, g);
        unsigned keep = 1u;
        if (DROP) {
          const unsigned long long idx = idx0 + (unsigned)u;
          uint32_t o[4];
          philox_block((uint32_t)(idx >> 3), (uint32_t)(idx >> 35), p.key, o);
          const uint32_t el = (uint32_t)(idx & 7ull);
          const uint32_t word = (el >> 1) == 0 ? o[0] : (el >> 1) == 1 ? o[1] : (el >> 1) == 2 ? o[2] : o[3];
          keep = ((word >> (16u * (el & 1u))) & 0x7FFFu) >= p.thr;
          if (!keep) y = 0.0f;
        }
        p.mask[row * L + u] = (unsigned char)keep;
        if constexpr (sizeof(T) == 2) out[row * L + u] = __float2half_rn(y);
        else out[row * L + u] = y;
      }
    }
  }
}

// ------------------------------------------- long rows: shared-memory resident
// One CTA of 8 warps per row.  The row (contiguous in memory) is brought into
// shared memory once by the copy engine (cp.async.bulk, completion counted on an
// mbarrier); the three sweeps -- maximum, sum of exponentials, normalise / drop /
// store -- then read shared memory, so the row crosses HBM once in each
// direction.  With two row buffers the next row of the CTA is in flight while the
// current one is processed.  Unit u belongs to thread u % 256 and every sum
// follows the order of softmax_block_kernel<T, 8, ...>, so the two kernels
// produce the same bits (the CPU restatement of that schedule covers both).
namespace longrow {

constexpr int THREADS = 256;
enum : int { kWdRowFull = 311 };

// UPT > 0: rows of at most UPT * 2048 elements; a thread's units are read from
// shared memory once and stay in registers through the three steps, and every
// exponential is computed once.  UPT = 0: any length, three sweeps over shared
// memory.  Same order of operations either way.
template <typename T, int UPT, bool DROP, bool EXT>
__global__ void __launch_bounds__(THREADS) softmax_smem_row_kernel(const SmParams p, int nbuf, int* status) {
  constexpr bool HF = sizeof(T) == 2 && !EXT;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[8];
  __shared__ __align__(8) uint64_t bar_store[2];
  __shared__ int abort_word;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = p.L;
  const int units = L / 8;
  const uint32_t row_bytes = (uint32_t)L * (uint32_t)sizeof(T);
  const uint32_t buf_bytes = (row_bytes + 127u) & ~127u;
  const uint32_t s_rows = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bar_store);
  volatile int* abort_flag = &abort_word;
  const char* in = static_cast<const char*>(p.in);
  T* out = static_cast<T*>(p.out);

  if (tid == 0) {
    for (int b = 0; b < nbuf; ++b) mbar_init(bar0 + 8u * b, 1);
    abort_word = 0;
    mbar_fence_init();
    // prologue: the first nbuf rows of this CTA
    for (int b = 0; b < nbuf; ++b) {
      const long long r = (long long)blockIdx.x + (long long)b * gridDim.x;
      if (r < p.rows) {
        mbar_arrive_expect_tx(bar0 + 8u * b, row_bytes);
        stream::bulk_load(s_rows + b * buf_bytes, in + r * (long long)row_bytes, row_bytes, bar0 + 8u * b);
      }
    }
  }
  __syncthreads();

  uint32_t it = 0;
  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x, ++it) {
    const uint32_t b = it % (uint32_t)nbuf, parity = (it / (uint32_t)nbuf) & 1u;
    const uint32_t xs = s_rows + b * buf_bytes;
    const int len = valid_length<EXT>(p, row);

    if constexpr (UPT > 0) {
      // ---- register-resident form
      // dropout decisions of this thread's units, four Philox blocks at a time: they
      // depend on the row number only, so they are drawn while the row is still on its way
      uint32_t km[UPT][4];
      {
        const unsigned long long blk0 = ((p.first_row + (unsigned long long)row) * (unsigned long long)L) >> 3;
        constexpr int NB = UPT < 4 ? UPT : 4;
#pragma unroll
        for (int j0 = 0; j0 < UPT; j0 += NB) {
          if (DROP) {
            unsigned long long blk[NB];
            uint32_t o[NB][4];
#pragma unroll
            for (int q = 0; q < NB; ++q) blk[q] = blk0 + (unsigned)(tid + (j0 + q) * THREADS);
            philox_blocks<NB>(blk, p.key, o);
#pragma unroll
            for (int q = 0; q < NB; ++q) masks_from_words<true>(p, o[q], km[j0 + q]);
          } else {
#pragma unroll
            for (int q = 0; q < NB; ++q) masks_from_words<false>(p, km[j0 + q], km[j0 + q]);
          }
        }
      }
      if (!mbar_wait(bar0 + 8u * b, parity, abort_flag, status, kWdRowFull)) break;
      Unit<T> un[UPT];
      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < UPT; ++j) {
        const int u = tid + j * THREADS;
        if (u < units) {
          stream::unit_from_smem<T>(un[j], xs + (uint32_t)u * 8u * (uint32_t)sizeof(T));
          float x[8]; un[j].widen(x);
          adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
          for (int i = 0; i < 8; ++i) m = fmaxf(m, x[i]);
        }
      }
      __syncthreads();                        // every thread holds its part of the row: the buffer is free
      if (tid == 0) {
        const long long nr = row + (long long)nbuf * gridDim.x;
        if (nr < p.rows) {
          mbar_arrive_expect_tx(bar0 + 8u * b, row_bytes);
          stream::bulk_load(xs, in + nr * (long long)row_bytes, row_bytes, bar0 + 8u * b);
        }
      }
      m = warp_max(m);
      if (lane == 0) red[warp] = m;
      __syncthreads();
      m = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
      __syncthreads();
      const bool all_masked = m == -INFINITY;
      if (all_masked) m = 0.0f;
      const ExpCtx ctx = make_exp_ctx<HF>(m);
      uint64_t e2[UPT][4];
      uint64_t s2 = pack2(0.0f, 0.0f);
#pragma unroll
      for (int j = 0; j < UPT; ++j) {
        const int u = tid + j * THREADS;
        if (u < units) {
          float x[8]; un[j].widen(x);
          adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            e2[j][k] = exp_pair<HF>(x[2 * k], x[2 * k + 1], ctx);
            s2 = add2(s2, e2[j][k]);
          }
        }
      }
      const float2 sp = unpack2(s2);
      const float lane_sum = warp_sum_butterfly(__fadd_rn(sp.x, sp.y));
      if (lane == 0) red[warp] = lane_sum;
      __syncthreads();
      float total = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) total = __fadd_rn(total, red[w]);
      __syncthreads();                        // red[] is reused by the next row
      const float inv = (total == 0.0f || all_masked) ? 0.0f : __fdiv_rn(1.0f, total);
      const float g = __fmul_rn(inv, p.keep_scale);
      const uint64_t g2 = pack2(g, g);
#pragma unroll
      for (int j = 0; j < UPT; ++j) {
        const int u = tid + j * THREADS;
        if (u < units) {
          const long long off = row * L + (long long)u * 8;
          finish_unit_masked<T, DROP>(e2[j], g2, out + off, p.mask + off, km[j]);
        }
      }
      continue;
    }

    // ---- three sweeps over shared memory
    if (!mbar_wait(bar0 + 8u * b, parity, abort_flag, status, kWdRowFull)) break;
    // sweep 1: maximum
    float m = -INFINITY;
    for (int u = tid; u < units; u += THREADS) {
      Unit<T> un; stream::unit_from_smem<T>(un, xs + (uint32_t)u * 8u * (uint32_t)sizeof(T));
      float x[8]; un.widen(x);
      adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, x[i]);
    }
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    const bool all_masked = m == -INFINITY;
    if (all_masked) m = 0.0f;
    const ExpCtx ctx = make_exp_ctx<HF>(m);

    // sweep 2: sum of exponentials
    uint64_t s2 = pack2(0.0f, 0.0f);
    for (int u = tid; u < units; u += THREADS) {
      Unit<T> un; stream::unit_from_smem<T>(un, xs + (uint32_t)u * 8u * (uint32_t)sizeof(T));
      float x[8]; un.widen(x);
      adjust8<EXT>(x, u * 8, len, p.scale);
#pragma unroll
      for (int k = 0; k < 4; ++k) s2 = add2(s2, exp_pair<HF>(x[2 * k], x[2 * k + 1], ctx));
    }
    const float2 sp = unpack2(s2);
    float lane_sum = warp_sum_butterfly(__fadd_rn(sp.x, sp.y));
    if (lane == 0) red[warp] = lane_sum;
    __syncthreads();
    float total = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total = __fadd_rn(total, red[w]);
    const float inv = (total == 0.0f || all_masked) ? 0.0f : __fdiv_rn(1.0f, total);
    const float g = __fmul_rn(inv, p.keep_scale);
    const uint64_t g2 = pack2(g, g);

    // sweep 3: normalise, drop, store
    const unsigned long long idx0 = (p.first_row + (unsigned long long)row) * (unsigned long long)L;
    for (int u = tid; u < units; u += THREADS) {
      Unit<T> un; stream::unit_from_smem<T>(un, xs + (uint32_t)u * 8u * (uint32_t)sizeof(T));
      float x[8]; un.widen(x);
      adjust8<EXT>(x, u * 8, len, p.scale);
      uint64_t e2[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) e2[k] = exp_pair<HF>(x[2 * k], x[2 * k + 1], ctx);
      const long long off = row * L + (long long)u * 8;
      finish_unit<T, DROP>(e2, g2, out + off, p.mask + off, p, (idx0 >> 3) + (unsigned)u);
    }
    __syncthreads();     // every thread is done with this buffer (and with red[])
    if (tid == 0) {
      const long long nr = row + (long long)nbuf * gridDim.x;
      if (nr < p.rows) {
        mbar_arrive_expect_tx(bar0 + 8u * b, row_bytes);
        stream::bulk_load(xs, in + nr * (long long)row_bytes, row_bytes, bar0 + 8u * b);
      }
    }
  }
}

// --------------------------------------------- long rows: online single pass
// Rows too long for shared memory.  Sweep 1 reads the row once and keeps, per
// thread, a running maximum m_t and a sum of exponentials relative to it,
// rescaled by 2^((m_old - m_new) log2 e) whenever a unit raises the maximum
// (a unit whose elements are all -inf is skipped).  The threads' pairs (m_t, s_t)
// are then brought to the row maximum and added in the fixed order (xor
// butterfly per warp, warps ascending).  Sweep 2 reads the row again to write
// e_j * g.  FP32-storage arithmetic for both storage types.
template <typename T, bool DROP, bool EXT>
__global__ void __launch_bounds__(THREADS) softmax_online_kernel(const SmParams p) {
  __shared__ float red[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int L = p.L;
  const int units = L / 8;
  const T* in = static_cast<const T*>(p.in);
  T* out = static_cast<T*>(p.out);
  const uint64_t log2e2 = pack2(kLog2e, kLog2e);

  for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = in + row * L;
    const int len = valid_length<EXT>(p, row);
    float mt = -INFINITY;
    uint64_t s2 = pack2(0.0f, 0.0f);
    uint64_t negc2 = pack2(0.0f, 0.0f);
    // four units per thread and step: the loads are issued together, the units are
    // then taken in ascending order (the order of the CPU restatement)
    for (int u0 = tid; u0 < units; u0 += 4 * THREADS) {
      Unit<T> un[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (u0 + j * THREADS < units) un[j].load_keep(xr + (size_t)(u0 + j * THREADS) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int u = u0 + j * THREADS;
        if (u >= units) break;
        float x[8]; un[j].widen(x);
        adjust8<EXT>(x, u * 8, len, p.scale);
        float mu = x[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mu = fmaxf(mu, x[i]);
        if (mu == -INFINITY) continue;                 // contributes nothing
        if (mu > mt) {
          const float negc = -__fmul_rn(mu, kLog2e);
          if (mt != -INFINITY) {
            const float t = fmaxf(__fmaf_rn(mt, kLog2e, negc), -127.0f);
            const float2 f = unpack2(exp2_pair(pack2(t, t)));
            s2 = mul2(s2, pack2(f.x, f.x));
          }
          mt = mu;
          negc2 = pack2(negc, negc);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 t = unpack2(fma2(pack2(x[2 * k], x[2 * k + 1]), log2e2, negc2));
          s2 = add2(s2, exp2_pair(pack2(fmaxf(t.x, -127.0f), fmaxf(t.y, -127.0f))));
        }
      }
    }
    // row maximum
    float m = warp_max(mt);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    const bool all_masked = m == -INFINITY;
    if (all_masked) m = 0.0f;
    const float negc = -__fmul_rn(m, kLog2e);
    // this thread's sum relative to the row maximum
    const float2 sp = unpack2(s2);
    float st = __fadd_rn(sp.x, sp.y);
    if (mt == -INFINITY) st = 0.0f;
    else {
      const float t = fmaxf(__fmaf_rn(mt, kLog2e, negc), -127.0f);
      st = __fmul_rn(st, unpack2(exp2_pair(pack2(t, t))).x);
    }
    st = warp_sum_butterfly(st);
    if (lane == 0) red[warp] = st;
    __syncthreads();
    float total = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) total = __fadd_rn(total, red[w]);
    __syncthreads();
    const float inv = (total == 0.0f || all_masked) ? 0.0f : __fdiv_rn(1.0f, total);
    const float g = __fmul_rn(inv, p.keep_scale);
    const uint64_t g2 = pack2(g, g);
    const uint64_t rowc2 = pack2(negc, negc);

    const unsigned long long idx0 = (p.first_row + (unsigned long long)row) * (unsigned long long)L;
    for (int u0 = tid; u0 < units; u0 += 4 * THREADS) {
      Unit<T> un[4];
      uint32_t km[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (u0 + j * THREADS < units) un[j].load(xr + (size_t)(u0 + j * THREADS) * 8);
      if (DROP) {
        unsigned long long blk[4];
        uint32_t o[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) blk[j] = (idx0 >> 3) + (unsigned)(u0 + j * THREADS);
        philox_blocks<4>(blk, p.key, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) masks_from_words<true>(p, o[j], km[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) masks_from_words<false>(p, km[j], km[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int u = u0 + j * THREADS;
        if (u >= units) break;
        float x[8]; un[j].widen(x);
        adjust8<EXT>(x, u * 8, len, p.scale);
        uint64_t e2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 t = unpack2(fma2(pack2(x[2 * k], x[2 * k + 1]), log2e2, rowc2));
          e2[k] = exp2_pair(pack2(fmaxf(t.x, -127.0f), fmaxf(t.y, -127.0f)));
        }
        const long long off = row * L + (long long)u * 8;
        finish_unit_masked<T, DROP>(e2, g2, out + off, p.mask + off, km[j]);
      }
    }
  }
}

}  // namespace longrow

// Largest row that the shared-memory resident kernel takes (one buffer).
constexpr size_t kSmemRowLimit = 200 * 1024;

template <typename T, bool DROP, bool EXT>
void launch_smem_row_t(const SmParams& p, int sms, cudaStream_t stream) {
  const size_t row_bytes = (size_t)p.L * sizeof(T);
  const size_t buf = (row_bytes + 127) & ~(size_t)127;
  const int nbuf = 2 * buf <= 100 * 1024 ? 2 : 1;
  const size_t smem = nbuf * buf;
  const int units_per_thread = (p.L / 8 + longrow::THREADS - 1) / longrow::THREADS;
  void (*kern)(const SmParams, int, int*) =
      units_per_thread <= 2   ? longrow::softmax_smem_row_kernel<T, 2, DROP, EXT>
      : units_per_thread <= 4 ? longrow::softmax_smem_row_kernel<T, 4, DROP, EXT>
      : units_per_thread <= 8 ? longrow::softmax_smem_row_kernel<T, 8, DROP, EXT>
                              : longrow::softmax_smem_row_kernel<T, 0, DROP, EXT>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, longrow::THREADS, smem);
  if (per_sm < 1) per_sm = 1;
  const long long cap = (long long)sms * per_sm;
  const int grid = (int)(p.rows < cap ? p.rows : cap);
  kern<<<grid, longrow::THREADS, smem, stream>>>(p, nbuf, watchdog_word());
}
template <typename T, bool DROP, bool EXT>
void launch_online_t(const SmParams& p, int sms, cudaStream_t stream) {
  const long long cap = (long long)sms * 8;
  const int grid = (int)(p.rows < cap ? p.rows : cap);
  longrow::softmax_online_kernel<T, DROP, EXT><<<grid, longrow::THREADS, 0, stream>>>(p);
}
template <typename T>
void launch_long(const SmParams& p, bool drop, bool ext, bool online, int sms, cudaStream_t stream) {
#define TFB_LONG(DROP, EXT)                                              \
  do {                                                                   \
    if (online) launch_online_t<T, DROP, EXT>(p, sms, stream);           \
    else launch_smem_row_t<T, DROP, EXT>(p, sms, stream);                \
  } while (0)
  if (ext) { if (drop) TFB_LONG(true, true); else TFB_LONG(false, true); }
  else { if (drop) TFB_LONG(true, false); else TFB_LONG(false, false); }
#undef TFB_LONG
}

template <typename T, int CH, bool DROP, bool EXT>
void launch_warp_t(const SmParams& p, int sms, cudaStream_t stream) {
  const long long ctas_needed = (p.rows + 7) / 8;
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, softmax_warp_kernel<T, CH, DROP, EXT>, 256, 0);
  if (per_sm < 1) per_sm = 1;
  const long long cap = (long long)sms * per_sm;
  const int grid = (int)(ctas_needed < cap ? ctas_needed : cap);
  softmax_warp_kernel<T, CH, DROP, EXT><<<grid, 256, 0, stream>>>(p);
}
template <typename T, int CH>
void launch_warp(const SmParams& p, bool drop, bool ext, int sms, cudaStream_t stream) {
  if (ext) {
    if (drop) launch_warp_t<T, CH, true, true>(p, sms, stream);
    else launch_warp_t<T, CH, false, true>(p, sms, stream);
  } else {
    if (drop) launch_warp_t<T, CH, true, false>(p, sms, stream);
    else launch_warp_t<T, CH, false, false>(p, sms, stream);
  }
}

// Streaming kernel (dropout-free only): needs whole 16-byte mask rows (L % 16 == 0,
// 16-byte aligned mask pointer) and rows of at most 4 KB.
template <typename T, int CH, bool EXT>
void launch_stream_t(const SmParams& p, int sms, cudaStream_t stream) {
  using C = stream::Cfg<T, CH>;
  const size_t row_bytes = (size_t)p.L * sizeof(T);
  const size_t smem = stream::STAGES * C::R * row_bytes + (size_t)stream::WARPS * 2 * C::RPW * (row_bytes + p.L) +
                      16 * stream::STAGES + 16;
  auto kern = stream::softmax_stream_kernel<T, CH, EXT>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int per_sm = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, stream::THREADS, smem);
  if (per_sm < 1) per_sm = 1;
  const long long tiles = (p.rows + C::R - 1) / C::R;
  const long long cap = (long long)sms * per_sm;
  const int grid = (int)(tiles < cap ? tiles : cap);
  kern<<<grid, stream::THREADS, smem, stream>>>(p, watchdog_word());
}
template <typename T, int CH>
void launch_stream(const SmParams& p, bool ext, int sms, cudaStream_t stream) {
  if (ext) launch_stream_t<T, CH, true>(p, sms, stream);
  else launch_stream_t<T, CH, false>(p, sms, stream);
}

// 0 = choose by shape, 1 = warp kernel only, 2 = streaming kernel wherever it is eligible.
// TENSORFUSE_B200_SOFTMAX_FORM=warp|stream, read once; meant for measurements and tests.
int softmax_form_override() {
  static const int form = [] {
    const char* e = getenv("TENSORFUSE_B200_SOFTMAX_FORM");
    if (e == nullptr) return 0;
    if (strcmp(e, "warp") == 0) return 1;
    if (strcmp(e, "stream") == 0) return 2;
    return 0;
  }();
  return form;
}

template <typename T>
bool stream_eligible(const SmParams& p, bool drop) {
  if (drop) return false;    // bound by instruction issue: the warp-per-row kernel is faster there
  if (p.L % 16 != 0 || ((uintptr_t)p.mask & 15u) != 0) return false;
  if ((size_t)p.L * sizeof(T) > 4096) return false;
  const int form = softmax_form_override();
  if (form == 1) return false;
  if (form == 2) return true;
  return p.rows >= 4096;     // small problems: the plain kernel has less set-up
}

template <typename T, int VEC>
void launch_block(const SmParams& p, bool drop, bool ext, int warps, int sms, cudaStream_t stream) {
  const long long cap = (long long)sms * (warps == 1 ? 32 : 8);
  const int grid = (int)(p.rows < cap ? p.rows : cap);
  if (ext) {
    if (drop) softmax_block_kernel<T, VEC, true, true><<<grid, 32 * warps, 0, stream>>>(p);
    else softmax_block_kernel<T, VEC, false, true><<<grid, 32 * warps, 0, stream>>>(p);
  } else {
    if (drop) softmax_block_kernel<T, VEC, true, false><<<grid, 32 * warps, 0, stream>>>(p);
    else softmax_block_kernel<T, VEC, false, false><<<grid, 32 * warps, 0, stream>>>(p);
  }
}

template <typename T>
void dispatch(const SmParams& p, bool drop, bool ext, SoftmaxSchedule sch, int sms, cudaStream_t stream) {
  if (sch.vec == 8 && sch.warps == 1 && stream_eligible<T>(p, drop)) {
    if (p.L <= 256) launch_stream<T, 1>(p, ext, sms, stream);
    else if (p.L <= 512) launch_stream<T, 2>(p, ext, sms, stream);
    else if (p.L <= 1024) launch_stream<T, 4>(p, ext, sms, stream);
    else launch_stream<T, 8>(p, ext, sms, stream);
  } else if (sch.vec == 8 && sch.warps == 1) {
    if (p.L <= 256) launch_warp<T, 1>(p, drop, ext, sms, stream);
    else if (p.L <= 512) launch_warp<T, 2>(p, drop, ext, sms, stream);
    else if (p.L <= 1024) launch_warp<T, 4>(p, drop, ext, sms, stream);
    else launch_warp<T, 8>(p, drop, ext, sms, stream);
  } else if (sch.vec == 8 && sch.warps == 8 && softmax_form_override() != 1) {
    launch_long<T>(p, drop, ext, sch.online != 0, sms, stream);
  } else if (sch.vec == 8) {
    launch_block<T, 8>(p, drop, ext, sch.warps, sms, stream);
  } else {
    launch_block<T, 1>(p, drop, ext, sch.warps, sms, stream);
  }
}

int sm_count_of_current_device() {
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

}  // namespace

SoftmaxSchedule softmax_schedule(int L, int dtype, bool aligned16) {
  SoftmaxSchedule s;
  s.online = 0;
  if (aligned16 && L % 8 == 0) {
    s.vec = 8;
    s.warps = L <= 2048 ? 1 : 8;
    // rows beyond the shared-memory resident kernel: one online sweep + one write sweep
    if ((size_t)L * (dtype == kF16 ? 2 : 4) > kSmemRowLimit) s.online = 1;
  } else {
    s.vec = 1;
    s.warps = L <= 1024 ? 1 : 8;
  }
  return s;
}

LaunchResult launch_softmax_dropout(const void* in, void* out, unsigned char* mask,
                                    long long rows, int L, int dtype, float p,
                                    unsigned long long seed, unsigned long long first_row,
                                    cudaStream_t stream) {
  return launch_softmax_dropout_ext(in, out, mask, rows, L, dtype, p, seed, first_row, 1.0f, nullptr, 0, false, stream);
}

LaunchResult launch_softmax_dropout_ext(const void* in, void* out, unsigned char* mask, long long rows, int L,
                                        int dtype, float p, unsigned long long seed, unsigned long long first_row,
                                        float scale, const int* lengths, long long rows_per_item, bool extended,
                                        cudaStream_t stream) {
  if (!in || !out || !mask) return kInvalidArgument;
  if (extended && (!(scale > 0.0f) || (lengths != nullptr && rows_per_item <= 0))) return kInvalidArgument;
  if (!(p >= 0.0f && p <= 1.0f)) return kInvalidArgument;
  if (dtype != kF16 && dtype != kF32) return kUnsupported;
  if (rows < 0 || L < 0) return kInvalidArgument;
  if (rows == 0 || L == 0) return kOk;

  SmParams sp;
  sp.in = in; sp.out = out; sp.mask = mask; sp.rows = rows; sp.L = L;
  sp.keep_scale = p >= 1.0f ? 0.0f : 1.0f / (1.0f - p);
  sp.thr = dropout_threshold(p);
  sp.thr_h2 = (sp.thr & 0xFFFFu) * 0x00010001u;
  sp.hcmp = sp.thr <= 0x7C00u ? 1 : 0;
  sp.first_row = first_row;
  philox_round_keys(seed, sp.key);
  sp.scale = scale; sp.lengths = lengths; sp.rows_per_item = rows_per_item > 0 ? rows_per_item : 1;
  const bool drop = sp.thr != 0u;
  const uintptr_t bits = (uintptr_t)in | (uintptr_t)out | ((uintptr_t)mask << 1);
  const bool aligned16 = (bits & 15u) == 0;
  const SoftmaxSchedule sch = softmax_schedule(L, dtype, aligned16);
  const int sms = sm_count_of_current_device();
  if (dtype == kF16) dispatch<__half>(sp, drop, extended, sch, sms, stream);
  else dispatch<float>(sp, drop, extended, sch, sms, stream);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace tfb
