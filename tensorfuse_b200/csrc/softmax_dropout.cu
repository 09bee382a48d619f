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
// Dropout uses Philox4x32-10: eight consecutive elements share one block
// (counter = global element index / 8, key = seed), each element takes a 16-bit
// field and is kept when its low 15 bits are >= round(p * 32768).  The counter depends only on
// the element's position in the whole tensor, so any row-sharding across GPUs
// reproduces the same mask.
#include <cuda_fp16.h>
#include <math.h>

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

// CH = units per lane (row length <= 256*CH).  8 warps per CTA, grid-stride
// over rows, next row's loads in flight while the current row is processed.
// FP16 storage keeps the row packed for as long as possible: the maximum and
// the clamp at lo are taken on half2 words, the widening to FP32 happens once.
template <typename T, int CH, bool DROP, bool EXT>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const SmParams p) {
  constexpr bool HF = sizeof(T) == 2 && !EXT;
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

    // Dropout decisions of this lane's units.  They depend on positions only, so they are
    // generated here, up to four Philox blocks with interleaved rounds, where their integer
    // work overlaps the latency of the loads above and the reductions below.
    uint32_t km[CH][4];
    {
      const unsigned long long blk0 = ((p.first_row + (unsigned long long)row) * (unsigned long long)L) >> 3;
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

    uint64_t e2[CH][4];
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
    const uint64_t g2 = pack2(g, g);

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
  if (sch.vec == 8 && sch.warps == 1) {
    if (p.L <= 256) launch_warp<T, 1>(p, drop, ext, sms, stream);
    else if (p.L <= 512) launch_warp<T, 2>(p, drop, ext, sms, stream);
    else if (p.L <= 1024) launch_warp<T, 4>(p, drop, ext, sms, stream);
    else launch_warp<T, 8>(p, drop, ext, sms, stream);
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
  (void)dtype;
  SoftmaxSchedule s;
  if (aligned16 && L % 8 == 0) {
    s.vec = 8;
    s.warps = L <= 2048 ? 1 : 8;
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
