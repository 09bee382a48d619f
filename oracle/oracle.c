/* oracle.c -- CPU restatement of the two TensorFuse hot paths.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this file; it exists so that the tests, the smoke check and the
 * CPU-baseline leg of the benchmark have an independent statement of what the
 * CUDA kernels must compute.
 *
 * Provenance of each function (paths are inside the reference project):
 *   tfo_gelu_f32                 gelu_ref,            src/tests/test_kernels.cu:43-47
 *   tfo_gemm_bias_gelu_f32       gemm_bias_gelu_ref,  src/tests/test_kernels.cu:50-64
 *   tfo_gemm_bias_gelu_f16       same loop on FP16 storage: FP32 accumulate, one rounding
 *                                to FP16 at the end (the data flow of
 *                                src/kernels/fused_gemm_bias_gelu_optimized.cu:24-55,115-169
 *                                without its intermediate FP16 rounding)
 *   tfo_gemm_i8_acc / _epilogue  INT32 accumulation and the two dequant conventions:
 *                                legacy = apply_scaled_gelu_kernel,
 *                                src/kernels/fused_gemm_bias_gelu_int8.cu:51-99
 *   tfo_softmax_ref_f32          softmax_ref,         src/tests/test_softmax_dropout.cu:36-64
 *   tfo_dropout semantics        keep = u > p, scale 1/(1-p): src/tests/test_softmax_dropout.cu:66-79
 *                                and src/kernels/fused_softmax_dropout.cu:213-231
 *   tfo_softmax_dropout_exact    same mathematics with the exponential, the summation
 *                                order and the random stream written out operation by
 *                                operation, so that an implementation which performs the
 *                                same IEEE operations in the same order reproduces it bit
 *                                for bit.  The reference's own GPU kernel uses fast-math
 *                                __expf and XORWOW and is not reproducible on a CPU; this
 *                                function is the reproducible statement of the same math.
 *
 * Parity status: pinned.  The GELU/GEMM/softmax functions are held to the
 * known-answer values of the reference's C++ tests, to the fixtures under
 * tests/golden/ produced by importing the reference's own numpy oracle, and to
 * outputs of the reference's own GPU kernels (its library compiled for sm_100a
 * and run on a B200: tests/golden/reference_gpu_kernels.npz, FP32, FP16 and INT8
 * GEMM and both softmax types).  The FP16 and INT8 GEMM paths have no numeric
 * pin in the reference's own tests ("parity unpinned" upstream); those GPU
 * outputs and the FP32 loop they share are what pins them here.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 half_t;

static inline float h2f(uint16_t h) { half_t v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f2h(float f) { half_t v = (half_t)f; uint16_t h; memcpy(&h, &v, 2); return h; }

static void set_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
}

int tfo_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------ GELU */

float tfo_gelu_f32(float x) {
  const float a = 0.7978845608028654f; /* sqrt(2/pi) */
  const float b = 0.044715f;
  return x * 0.5f * (1.0f + tanhf(a * (x + b * x * x * x)));
}

void tfo_gelu_f32_array(const float* x, float* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = tfo_gelu_f32(x[i]);
}

/* Legacy INT8 activation: tanh argument clamped to [-10, 10]. */
static inline float gelu_clamped(float v) {
  const float a = 0.7978845608028654f, b = 0.044715f;
  float arg = a * (v + b * v * v * v);
  arg = fmaxf(-10.0f, fminf(10.0f, arg));
  return v * 0.5f * (1.0f + tanhf(arg));
}

/* ------------------------------------------------- FP32 GEMM + bias + GELU
 * C[m,n] = gelu(alpha * sum_k A[m,k]*B[k,n] + beta*bias[n]); the sum runs over
 * k = 0..K-1 in order with one FP32 multiply and one FP32 add per term.  The
 * loops are ordered m,k,n so the compiler can vectorise over n; every C[m,n]
 * still sees its K terms in ascending k, so results equal the m,n,k loop. */
void tfo_gemm_bias_gelu_f32(const float* A, const float* B, const float* bias, float* C,
                            int M, int N, int K, float alpha, float beta, int threads) {
  set_threads(threads);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* acc = C + (size_t)m * N;
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const float a = A[(size_t)m * K + k];
      const float* b = B + (size_t)k * N;
      for (int n = 0; n < N; ++n) acc[n] += a * b[n];
    }
    for (int n = 0; n < N; ++n) acc[n] = tfo_gelu_f32(alpha * acc[n] + beta * bias[n]);
  }
}

/* FP16 storage, FP32 arithmetic, one rounding to FP16 at the end. */
void tfo_gemm_bias_gelu_f16(const uint16_t* A, const uint16_t* B, const uint16_t* bias,
                            uint16_t* C, int M, int N, int K, float alpha, float beta,
                            int threads) {
  set_threads(threads);
  float* Bf = (float*)malloc(sizeof(float) * (size_t)K * N);
  for (size_t i = 0; i < (size_t)K * N; ++i) Bf[i] = h2f(B[i]);
#pragma omp parallel
  {
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      for (int n = 0; n < N; ++n) acc[n] = 0.0f;
      for (int k = 0; k < K; ++k) {
        const float a = h2f(A[(size_t)m * K + k]);
        const float* b = Bf + (size_t)k * N;
        for (int n = 0; n < N; ++n) acc[n] += a * b[n];
      }
      for (int n = 0; n < N; ++n)
        C[(size_t)m * N + n] = f2h(tfo_gelu_f32(alpha * acc[n] + beta * h2f(bias[n])));
    }
    free(acc);
  }
  free(Bf);
}

/* ------------------------------------------------------------ INT8 GEMM */

void tfo_gemm_i8_acc(const int8_t* A, const int8_t* B, int32_t* acc, int M, int N, int K,
                     int threads) {
  set_threads(threads);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    int32_t* row = acc + (size_t)m * N;
    for (int n = 0; n < N; ++n) row[n] = 0;
    for (int k = 0; k < K; ++k) {
      const int32_t a = A[(size_t)m * K + k];
      const int8_t* b = B + (size_t)k * N;
      for (int n = 0; n < N; ++n) row[n] += a * (int32_t)b[n];
    }
  }
}

/* Dequant-by-multiply convention: scale = max|x|/127 per tensor,
 * out = half(gelu(fma(float(acc), sA*sB, float(bias)))) with FP16 bias/output. */
void tfo_i8_epilogue_f16(const int32_t* acc, const uint16_t* bias, uint16_t* C, long M, int N,
                         float scale_a, float scale_b) {
  const float s = scale_a * scale_b;
  for (long m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float x = fmaf((float)acc[m * N + n], s, h2f(bias[n]));
      C[m * N + n] = f2h(tfo_gelu_f32(x));
    }
}

/* Legacy convention of the reference kernel: scale = 127/max|x|,
 * out = gelu_clamped(acc/(sA*sB) + bias) * (sA*sB), non-finite -> 0, FP32. */
void tfo_i8_epilogue_legacy_f32(const int32_t* acc, const float* bias, float* C, long M, int N,
                                float scale_a, float scale_b) {
  const float s = scale_a * scale_b;
  for (long m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float raw = (float)acc[m * N + n];
      float v = raw / s + bias[n];
      float r = gelu_clamped(v) * s;
      C[m * N + n] = isfinite(r) ? r : 0.0f;
    }
}

/* ----------------------------------------------------- softmax, reference */

void tfo_softmax_ref_f32(const float* in, float* out, long rows, int L, int threads) {
  set_threads(threads);
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) {
    const float* x = in + r * L;
    float* y = out + r * L;
    float mx = -INFINITY;
    for (int j = 0; j < L; ++j) mx = fmaxf(mx, x[j]);
    float sum = 0.0f;
    for (int j = 0; j < L; ++j) { float e = expf(x[j] - mx); y[j] = e; sum += e; }
    for (int j = 0; j < L; ++j) y[j] /= sum;
  }
}

/* FP16 storage twin used as the timed CPU baseline of the FP16 attention shape:
 * same three passes, FP32 arithmetic, mask written as all-ones (p = 0). */
void tfo_softmax_ref_f16(const uint16_t* in, uint16_t* out, uint8_t* mask, long rows, int L,
                         int threads) {
  set_threads(threads);
#pragma omp parallel
  {
    float* y = (float*)malloc(sizeof(float) * (size_t)L);
#pragma omp for schedule(static)
    for (long r = 0; r < rows; ++r) {
      const uint16_t* x = in + r * L;
      float mx = -INFINITY;
      for (int j = 0; j < L; ++j) mx = fmaxf(mx, h2f(x[j]));
      float sum = 0.0f;
      for (int j = 0; j < L; ++j) { float e = expf(h2f(x[j]) - mx); y[j] = e; sum += e; }
      for (int j = 0; j < L; ++j) { out[r * L + j] = f2h(y[j] / sum); mask[r * L + j] = 1; }
    }
    free(y);
  }
}

/* ---------------------------------------------------------------- Philox
 * Philox4x32 (Salmon et al., SC'11) with a selectable number of rounds, multipliers 0xD2511F53 /
 * 0xCD9E8D57, Weyl key increments 0x9E3779B9 / 0xBB67AE85. */
void tfo_philox4x32_r(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                      uint32_t k1, int rounds, uint32_t out[4]) {
  for (int r = 0; r < rounds; ++r) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
/* The 10-round generator of the Random123 distribution (known-answer vectors). */
void tfo_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                       uint32_t k1, uint32_t out[4]) {
  tfo_philox4x32_r(c0, c1, c2, c3, k0, k1, 10, out);
}
/* Rounds of the library's dropout stream: 7, the fewest rounds for which the
 * Philox paper reports a clean BigCrush (tensorfuse_b200/csrc/philox.cuh). */
#define TFO_DROPOUT_ROUNDS 7

/* Dropout decision for the element with global flat index idx: eight
 * consecutive elements share one Philox block (counter = idx/8, key = seed);
 * element e = idx%8 takes the 16-bit field e%2 of word e/2 and is kept when
 * the low 15 bits of that field are >= thr, thr = round(p * 32768). */
uint32_t tfo_dropout_threshold(float p) {
  if (!(p > 0.0f)) return 0u;
  if (p >= 1.0f) return 32768u;
  double t = floor((double)p * 32768.0 + 0.5);
  if (t > 32768.0) t = 32768.0;
  return (uint32_t)t;
}

static inline int dropout_keep(uint64_t idx, uint64_t seed, uint32_t thr) {
  uint32_t o[4];
  uint64_t blk = idx >> 3;
  tfo_philox4x32_r((uint32_t)blk, (uint32_t)(blk >> 32), 0u, 0u, (uint32_t)seed,
                   (uint32_t)(seed >> 32), TFO_DROPOUT_ROUNDS, o);
  uint32_t e = (uint32_t)(idx & 7u);
  uint32_t field = (o[e >> 1] >> (16u * (e & 1u))) & 0x7FFFu;
  return field >= thr;
}

void tfo_dropout_mask(uint8_t* mask, uint64_t first_idx, long n, float p, uint64_t seed) {
  const uint32_t thr = tfo_dropout_threshold(p);
  for (long i = 0; i < n; ++i) mask[i] = thr == 0 ? 1 : (uint8_t)dropout_keep(first_idx + i, seed, thr);
}

/* ------------------------------------------------ softmax+dropout, exact
 * exp2 of a value t in [-127, ~0]: n = round-to-nearest-even(t) through the
 * 1.5*2^23 trick, f = t - n in [-0.5, 0.5], degree-5 polynomial in f evaluated
 * with FMAs (Horner), scaled by 2^n built from the integer bits (n = -127 gives
 * an exact 0). */
static inline float exp2_poly(float t) {
  const float MAGIC = 12582912.0f;
  const float c0 = 0x1.000002p+0f, c1 = 0x1.62e428p-1f, c2 = 0x1.ebf918p-3f,
              c3 = 0x1.c6b6e4p-5f, c4 = 0x1.3d0c52p-7f, c5 = 0x1.5c08e6p-10f;
  float r = t + MAGIC;
  float nf = r - MAGIC;
  float f = t - nf;
  float p = c5;
  p = fmaf(p, f, c4);
  p = fmaf(p, f, c3);
  p = fmaf(p, f, c2);
  p = fmaf(p, f, c1);
  p = fmaf(p, f, c0);
  uint32_t rb; memcpy(&rb, &r, 4);
  uint32_t sb = (rb << 23) + 0x3f800000u;
  float s; memcpy(&s, &sb, 4);
  return p * s;
}

/* FP16-storage form of the exponential: the input is clamped from below at
 * lo (about max - 64) before the multiply, so t stays within about [-116, 0]
 * and 2^n is added straight into the exponent field; degree-4 polynomial. */
static inline float exp2_poly_h(float t) {
  const float MAGIC = 12582912.0f;
  const float d0 = 0x1.ffffe8p-1f, d1 = 0x1.62e0dcp-1f, d2 = 0x1.ec06dap-3f,
              d3 = 0x1.ca144p-5f, d4 = 0x1.3997d6p-7f;
  float r = t + MAGIC;
  float nf = r - MAGIC;
  float f = t - nf;
  float p = d4;
  p = fmaf(p, f, d3);
  p = fmaf(p, f, d2);
  p = fmaf(p, f, d1);
  p = fmaf(p, f, d0);
  uint32_t rb, pb; memcpy(&rb, &r, 4); memcpy(&pb, &p, 4);
  uint32_t eb = pb + (rb << 23);
  float e; memcpy(&e, &eb, 4);
  return e;
}

/* One row.  x: L inputs already widened to FP32.  half_form selects the
 * FP16-storage exponential above (inputs are FP16 values), else the FP32 one.  The summation order is the
 * one a team of `warps` warps uses when unit u (V consecutive elements, V = vec)
 * belongs to thread u % (32*warps): every thread adds its elements in ascending
 * order into two accumulators (even / odd position inside the unit), adds the
 * two, the 32 lanes of a warp combine by an xor butterfly (16,8,4,2,1) and the
 * warp totals are added in ascending warp order.  y receives e_j * g with
 * g = (1/sum) * keep_scale; an all -inf row gives zeros. */
static void softmax_row_exact(const float* x, float* y, int L, int vec, int warps,
                              float keep_scale, int half_form) {
  const float LOG2E = 0x1.715476p+0f;
  float mx = -INFINITY;
  for (int j = 0; j < L; ++j) mx = fmaxf(mx, x[j]);
  const int all_masked = mx == -INFINITY;
  if (all_masked) mx = 0.0f;
  const float c = mx * LOG2E;
  const float lo = h2f(f2h(mx - 64.0f));
  const int T = 32 * warps;
  const int units = (L + vec - 1) / vec;
  float lane_sum[32 * 32];
  for (int t = 0; t < T; ++t) {
    float s0 = 0.0f, s1 = 0.0f;
    for (int u = t; u < units; u += T) {
      for (int i = 0; i < vec; ++i) {
        int j = u * vec + i;
        if (j >= L) break;
        float e = half_form ? exp2_poly_h(fmaf(fmaxf(x[j], lo), LOG2E, -c))
                            : exp2_poly(fmaxf(fmaf(x[j], LOG2E, -c), -127.0f));
        y[j] = e;
        if (i & 1) s1 += e; else s0 += e;
      }
    }
    lane_sum[t] = s0 + s1;
  }
  float total = 0.0f;
  for (int w = 0; w < warps; ++w) {
    float v[32];
    memcpy(v, lane_sum + 32 * w, sizeof(v));
    for (int off = 16; off >= 1; off >>= 1) {
      float nv[32];
      for (int l = 0; l < 32; ++l) nv[l] = v[l] + v[l ^ off];
      memcpy(v, nv, sizeof(v));
    }
    total = (w == 0) ? v[0] : total + v[0];
  }
  const float inv = (total == 0.0f || all_masked) ? 0.0f : 1.0f / total;
  const float g = inv * keep_scale;
  for (int j = 0; j < L; ++j) y[j] = y[j] * g;
}

/* One row, online form: the schedule of the library's kernel for rows that do
 * not fit in shared memory (tensorfuse_b200/csrc/softmax_dropout.cu,
 * softmax_online_kernel).  Thread t of T = 32*warps owns the units t, t+T, ...
 * (V = vec consecutive elements each) and keeps a running maximum m_t and two
 * partial sums (even / odd position inside the unit) relative to it: a unit
 * whose maximum mu exceeds m_t first multiplies both sums by
 * 2^(max(fma(m_t, log2e, -(mu*log2e)), -127)); a unit that is all -inf is
 * skipped.  At the end every thread's sum s0+s1 is multiplied by
 * 2^(max(fma(m_t, log2e, -(m*log2e)), -127)) with m the row maximum (0 for a
 * thread that saw nothing), lanes combine by the xor butterfly, warps in
 * ascending order.  FP32-storage exponential for both storage types. */
static void softmax_row_online(const float* x, float* y, int L, int vec, int warps, float keep_scale) {
  const float LOG2E = 0x1.715476p+0f;
  const int T = 32 * warps;
  const int units = (L + vec - 1) / vec;
  float lane_m[32 * 32], lane_s[32 * 32];
  float mx = -INFINITY;
  for (int t = 0; t < T; ++t) {
    float mt = -INFINITY, s0 = 0.0f, s1 = 0.0f, negc = 0.0f;
    for (int u = t; u < units; u += T) {
      const int j0 = u * vec, j1 = j0 + vec < L ? j0 + vec : L;
      float mu = -INFINITY;
      for (int j = j0; j < j1; ++j) mu = fmaxf(mu, x[j]);
      if (mu == -INFINITY) continue;
      if (mu > mt) {
        const float nc = -(mu * LOG2E);
        if (mt != -INFINITY) {
          const float f = exp2_poly(fmaxf(fmaf(mt, LOG2E, nc), -127.0f));
          s0 *= f; s1 *= f;
        }
        mt = mu; negc = nc;
      }
      for (int j = j0; j < j1; ++j) {
        const float e = exp2_poly(fmaxf(fmaf(x[j], LOG2E, negc), -127.0f));
        if ((j - j0) & 1) s1 += e; else s0 += e;
      }
    }
    lane_m[t] = mt; lane_s[t] = s0 + s1;
    mx = fmaxf(mx, mt);
  }
  const int all_masked = mx == -INFINITY;
  if (all_masked) mx = 0.0f;
  const float negc = -(mx * LOG2E);
  float total = 0.0f;
  for (int w = 0; w < warps; ++w) {
    float v[32];
    for (int l = 0; l < 32; ++l) {
      const int t = 32 * w + l;
      v[l] = lane_m[t] == -INFINITY ? 0.0f
                                    : lane_s[t] * exp2_poly(fmaxf(fmaf(lane_m[t], LOG2E, negc), -127.0f));
    }
    for (int off = 16; off >= 1; off >>= 1) {
      float nv[32];
      for (int l = 0; l < 32; ++l) nv[l] = v[l] + v[l ^ off];
      memcpy(v, nv, sizeof(v));
    }
    total = (w == 0) ? v[0] : total + v[0];
  }
  const float inv = (total == 0.0f || all_masked) ? 0.0f : 1.0f / total;
  const float g = inv * keep_scale;
  for (int j = 0; j < L; ++j) y[j] = exp2_poly(fmaxf(fmaf(x[j], LOG2E, negc), -127.0f)) * g;
}

static inline float keep_scale_of(float p) { return p >= 1.0f ? 0.0f : 1.0f / (1.0f - p); }

/* dtype: 0 = FP32 storage, 1 = FP16 storage.  first_row offsets the Philox
 * element index so that a shard of a larger tensor reproduces the mask of the
 * whole. */
static void softmax_dropout_exact_impl(const void* in, void* out, uint8_t* mask, long rows, int L,
                                       int dtype, float p, uint64_t seed, uint64_t first_row, int vec,
                                       int warps, int online, int threads);

void tfo_softmax_dropout_exact(const void* in, void* out, uint8_t* mask, long rows, int L,
                               int dtype, float p, uint64_t seed, uint64_t first_row, int vec,
                               int warps, int threads) {
  softmax_dropout_exact_impl(in, out, mask, rows, L, dtype, p, seed, first_row, vec, warps, 0, threads);
}

/* The same with the online schedule (softmax_row_online). */
void tfo_softmax_dropout_exact_online(const void* in, void* out, uint8_t* mask, long rows, int L,
                                      int dtype, float p, uint64_t seed, uint64_t first_row, int vec,
                                      int warps, int threads) {
  softmax_dropout_exact_impl(in, out, mask, rows, L, dtype, p, seed, first_row, vec, warps, 1, threads);
}

static void softmax_dropout_exact_impl(const void* in, void* out, uint8_t* mask, long rows, int L,
                                       int dtype, float p, uint64_t seed, uint64_t first_row, int vec,
                                       int warps, int online, int threads) {
  set_threads(threads);
  const uint32_t thr = tfo_dropout_threshold(p);
  const float ks = keep_scale_of(p);
#pragma omp parallel
  {
    float* x = (float*)malloc(sizeof(float) * (size_t)L);
    float* y = (float*)malloc(sizeof(float) * (size_t)L);
#pragma omp for schedule(static)
    for (long r = 0; r < rows; ++r) {
      if (dtype == 1) {
        const uint16_t* xi = (const uint16_t*)in + r * L;
        for (int j = 0; j < L; ++j) x[j] = h2f(xi[j]);
      } else {
        memcpy(x, (const float*)in + r * L, sizeof(float) * (size_t)L);
      }
      if (online) softmax_row_online(x, y, L, vec, warps, ks);
      else softmax_row_exact(x, y, L, vec, warps, ks, dtype == 1);
      for (int j = 0; j < L; ++j) {
        uint64_t idx = (first_row + (uint64_t)r) * (uint64_t)L + (uint64_t)j;
        int keep = thr == 0 ? 1 : dropout_keep(idx, seed, thr);
        float v = keep ? y[j] : 0.0f;
        mask[r * L + j] = (uint8_t)keep;
        if (dtype == 1) ((uint16_t*)out)[r * L + j] = f2h(v);
        else ((float*)out)[r * L + j] = v;
      }
    }
    free(x); free(y);
  }
}

/* Extended form of the library's softmax+dropout: softmax(scale * x) with the
 * columns >= lengths[item] masked (item = row / rows_per_item; lengths may be
 * NULL).  Widen, multiply by scale in FP32, mask, then the FP32-storage
 * arithmetic of softmax_row_exact for both storage types. */
void tfo_softmax_dropout_exact_ext(const void* in, void* out, uint8_t* mask, long rows, int L, int dtype,
                                   float p, uint64_t seed, int vec, int warps, float scale,
                                   const int* lengths, long rows_per_item, int threads) {
  set_threads(threads);
  const uint32_t thr = tfo_dropout_threshold(p);
  const float ks = keep_scale_of(p);
#pragma omp parallel
  {
    float* x = (float*)malloc(sizeof(float) * (size_t)L);
    float* y = (float*)malloc(sizeof(float) * (size_t)L);
#pragma omp for schedule(static)
    for (long r = 0; r < rows; ++r) {
      int len = L;
      if (lengths) { len = lengths[r / rows_per_item]; if (len > L) len = L; if (len < 0) len = 0; }
      for (int j = 0; j < L; ++j) {
        const float v = dtype == 1 ? h2f(((const uint16_t*)in)[r * L + j]) : ((const float*)in)[r * L + j];
        x[j] = j < len ? v * scale : -INFINITY;
      }
      softmax_row_exact(x, y, L, vec, warps, ks, 0);
      for (int j = 0; j < L; ++j) {
        uint64_t idx = (uint64_t)r * (uint64_t)L + (uint64_t)j;
        int keep = thr == 0 ? 1 : dropout_keep(idx, seed, thr);
        float v = keep ? y[j] : 0.0f;
        mask[r * L + j] = (uint8_t)keep;
        if (dtype == 1) ((uint16_t*)out)[r * L + j] = f2h(v);
        else ((float*)out)[r * L + j] = v;
      }
    }
    free(x); free(y);
  }
}

/* ---------------------------------------------------------------- helpers */

/* ------------------------------------------------- multi-head attention
 * The reference only declares this operator (src/tensorfuse/tensorfuse.h:90-114:
 * query/key/value/output [batch, seq, hidden], heads split hidden, dropout on
 * the attention weights) and leaves its body empty (src/tensorfuse_c_api.cpp:
 * 288-311), so there is nothing of the reference's to pin this against: the
 * restatement composes the reference's own softmax_ref / dropout_ref semantics
 * (src/tests/test_softmax_dropout.cu:36-79) with two plain matrix products.
 *   out[b,i,h,:] = sum_j keep/(1-p) * softmax_j(scale * q[b,i,h,:].k[b,j,h,:]) * v[b,j,h,:]
 * Inputs FP32 [batch, seq, heads*hd] (FP16 callers widen first), FP32 scores,
 * double accumulation of the weighted sum; keys j >= kv_len[b] are masked; the
 * keep decision of (b,h,i,j) is dropout_keep(((b*heads+h)*seq_q+i)*seq_kv+j). */
void tfo_attention_f32(const float* q, const float* k, const float* v, float* out, int batch,
                       int seq_q, int seq_kv, int heads, int hd, float scale, float p, uint64_t seed,
                       const int* kv_len, int threads) {
  set_threads(threads);
  const uint32_t thr = tfo_dropout_threshold(p);
  const float ks = p >= 1.0f ? 0.0f : 1.0f / (1.0f - p);
  const long hidden = (long)heads * hd;
  const long rows = (long)batch * heads * seq_q;
#pragma omp parallel
  {
    float* sc = (float*)malloc(sizeof(float) * (size_t)(seq_kv > 0 ? seq_kv : 1));
    double* acc = (double*)malloc(sizeof(double) * (size_t)hd);
#pragma omp for schedule(static)
    for (long r = 0; r < rows; ++r) {
      const int i = (int)(r % seq_q), h = (int)((r / seq_q) % heads), b = (int)(r / ((long)seq_q * heads));
      int n = seq_kv;
      if (kv_len) { n = kv_len[b] < n ? kv_len[b] : n; if (n < 0) n = 0; }
      const float* qr = q + ((long)b * seq_q + i) * hidden + (long)h * hd;
      float* o = out + ((long)b * seq_q + i) * hidden + (long)h * hd;
      float mx = -INFINITY;
      for (int j = 0; j < n; ++j) {
        const float* kr = k + ((long)b * seq_kv + j) * hidden + (long)h * hd;
        float d = 0.0f;
        for (int c = 0; c < hd; ++c) d += qr[c] * kr[c];
        sc[j] = d * scale;
        mx = fmaxf(mx, sc[j]);
      }
      float sum = 0.0f;
      for (int j = 0; j < n; ++j) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
      for (int c = 0; c < hd; ++c) acc[c] = 0.0;
      for (int j = 0; j < n; ++j) {
        if (thr != 0 && !dropout_keep((uint64_t)r * (uint64_t)seq_kv + (uint64_t)j, seed, thr)) continue;
        const float w = sc[j] / sum * ks;
        const float* vr = v + ((long)b * seq_kv + j) * hidden + (long)h * hd;
        for (int c = 0; c < hd; ++c) acc[c] += (double)w * vr[c];
      }
      for (int c = 0; c < hd; ++c) o[c] = n > 0 ? (float)acc[c] : 0.0f;
    }
    free(sc);
    free(acc);
  }
}

void tfo_f32_to_f16(const float* src, uint16_t* dst, long n) { for (long i = 0; i < n; ++i) dst[i] = f2h(src[i]); }
void tfo_f16_to_f32(const uint16_t* src, float* dst, long n) { for (long i = 0; i < n; ++i) dst[i] = h2f(src[i]); }
