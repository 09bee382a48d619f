// kernels.h -- internal launcher interface between the C ABI layer and the
// CUDA translation units.  Plain pointers and sizes only.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tfb {

// Storage types as seen by the launchers (values equal TensorFuseDataType).
enum DType : int { kF32 = 0, kF16 = 1, kBF16 = 2, kI8 = 3, kU8 = 4, kI32 = 5, kFp8E4M3 = 6, kFp8E5M2 = 7 };

// Result of a launcher; mapped 1:1 on TensorFuseStatus by the ABI layer.
enum LaunchResult : int {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kLaunchFailed = 6,
  kUnsupported = 10,
};

// ------------------------------------------------------- softmax + dropout
// Summation schedule the kernel uses for a row of L elements; the CPU oracle
// takes the same two numbers to reproduce the result bit for bit.
//   vec    : consecutive elements owned by one thread per step (8 or 1)
//   warps  : warps cooperating on one row (1 = warp-per-row kernel)
//   online : 1 when the row is too long for shared memory and the sum is formed
//            in one sweep with a running maximum (rescaled partial sums)
struct SoftmaxSchedule {
  int vec;
  int warps;
  int online;
};
SoftmaxSchedule softmax_schedule(int L, int dtype, bool aligned16);

// rows x L, softmax over L, dropout with probability p, Philox stream keyed by
// seed and indexed by (first_row + row) * L + col.
LaunchResult launch_softmax_dropout(const void* in, void* out, unsigned char* mask,
                                    long long rows, int L, int dtype, float p,
                                    unsigned long long seed, unsigned long long first_row,
                                    cudaStream_t stream);

// Extended form: softmax(scale * x) with the columns >= lengths[item] of every
// row masked (item = (first_row + row) / rows_per_item; lengths may be null).
// Both storage types use the FP32-storage arithmetic here.
LaunchResult launch_softmax_dropout_ext(const void* in, void* out, unsigned char* mask, long long rows, int L,
                                        int dtype, float p, unsigned long long seed, unsigned long long first_row,
                                        float scale, const int* lengths, long long rows_per_item, bool extended,
                                        cudaStream_t stream);

// ------------------------------------------------------ GEMM + bias + GELU
enum Epilogue : int {
  kEpiGelu = 0,        // out = gelu(alpha*acc + beta*bias)                 (FP32 / FP16 paths)
  kEpiI8Dequant = 1,   // out = gelu(fma(float(acc), scale, bias))          (INT8 and FP8 operands, multiply convention)
  kEpiI8Legacy = 2,    // out = gelu_clamped(acc/scale + bias)*scale, non-finite -> 0 (INT8, reference convention)
  kEpiI8Raw = 3,       // out = acc (INT32), no bias, no activation
  kEpiLinear = 4,      // out = alpha*acc + beta*bias, no activation        (FP32 / FP16 paths, e.g. FFN-down)
};

struct GemmArgs {
  const void* A;     // [M,K] row-major
  const void* B;     // [K,N] row-major
  const void* bias;  // [N]
  void* C;           // [M,N] row-major
  int M, N, K;
  int in_dtype;      // kF32 | kF16 | kBF16 | kI8 | kFp8E4M3
  int bias_dtype;    // kF32 | kF16 | kBF16
  int out_dtype;     // kF32 | kF16 | kBF16 | kI32
  int epilogue;
  float alpha, beta, scale;       // scale: product of the host-known dequant factors
  const float* scale_a_dev;       // optional device pointers to one float each; multiplied
  const float* scale_b_dev;       // into `scale` on the device
  const float* scale_b_cols;      // optional device array of N floats: per-column factor of B (kEpiI8Dequant only);
                                  // needs 16-byte alignment
};

// True when the tensor-core (TMA + tcgen05) kernel can take this problem:
// FP16, BF16, INT8 or FP8-E4M3 operands, 16-byte aligned base pointers and row pitches.
bool gemm_tc_eligible(const GemmArgs& a);
LaunchResult launch_gemm_tc(const GemmArgs& a, cudaStream_t stream);
// FP32 operands on the tensor cores (three TF32 products per FP32 product, FP32
// accumulation): 16-byte aligned pointers, K and N multiples of 4, problems of at
// least 2^24 multiply-adds.  Uses stream-ordered scratch for the split operands.
bool gemm_tf32x3_eligible(const GemmArgs& a);
// Any shape, any alignment; CUDA-core FMA kernel with the same fused epilogue.
LaunchResult launch_gemm_simt(const GemmArgs& a, cudaStream_t stream);
// Picks the tensor-core kernel when eligible, else the CUDA-core kernel.
LaunchResult launch_gemm(const GemmArgs& a, cudaStream_t stream);

// ------------------------------------------------- multi-head attention
// out[b, i, h, :] = sum_j keep(b,h,i,j)/(1-p) * softmax_j(scale * q[b,i,h,:].k[b,j,h,:]) * v[b,j,h,:]
// Element (b, s, h, c) of a tensor sits at base + b*bs + s*ld + h*hs + c (in
// elements); [batch, seq, hidden] is ld = hidden, hs = head_dim, bs = seq*hidden.
// Keys j >= kv_lengths[b] (when given) are masked; a row with no valid key
// yields zeros.  The dropout decision of probability (b, h, i, j) is that of
// element ((b*heads + h)*seq_q + i)*seq_kv + j of a [B, H, Sq, Skv] tensor in
// the softmax+dropout operator, so the fused result equals the composition
// softmax_dropout(scores) . V for the same seed.
struct AttnArgs {
  const void* q; const void* k; const void* v; void* out;
  int batch, seq_q, seq_kv, heads, head_dim;
  long long ld_q, ld_k, ld_v, ld_o;   // between sequence positions
  long long hs_q, hs_k, hs_v, hs_o;   // between heads
  long long bs_q, bs_k, bs_v, bs_o;   // between batch items
  int dtype;                          // kF16 | kF32
  float scale;                        // <= 0 selects 1/sqrt(head_dim)
  float p;
  unsigned long long seed;
  const int* kv_lengths;              // device pointer to `batch` ints, or null
};
bool attention_tc_eligible(const AttnArgs& a);
LaunchResult launch_attention(const AttnArgs& a, cudaStream_t stream);

// ------------------------------------------------------ INT8 quantisation
// Per-tensor symmetric: *scale_dev = max|x|/127 (1 for an all-zero tensor),
// q = clip(rint(x / scale), -127, 127).  Allocates nothing: the scale word is
// the reduction's scratch.
LaunchResult launch_quantize_int8(const void* x, int dtype, long long n, signed char* q, float* scale_dev,
                                  cudaStream_t stream);

// ------------------------------------------------- residual + layer norm
// out = LayerNorm(x + residual) * gamma + beta over rows of `hidden` elements
// (residual may be null); FP32 arithmetic, x/residual/gamma/beta/out of `dtype`.
LaunchResult launch_add_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* out,
                                  long long rows, int hidden, int dtype, float eps, cudaStream_t stream);

// Column-wise variant for weights: scales[n] = max_k |w[k,n]| / 127 (1 for an
// all-zero column), q[k,n] = clip(rint(w[k,n] / scales[n]), -127, 127); w is
// [K, N] row-major FP16 or FP32.
LaunchResult launch_quantize_int8_columns(const void* w, int dtype, int K, int N, signed char* q, float* scales_dev,
                                          cudaStream_t stream);

// Device-side watchdog: 0 when no bounded wait has expired since the last
// reset, else the code of the first wait that gave up.
int watchdog_status();
void watchdog_reset();
int* watchdog_word();  // host-mapped word the kernels write

// Number of kernels this library has launched in the calling process.
unsigned long long launch_count();
void count_launch(int n = 1);

}  // namespace tfb
