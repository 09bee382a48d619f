// transformer_layer.cpp -- tensorfuse_fused_transformer_layer as a composition
// of the library's own kernels on one stream:
//     q|k|v = x [Wq|Wk|Wv] + [bq|bk|bv]            (one GEMM, bias-only epilogue, on a concatenated weight)
//     ctx   = attention(q, k, v; heads, dropout)    (fused attention kernel)
//     h1    = LayerNorm1(x + ctx Wo + bo)           (GEMM, then residual + LN kernel)
//     out   = LayerNorm2(h1 + act(h1 W1 + b1) W2 + b2)   (GEMM+bias+GELU, GEMM+bias, residual + LN)
// i.e. a post-LN (BERT-style) encoder layer; dropout acts on the attention
// weights only.  The reference declares the entry point and the parameter block
// (src/tensorfuse/tensorfuse.h:116-133, src/tensorfuse/types.h:153-185) and
// returns success without touching the output (src/tensorfuse_c_api.cpp:313-329).
// Workspace (4 x [tokens, hidden] + [tokens, ffn] + the concatenated weight) comes
// from a stream-ordered memory pool that the library owns (one per device, kept
// until shutdown) and is returned to it on the same stream, so the call stays
// asynchronous, calls on different streams do not share buffers, and the
// process's default pool is left alone.  When the three projection weights are
// registered as immutable the concatenated weight is built once and kept.
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"
#include "runtime.h"
#include "tensorfuse/tensorfuse.h"

using namespace tfb;

namespace {

TensorFuseStatus st_of(LaunchResult r) { return static_cast<TensorFuseStatus>(static_cast<int>(r)); }

bool is_matrix(const TensorFuseTensor* t, int rows, int cols, TensorFuseDataType dt) {
  return t && t->data && t->shape.ndims == 2 && t->shape.dims[0] == rows && t->shape.dims[1] == cols && t->dtype == dt;
}
bool is_vector(const TensorFuseTensor* t, int n, TensorFuseDataType dt) {
  return t && t->data && t->shape.ndims == 1 && t->shape.dims[0] == n && t->dtype == dt;
}

LaunchResult gemm(const void* A, const void* B, const void* bias, void* C, int M, int N, int K, int dt, int epi,
                  float beta, cudaStream_t stream) {
  GemmArgs a{};
  a.A = A; a.B = B; a.bias = bias; a.C = C;
  a.M = M; a.N = N; a.K = K;
  a.in_dtype = dt; a.bias_dtype = dt; a.out_dtype = dt;
  a.epilogue = epi;
  a.alpha = 1.0f; a.beta = beta; a.scale = 1.0f;
  return launch_gemm(a, stream);
}

}  // namespace

extern "C" TensorFuseStatus tensorfuse_fused_transformer_layer(const TensorFuseTensor* input, TensorFuseTensor* output,
                                                               const TensorFuseTransformerParams* p,
                                                               cudaStream_t stream) {
  if (!Runtime::get().initialized()) return TENSORFUSE_ERROR_NOT_INITIALIZED;
  if (!input || !output || !p) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (p->num_heads <= 0 || !(p->dropout_prob >= 0.0f && p->dropout_prob <= 1.0f) || !(p->layer_norm_eps >= 0.0f))
    return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (input->shape.ndims != 3 || output->shape.ndims != 3) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const int B = input->shape.dims[0], S = input->shape.dims[1], H = input->shape.dims[2];
  if (B < 0 || S < 0 || H <= 0 || H % p->num_heads != 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (output->shape.dims[i] != input->shape.dims[i]) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const TensorFuseDataType dt = input->dtype;
  if (output->dtype != dt) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (dt != TENSORFUSE_FLOAT16 && dt != TENSORFUSE_BFLOAT16 && dt != TENSORFUSE_FLOAT32)
    return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  int epi_ffn;
  if (p->ffn_activation == TENSORFUSE_ACTIVATION_GELU) epi_ffn = kEpiGelu;
  else if (p->ffn_activation == TENSORFUSE_ACTIVATION_NONE) epi_ffn = kEpiLinear;
  else return TENSORFUSE_ERROR_UNSUPPORTED_OPERATION;
  if (!p->ffn_weight1 || p->ffn_weight1->shape.ndims != 2) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  const int F = p->ffn_weight1->shape.dims[1];
  if (F <= 0) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (!is_matrix(p->query_weight, H, H, dt) || !is_matrix(p->key_weight, H, H, dt) ||
      !is_matrix(p->value_weight, H, H, dt) || !is_matrix(p->output_weight, H, H, dt) ||
      !is_matrix(p->ffn_weight1, H, F, dt) || !is_matrix(p->ffn_weight2, F, H, dt) ||
      !is_vector(p->ln1_weight, H, dt) || !is_vector(p->ln1_bias, H, dt) || !is_vector(p->ln2_weight, H, dt) ||
      !is_vector(p->ln2_bias, H, dt))
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  if (p->use_bias &&
      (!is_vector(p->query_bias, H, dt) || !is_vector(p->key_bias, H, dt) || !is_vector(p->value_bias, H, dt) ||
       !is_vector(p->output_bias, H, dt) || !is_vector(p->ffn_bias1, F, dt) || !is_vector(p->ffn_bias2, H, dt)))
    return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const long long tokens = (long long)B * S;
  if (tokens == 0) return TENSORFUSE_SUCCESS;
  if (!input->data || !output->data) return TENSORFUSE_ERROR_INVALID_ARGUMENT;
  if (tokens > 0x7FFFFFFFll) return TENSORFUSE_ERROR_INVALID_TENSOR_SHAPE;
  const int M = (int)tokens;
  const int kdt = dt == TENSORFUSE_FLOAT16 ? kF16 : dt == TENSORFUSE_BFLOAT16 ? kBF16 : kF32;
  const size_t es = kdt == kF32 ? 4 : 2;

  const int dev = device_of_pointer(output->data);
  DeviceGuard guard(dev);
  // workspace from the library's own stream-ordered pool (kept cached between calls)
  int pool_dev = dev;
  if (pool_dev < 0) cudaGetDevice(&pool_dev);
  cudaMemPool_t pool = Runtime::get().workspace_pool(pool_dev);
  if (pool == nullptr) return TENSORFUSE_ERROR_OUT_OF_MEMORY;
  auto round_up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t mh = round_up((size_t)M * H * es), mf = round_up((size_t)M * F * es);
  const size_t wcat_bytes = round_up((size_t)3 * H * H * es);
  const size_t bcat_bytes = round_up((size_t)(3 * H > F ? 3 * H : F) * es);
  char* ws = nullptr;
  if (cudaMallocFromPoolAsync(reinterpret_cast<void**>(&ws), 4 * mh + mf + wcat_bytes + bcat_bytes, pool, stream) !=
      cudaSuccess) {
    cudaGetLastError();
    return TENSORFUSE_ERROR_OUT_OF_MEMORY;
  }
  // ws: [tokens, 3*hidden] fused Q|K|V (reused after the attention as three [tokens, hidden]
  // buffers), ctx, the FFN intermediate, the concatenated projection weight and bias.
  char* qkv = ws; char* ctx = ws + 3 * mh; char* up = ws + 4 * mh;
  char* wcat = ws + 4 * mh + mf; char* bcat = wcat + wcat_bytes;
  char* attn = ws;            // Q|K|V are dead after the attention
  char* h1 = ws + mh;
  char* down = ws + 2 * mh;
  const float beta = p->use_bias ? 1.0f : 0.0f;
  const void* zero = bcat;    // without biases bcat is all zeros and beta is 0

  LaunchResult r = kOk;
  auto step = [&](LaunchResult x) { if (r == kOk) r = x; };
  auto cuda_step = [&](cudaError_t e) { if (e != cudaSuccess) { cudaGetLastError(); if (r == kOk) r = kCudaError; } };
  auto bias_of = [&](const TensorFuseTensor* t) -> const void* { return p->use_bias ? t->data : zero; };
  // One projection GEMM for Q, K and V: the three [hidden, hidden] weights are laid side by side
  // as [hidden, 3*hidden] (6 MB of copies at BERT-large size against two fewer passes over the
  // activations), the biases likewise.
  const size_t wrow = (size_t)H * es;
  const TensorFuseTensor* wq[3] = {p->query_weight, p->key_weight, p->value_weight};
  const TensorFuseTensor* bq[3] = {p->query_bias, p->key_bias, p->value_bias};
  auto concatenate = [&](char* wdst, char* bdst) {
    for (int i = 0; i < 3; ++i) {
      cuda_step(cudaMemcpy2DAsync(wdst + i * wrow, 3 * wrow, wq[i]->data, wrow, wrow, (size_t)H,
                                  cudaMemcpyDeviceToDevice, stream));
      if (p->use_bias) cuda_step(cudaMemcpyAsync(bdst + i * wrow, bq[i]->data, wrow, cudaMemcpyDeviceToDevice, stream));
    }
  };
  // Weights registered as immutable (tensorfuse_b200_register_weights on the three
  // device matrices): the concatenation is built once per device and kept.
  const char* w_qkv = wcat;
  const char* b_qkv = bcat;
  bool fresh = false;
  Runtime::FusedQkv* slot = Runtime::get().fused_qkv_slot(pool_dev, wq[0]->data, wq[1]->data, wq[2]->data, &fresh);
  if (!p->use_bias) cuda_step(cudaMemsetAsync(bcat, 0, bcat_bytes, stream));
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(stream, &capturing);
  std::unique_lock<std::mutex> slot_lock;
  if (slot != nullptr) slot_lock = std::unique_lock<std::mutex>(slot->mu);
  const bool must_build = slot != nullptr && (fresh || slot->w_bytes != wcat_bytes || slot->b_bytes != bcat_bytes);
  if (must_build && capturing != cudaStreamCaptureStatusNone) {   // building synchronises: not inside a capture
    slot_lock.unlock();
    slot = nullptr;
  }
  if (slot != nullptr && p->use_bias) {
    if (must_build) {
      if (slot->w) cudaFree(slot->w);
      if (slot->b) cudaFree(slot->b);
      slot->w = slot->b = nullptr;
      if (cudaMalloc(&slot->w, wcat_bytes) == cudaSuccess && cudaMalloc(&slot->b, bcat_bytes) == cudaSuccess) {
        slot->w_bytes = wcat_bytes; slot->b_bytes = bcat_bytes;
        concatenate(static_cast<char*>(slot->w), static_cast<char*>(slot->b));
        cudaStreamSynchronize(stream);    // later calls may come on other streams
      } else {
        cudaGetLastError();
        if (slot->w) cudaFree(slot->w);
        slot->w = slot->b = nullptr; slot->w_bytes = slot->b_bytes = 0;
      }
    }
    if (slot->w != nullptr) { w_qkv = static_cast<const char*>(slot->w); b_qkv = static_cast<const char*>(slot->b); }
  }
  if (slot_lock.owns_lock()) slot_lock.unlock();
  if (w_qkv == wcat) concatenate(wcat, bcat);
  step(gemm(input->data, w_qkv, b_qkv, qkv, M, 3 * H, H, kdt, kEpiLinear, beta, stream));
  if (r == kOk) {
    AttnArgs a{};
    a.q = qkv; a.k = qkv + wrow; a.v = qkv + 2 * wrow; a.out = ctx;
    a.batch = B; a.seq_q = S; a.seq_kv = S; a.heads = p->num_heads; a.head_dim = H / p->num_heads;
    a.ld_q = a.ld_k = a.ld_v = 3LL * H; a.ld_o = H;
    a.hs_q = a.hs_k = a.hs_v = a.hs_o = a.head_dim;
    a.bs_q = a.bs_k = a.bs_v = 3LL * S * H; a.bs_o = (long long)S * H;
    a.dtype = kdt; a.scale = 0.0f; a.p = p->dropout_prob; a.seed = Runtime::get().next_seed();
    a.kv_lengths = nullptr;
    step(launch_attention(a, stream));
  }
  step(gemm(ctx, p->output_weight->data, bias_of(p->output_bias), attn, M, H, H, kdt, kEpiLinear, beta, stream));
  step(launch_add_layernorm(input->data, attn, p->ln1_weight->data, p->ln1_bias->data, h1, M, H, kdt,
                            p->layer_norm_eps, stream));
  step(gemm(h1, p->ffn_weight1->data, bias_of(p->ffn_bias1), up, M, F, H, kdt, epi_ffn, beta, stream));
  step(gemm(up, p->ffn_weight2->data, bias_of(p->ffn_bias2), down, M, H, F, kdt, kEpiLinear, beta, stream));
  step(launch_add_layernorm(h1, down, p->ln2_weight->data, p->ln2_bias->data, output->data, M, H, kdt,
                            p->layer_norm_eps, stream));
  cudaFreeAsync(ws, stream);
  return st_of(r);
}
