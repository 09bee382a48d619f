// attention.cu -- host side of the fused multi-head attention forward and the
// CUDA-core kernel that serves the shapes the tensor-core kernel does not take.
//
// The reference exports tensorfuse_fused_multi_head_attention as a placeholder
// that validates its arguments and writes nothing (reference
// src/tensorfuse_c_api.cpp:288-311; header text src/tensorfuse/tensorfuse.h:90-114:
// query/key/value/output are [batch, seq_len, hidden_dim], dropout acts on the
// attention weights).  Here it computes.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <mutex>

#include "attention_tc_kernel.cuh"
#include "tma_host.h"

namespace tfb {
namespace {

// ------------------------------------------------------------ CUDA-core kernel
// One warp per (batch item, head, query row).  Keys are taken 32 at a time: lane
// = key for the score and the online softmax, lane = output column (c, c+32, ...)
// for the accumulation.  FP32 arithmetic, any head width up to 256, any strides.
struct SimtParams {
  const void* q; const void* k; const void* v; void* out;
  int batch, heads, seq_q, seq_kv, hd;
  long long ld_q, ld_k, ld_v, ld_o, hs_q, hs_k, hs_v, hs_o, bs_q, bs_k, bs_v, bs_o;
  float scale, keep_scale;
  uint32_t thr;
  const int* kv_lengths;
  uint32_t key[20];
};

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

constexpr int kSimtWarps = 4;
constexpr int kMaxHd = 256;

template <typename T>
__global__ void __launch_bounds__(kSimtWarps * 32)
attention_simt_kernel(const __grid_constant__ SimtParams p) {
  __shared__ float qs[kSimtWarps][kMaxHd];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long rows = (long long)p.batch * p.heads * p.seq_q;
  const long long rid = (long long)blockIdx.x * kSimtWarps + warp;
  if (rid >= rows) return;
  const int i = (int)(rid % p.seq_q);
  const int h = (int)((rid / p.seq_q) % p.heads);
  const int b = (int)(rid / ((long long)p.seq_q * p.heads));
  const T* q = static_cast<const T*>(p.q) + b * p.bs_q + i * p.ld_q + h * p.hs_q;
  const T* kb = static_cast<const T*>(p.k) + b * p.bs_k + h * p.hs_k;
  const T* vb = static_cast<const T*>(p.v) + b * p.bs_v + h * p.hs_v;
  T* o = static_cast<T*>(p.out) + b * p.bs_o + i * p.ld_o + h * p.hs_o;
  int kv_len = p.seq_kv;
  if (p.kv_lengths != nullptr) kv_len = max(0, min(kv_len, p.kv_lengths[b]));
  for (int c = lane; c < p.hd; c += 32) qs[warp][c] = to_f<T>(q[c]);
  __syncwarp();
  constexpr int kCols = kMaxHd / 32;
  float acc[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) acc[c] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;
  const unsigned long long idx_row = (unsigned long long)rid * (unsigned long long)p.seq_kv;
  for (int j0 = 0; j0 < kv_len; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j < kv_len) {
      const T* kr = kb + j * p.ld_k;
      float d = 0.0f;
      for (int c = 0; c < p.hd; ++c) d = fmaf(qs[warp][c], to_f<T>(kr[c]), d);
      s = d * p.scale;
    }
    float mx = s;
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, w));
    const float m_new = fmaxf(m_run, mx);
    const float alpha = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
    float e = j < kv_len ? expf(s - m_new) : 0.0f;
    float es = e;
#pragma unroll
    for (int w = 16; w > 0; w >>= 1) es += __shfl_xor_sync(0xFFFFFFFFu, es, w);
    l_run = l_run * alpha + es;
    m_run = m_new;
    if (p.thr != 0u && j < kv_len && !philox_keep(idx_row + (unsigned)j, p.key, p.thr)) e = 0.0f;
#pragma unroll
    for (int c = 0; c < kCols; ++c) acc[c] *= alpha;
    const int n = min(32, kv_len - j0);
    for (int t = 0; t < n; ++t) {
      const float pt = __shfl_sync(0xFFFFFFFFu, e, t);
      const T* vr = vb + (long long)(j0 + t) * p.ld_v;
#pragma unroll
      for (int c = 0; c < kCols; ++c)
        if (lane + 32 * c < p.hd) acc[c] = fmaf(pt, to_f<T>(vr[lane + 32 * c]), acc[c]);
    }
  }
  const float inv = l_run > 0.0f ? p.keep_scale / l_run : 0.0f;
#pragma unroll
  for (int c = 0; c < kCols; ++c)
    if (lane + 32 * c < p.hd) o[lane + 32 * c] = from_f<T>(acc[c] * inv);
}

LaunchResult run_simt(const AttnArgs& a, float scale, cudaStream_t stream) {
  if (a.head_dim > kMaxHd) return kUnsupported;
  SimtParams sp;
  sp.q = a.q; sp.k = a.k; sp.v = a.v; sp.out = a.out;
  sp.batch = a.batch; sp.heads = a.heads; sp.seq_q = a.seq_q; sp.seq_kv = a.seq_kv; sp.hd = a.head_dim;
  sp.ld_q = a.ld_q; sp.ld_k = a.ld_k; sp.ld_v = a.ld_v; sp.ld_o = a.ld_o;
  sp.hs_q = a.hs_q; sp.hs_k = a.hs_k; sp.hs_v = a.hs_v; sp.hs_o = a.hs_o;
  sp.bs_q = a.bs_q; sp.bs_k = a.bs_k; sp.bs_v = a.bs_v; sp.bs_o = a.bs_o;
  sp.scale = scale;
  sp.keep_scale = a.p >= 1.0f ? 0.0f : 1.0f / (1.0f - a.p);
  sp.thr = dropout_threshold(a.p);
  sp.kv_lengths = a.kv_lengths;
  philox_round_keys(a.seed, sp.key);
  const long long rows = (long long)a.batch * a.heads * a.seq_q;
  const long long blocks = (rows + kSimtWarps - 1) / kSimtWarps;
  if (blocks > 0x7FFFFFFFll) return kUnsupported;
  if (a.dtype == kF16) attention_simt_kernel<__half><<<(unsigned)blocks, kSimtWarps * 32, 0, stream>>>(sp);
  else if (a.dtype == kBF16) attention_simt_kernel<__nv_bfloat16><<<(unsigned)blocks, kSimtWarps * 32, 0, stream>>>(sp);
  else attention_simt_kernel<float><<<(unsigned)blocks, kSimtWarps * 32, 0, stream>>>(sp);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

// -------------------------------------------------------- tensor-core kernel
// FP16 tensor viewed as [batch][heads][seq][64]; a box is 128 sequence positions
// of one head: 128 rows of 128 bytes, 128-byte swizzle.
struct Map4Key {
  const void* base; int seq, heads, batch; long long ld, hs, bs;
  int box_rows = 128;     // sequence positions per box: 128 for loads, 32 for a warp's output rows
  bool operator==(const Map4Key& o) const {
    return base == o.base && seq == o.seq && heads == o.heads && batch == o.batch && ld == o.ld && hs == o.hs &&
           bs == o.bs && box_rows == o.box_rows;
  }
};
bool make_map4(CUtensorMap* m, const Map4Key& k) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t gdim[4] = {(cuuint64_t)attn::HD, (cuuint64_t)k.seq, (cuuint64_t)k.heads, (cuuint64_t)k.batch};
  const cuuint64_t gstride[3] = {(cuuint64_t)k.ld * 2, (cuuint64_t)k.hs * 2, (cuuint64_t)k.bs * 2};
  const cuuint32_t box[4] = {(cuuint32_t)attn::HD, (cuuint32_t)k.box_rows, 1u, 1u};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(k.base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool cached_map4(const Map4Key& k, CUtensorMap* out) {
  constexpr int kSlots = 16;
  thread_local Map4Key keys[kSlots];
  thread_local CUtensorMap maps[kSlots];
  thread_local bool used[kSlots] = {};
  thread_local int next = 0;
  for (int i = 0; i < kSlots; ++i)
    if (used[i] && keys[i] == k) { *out = maps[i]; return true; }
  const int slot = next;
  next = (next + 1) % kSlots;
  used[slot] = false;
  if (!make_map4(&maps[slot], k)) return false;
  keys[slot] = k;
  used[slot] = true;
  *out = maps[slot];
  return true;
}

template <bool DROP, bool BF16>
LaunchResult run_tc(const AttnArgs& a, float scale, cudaStream_t stream) {
  using namespace attn;
  auto kernel = attention_tc_kernel<DROP, BF16>;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return kCudaError;
  static bool ready[64] = {};
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    if (!ready[dev]) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return kCudaError;
      }
      ready[dev] = true;
    }
  }
  CUtensorMap mq, mk, mv, mo;
  if (!cached_map4(Map4Key{a.q, a.seq_q, a.heads, a.batch, a.ld_q, a.hs_q, a.bs_q}, &mq) ||
      !cached_map4(Map4Key{a.k, a.seq_kv, a.heads, a.batch, a.ld_k, a.hs_k, a.bs_k}, &mk) ||
      !cached_map4(Map4Key{a.v, a.seq_kv, a.heads, a.batch, a.ld_v, a.hs_v, a.bs_v}, &mv) ||
      !cached_map4(Map4Key{a.out, a.seq_q, a.heads, a.batch, a.ld_o, a.hs_o, a.bs_o, 32}, &mo))
    return kLaunchFailed;
  Params p;
  p.batch = a.batch; p.heads = a.heads; p.seq_q = a.seq_q; p.seq_kv = a.seq_kv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.keep_scale = a.p >= 1.0f ? 0.0f : 1.0f / (1.0f - a.p);
  p.thr = dropout_threshold(a.p);
  p.thr_h2 = (p.thr & 0xFFFFu) * 0x00010001u;
  p.hcmp = p.thr <= 0x7C00u ? 1 : 0;
  p.kv_lengths = a.kv_lengths;
  philox_round_keys(a.seed, p.key);
  p.q_tiles = (a.seq_q + BQ - 1) / BQ;
  const long long items = (long long)p.q_tiles * a.heads * a.batch;
  if (items > 0x7FFFFFFFll) return kUnsupported;
  p.n_tiles = (int)items;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const unsigned grid = (unsigned)(items < 2ll * sms ? items : 2ll * sms);
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(mq, mk, mv, mo, p, watchdog_word());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace

bool attention_tc_eligible(const AttnArgs& a) {
  if ((a.dtype != kF16 && a.dtype != kBF16) || a.head_dim != attn::HD) return false;
  const uintptr_t ptrs = (uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.out;
  if (ptrs & 15u) return false;
  const long long strides[12] = {a.ld_q, a.ld_k, a.ld_v, a.ld_o, a.hs_q, a.hs_k, a.hs_v, a.hs_o,
                                 a.bs_q, a.bs_k, a.bs_v, a.bs_o};
  for (long long s : strides)
    if (s <= 0 || (s % 8) != 0) return false;      // tensor-map strides: positive multiples of 16 bytes
  if (dropout_threshold(a.p) != 0u && (a.seq_kv % 8) != 0) return false;   // one Philox block = 8 keys of one row
  return true;
}

LaunchResult launch_attention(const AttnArgs& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.out) return kInvalidArgument;
  if (a.dtype != kF16 && a.dtype != kBF16 && a.dtype != kF32) return kUnsupported;
  if (a.batch < 0 || a.seq_q < 0 || a.seq_kv < 0 || a.heads <= 0 || a.head_dim <= 0) return kInvalidArgument;
  if (!(a.p >= 0.0f && a.p <= 1.0f)) return kInvalidArgument;
  if (a.batch == 0 || a.seq_q == 0) return kOk;
  const float scale = a.scale > 0.0f ? a.scale : 1.0f / sqrtf((float)a.head_dim);
  if (a.seq_kv > 0 && attention_tc_eligible(a)) {
    const bool drop = dropout_threshold(a.p) != 0u;
    if (a.dtype == kBF16) return drop ? run_tc<true, true>(a, scale, stream) : run_tc<false, true>(a, scale, stream);
    return drop ? run_tc<true, false>(a, scale, stream) : run_tc<false, false>(a, scale, stream);
  }
  return run_simt(a, scale, stream);
}

}  // namespace tfb

