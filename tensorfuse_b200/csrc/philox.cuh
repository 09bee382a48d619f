// philox.cuh -- Philox4x32 as the dropout generator of the library, with
// kPhiloxRounds = 7 rounds: the fewest for which Salmon et al. (SC'11) report
// the generator to pass every test of BigCrush ("crush-resistant"); the
// customary 10 rounds are that plus a safety margin, and three rounds are a
// third of the integer work of a kernel that is bound by instruction issue.
// The round function itself is pinned by the 10-round known-answer vectors of
// the Random123 distribution (tests of the CPU restatement).
//
// Eight consecutive elements of a tensor share one Philox block: counter =
// (global element index / 8, 0, 0) split into two 32-bit words, key = seed.
// Element e of the block takes the 16-bit field (word e/2, half e%2) and is
// kept when the low 15 bits of that field are >= round(p * 32768).  The
// decision depends only on the element's position in the whole tensor, so it
// does not change with the way rows are sharded across GPUs or tiled inside a
// kernel.
#pragma once
#include <math.h>
#include <stdint.h>

namespace tfb {

constexpr int kPhiloxRounds = 7;

// Round keys (the key schedule is a pair of additive Weyl sequences).
inline void philox_round_keys(unsigned long long seed, uint32_t (&key)[20]) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {   // the array has room for ten rounds; the kernels use the first kPhiloxRounds
    key[2 * r] = k0; key[2 * r + 1] = k1;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
}
// Drop when the 15-bit field < threshold; 0 disables dropout.
inline uint32_t dropout_threshold(float p) {
  if (!(p > 0.0f)) return 0u;
  const double t = floor((double)p * 32768.0 + 0.5);
  return (uint32_t)(t > 32768.0 ? 32768.0 : t);
}

#ifdef __CUDACC__
__device__ __forceinline__ void philox_block(uint32_t c0, uint32_t c1, const uint32_t* key,
                                             uint32_t (&o)[4]) {
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < kPhiloxRounds; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ key[2 * r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ key[2 * r + 1];
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
  }
  o[0] = c0; o[1] = c1; o[2] = c2; o[3] = c3;
}
// Four blocks with consecutive 64-bit counters blk .. blk+3, rounds outermost so
// that the four dependency chains interleave.
__device__ __forceinline__ void philox_block_x4(unsigned long long blk, const uint32_t* key,
                                                uint32_t (&o)[4][4]) {
  uint32_t a0[4], a1[4], a2[4], a3[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const unsigned long long b = blk + (unsigned)q;
    a0[q] = (uint32_t)b; a1[q] = (uint32_t)(b >> 32); a2[q] = 0u; a3[q] = 0u;
  }
#pragma unroll
  for (int r = 0; r < kPhiloxRounds; ++r) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint64_t p0 = (uint64_t)0xD2511F53u * a0[q];
      const uint64_t p1 = (uint64_t)0xCD9E8D57u * a2[q];
      const uint32_t n0 = (uint32_t)(p1 >> 32) ^ a1[q] ^ key[2 * r];
      const uint32_t n2 = (uint32_t)(p0 >> 32) ^ a3[q] ^ key[2 * r + 1];
      a1[q] = (uint32_t)p1;
      a3[q] = (uint32_t)p0;
      a0[q] = n0;
      a2[q] = n2;
    }
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) { o[q][0] = a0[q]; o[q][1] = a1[q]; o[q][2] = a2[q]; o[q][3] = a3[q]; }
}
// NB independent blocks (arbitrary counters), rounds outermost so that the
// dependency chains interleave.
template <int NB>
__device__ __forceinline__ void philox_blocks(const unsigned long long (&blk)[NB], const uint32_t* key,
                                              uint32_t (&o)[NB][4]) {
  uint32_t a0[NB], a1[NB], a2[NB], a3[NB];
#pragma unroll
  for (int q = 0; q < NB; ++q) { a0[q] = (uint32_t)blk[q]; a1[q] = (uint32_t)(blk[q] >> 32); a2[q] = 0u; a3[q] = 0u; }
#pragma unroll
  for (int r = 0; r < kPhiloxRounds; ++r) {
#pragma unroll
    for (int q = 0; q < NB; ++q) {
      const uint64_t p0 = (uint64_t)0xD2511F53u * a0[q];
      const uint64_t p1 = (uint64_t)0xCD9E8D57u * a2[q];
      const uint32_t n0 = (uint32_t)(p1 >> 32) ^ a1[q] ^ key[2 * r];
      const uint32_t n2 = (uint32_t)(p0 >> 32) ^ a3[q] ^ key[2 * r + 1];
      a1[q] = (uint32_t)p1;
      a3[q] = (uint32_t)p0;
      a0[q] = n0;
      a2[q] = n2;
    }
  }
#pragma unroll
  for (int q = 0; q < NB; ++q) { o[q][0] = a0[q]; o[q][1] = a1[q]; o[q][2] = a2[q]; o[q][3] = a3[q]; }
}
// Keep decision of the single element `idx` (global element index).
__device__ __forceinline__ bool philox_keep(unsigned long long idx, const uint32_t* key, uint32_t thr) {
  uint32_t o[4];
  philox_block((uint32_t)(idx >> 3), (uint32_t)(idx >> 35), key, o);
  const uint32_t el = (uint32_t)(idx & 7ull);
  const uint32_t word = (el >> 1) == 0 ? o[0] : (el >> 1) == 1 ? o[1] : (el >> 1) == 2 ? o[2] : o[3];
  return ((word >> (16u * (el & 1u))) & 0x7FFFu) >= thr;
}
#endif

}  // namespace tfb
