// Pieces shared by the two attention kernels (one Q block per CTA with tile lists; two Q blocks per CTA, dense):
// tile geometry, launch parameters, and the per-row softmax arithmetic.
#pragma once
#include "../../include/ksana_b200.h"
#include "common.cuh"

namespace ksb {
namespace attn {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int UMMA_K = 32;
constexpr int KST = 2, VST = 2;
constexpr int TILE_BYTES = 128 * 128;
constexpr int THREADS = 256;
constexpr int TMEM_COLS = 256;  // S: columns 0..127 (s32), O: columns 128..255 (f32)
constexpr int KERNEL_ID = 2;
constexpr float S_MAGIC = 12582912.0f;  // 1.5 * 2^23 = 0x4B400000: one ulp is 1 on [2^23, 2^24)
constexpr float REF_SLACK = 3.5f;  // a row's reference point moves only when its maximum exceeds it by more than this
constexpr float P_SHIFT = 5.0f;  // P carries a static factor 2^5 into e4m3: at most 2^(5 + REF_SLACK) = 362 is ever rounded
constexpr int PST = 2;  // P buffers: P of tile g goes to buffer g & 1, so it never waits for the previous P.V
constexpr int NUM_BARS = 16;
// Q | P x PST | K x KST | V x VST | barriers.  The dynamic shared memory window itself must be 1024-byte aligned
// (checked at kernel start): with two CTAs per SM there is no room for alignment slack.
constexpr int NUM_TILES = 1 + PST + KST + VST;
constexpr int CONST_BYTES = 768;  // two 384-byte blocks of repeated 16-byte chunks: A and B of the accumulator pre-load MMA
constexpr int SMEM_BYTES = NUM_TILES * TILE_BYTES + CONST_BYTES + 8 * NUM_BARS + 64;

struct Params {
  const float* qs;
  const float* ks;
  const float* vs;
  int H, Lq, Lk, nq, nkv;
  const int32_t* offsets;
  const int32_t* entries;
  const int32_t* order;  // optional permutation of the Q blocks of a head (longest list first)
  void* out;
  int64_t out_ts, out_hs;
  int* status;
  // optional fused exchange: output row l goes to peers[l / rows_per_peer], row l % rows_per_peer
  void* peers[KSB_MAX_PEERS];
  int n_peers;
  int rows_per_peer;
};

struct Work {
  int h, qt, n;
  const int32_t* ents;
};

__device__ __forceinline__ Work get_work(const Params& p, int idx) {
  Work w;
  w.h = idx / p.nq;
  w.qt = idx - w.h * p.nq;
  if (p.order) w.qt = p.order[w.qt];
  if (p.offsets) {
    const int a = p.offsets[w.qt], b = p.offsets[w.qt + 1];
    w.n = b - a;
    w.ents = p.entries + a;
  } else {
    w.n = p.nkv;
    w.ents = nullptr;
  }
  return w;
}
__device__ __forceinline__ int entry_at(const Work& w, int j) { return w.ents ? w.ents[j] : (j * 4 + 3); }


// Max over 64 scores (as floats) held in two 32-register chunks: four independent chains, each step
// folding two new values with a three-input max.
__device__ __forceinline__ float tree_max64(const uint32_t (&a)[32], const uint32_t (&b)[32]) {
  float m0 = fmaxf(__uint_as_float(a[0]), __uint_as_float(a[1])), m1 = fmaxf(__uint_as_float(a[2]), __uint_as_float(a[3]));
  float m2 = fmaxf(__uint_as_float(b[0]), __uint_as_float(b[1])), m3 = fmaxf(__uint_as_float(b[2]), __uint_as_float(b[3]));
#pragma unroll
  for (int i = 4; i < 32; i += 4) {
    m0 = fmax3(m0, __uint_as_float(a[i]), __uint_as_float(a[i + 1]));
    m1 = fmax3(m1, __uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
    m2 = fmax3(m2, __uint_as_float(b[i]), __uint_as_float(b[i + 1]));
    m3 = fmax3(m3, __uint_as_float(b[i + 2]), __uint_as_float(b[i + 3]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = exp2(f * sc + c) for one 32-score chunk (f = 12582912 + S as fp32) -> 8 words of packed e4m3; the
// exact (unrounded) values are added into four independent packed accumulators.  A masked score holds -inf
// and yields 0 (or 2^-126, which rounds to 0 and vanishes in the row sum).
__device__ __forceinline__ void exp_chunk(const uint32_t (&s)[32], float sc, float c, uint32_t* pk, float2 (&acc)[4]) {
  const float2 sc2 = make_float2(sc, sc), c2 = make_float2(c, c);
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc2, c2);
    const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), sc2, c2);
    const float2 e01 = make_float2(fast_exp2(x01.x), fast_exp2(x01.y));
    const float2 e23 = make_float2(fast_exp2(x23.x), fast_exp2(x23.y));
    acc[(i >> 2) & 3] = __fadd2_rn(acc[(i >> 2) & 3], e01);
    acc[((i >> 2) + 2) & 3] = __fadd2_rn(acc[((i >> 2) + 2) & 3], e23);
    pk[i >> 2] = cvt_e4m3x4(e01.x, e01.y, e23.x, e23.y);
  }
}


}  // namespace attn
}  // namespace ksb
