// HBM-bound pre-passes of the Sage-style attention: K token-mean (smoothing vector), per-block INT8
// quantisation of Q and K, per-(head, channel) FP8 quantisation of V with the token axis made
// contiguous.  Inputs are [L, H, 128] half tensors addressed by element strides, so they can be views
// into a fused QKV projection output.
//
// Algorithmic bytes per token and head (D = 128): Q or K quantiser 256 read + 128 written;
// K mean 256 read; V quantiser 2 x 256 read + 128 written.
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace prep {

constexpr int D = 128;
constexpr int THREADS = 256;
constexpr int MEAN_CHUNK = 512;  // tokens per CTA in the mean / amax passes

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const T* t = reinterpret_cast<const T*>(&a);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = HalfOps<T>::to_f(t[i]);
}

// ---------------------------------------------------------------------------------- K mean / V amax
// grid (chunks, H).  256 threads = 16 token lanes x 16 column groups of 8 channels.
template <typename T, bool IS_MAX>
__global__ void __launch_bounds__(THREADS) column_reduce_kernel(const T* __restrict__ x, int64_t L, int64_t ts, int64_t hs,
                                                                 float* __restrict__ out, int H) {
  __shared__ float red[16][D + 1];
  const int h = blockIdx.y, chunk = blockIdx.x;
  const int tl = threadIdx.x >> 4, cg = threadIdx.x & 15;
  const int64_t l0 = (int64_t)chunk * MEAN_CHUNK;
  const int64_t l1 = min(L, l0 + MEAN_CHUNK);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int64_t l = l0 + tl; l < l1; l += 16) {
    float f[8];
    load8<T>(x + l * ts + (int64_t)h * hs + cg * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = IS_MAX ? fmaxf(acc[i], fabsf(f[i])) : acc[i] + f[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[tl][cg * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < D) {
    float r = red[0][threadIdx.x];
#pragma unroll
    for (int j = 1; j < 16; ++j) r = IS_MAX ? fmaxf(r, red[j][threadIdx.x]) : r + red[j][threadIdx.x];
    if (IS_MAX) {
      // non-negative floats order like their bit patterns
      atomicMax(reinterpret_cast<int*>(out) + h * D + threadIdx.x, __float_as_int(r));
    } else {
      out[((int64_t)chunk * H + h) * D + threadIdx.x] = r;  // partial sums [chunk][h][d]
    }
  }
}

__global__ void mean_finish_kernel(const float* __restrict__ partial, int chunks, int HD, float inv_L, float* __restrict__ km) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= HD) return;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += partial[(int64_t)c * HD + i];
  km[i] = s * inv_L;
}

// ---------------------------------------------------------------------------------- INT8 block quantiser
// grid (Lpad / BLOCK, H).  A block of BLOCK tokens x 128 channels lives in registers between the
// absmax reduction and the quantisation.
template <typename T, int BLOCK>
__global__ void __launch_bounds__(BLOCK * 4, BLOCK == 128 ? 3 : 6) int8_block_quant_kernel(const T* __restrict__ x, int64_t L, int64_t ts, int64_t hs,
                                                                    float premul, const float* __restrict__ mean,
                                                                    int8_t* __restrict__ out, float* __restrict__ scale,
                                                                    int64_t Lpad) {
  constexpr int NT = BLOCK * 4;             // four threads per token: 512 threads for Q blocks, 256 for K blocks
  constexpr int VEC = BLOCK * D / 8 / NT;   // 4 sixteen-byte vectors per thread
  __shared__ float red[NT / 32];
  const int h = blockIdx.y, b = blockIdx.x;
  const int64_t l0 = (int64_t)b * BLOCK;
  // The block stays in registers in its packed form (16 registers, not 32 of fp32) and is unpacked in both
  // passes: the lower register count lets a third (sixth) CTA share the SM, which hides the load latency of
  // these single-shot CTAs better than saving the second unpack would.
  uint4 raw[VEC];
  const int c = (threadIdx.x & 15) * 8;     // NT is a multiple of 16: the same 8 channels in every vector of a thread
  float mu[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) mu[e] = mean ? mean[h * D + c + e] : 0.f;
  auto value = [&](const uint4& r, float (&f)[8]) {
    const T* t = reinterpret_cast<const T*>(&r);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = HalfOps<T>::to_f(t[e]);
      if (mean) v = v - mu[e];
      if (premul != 0.f) v = v * premul;
      f[e] = v;
    }
  };
  float am = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int j = threadIdx.x + i * NT;
    const int64_t l = l0 + (j >> 4);
    raw[i] = (l < L) ? *reinterpret_cast<const uint4*>(x + l * ts + (int64_t)h * hs + c) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int j = threadIdx.x + i * NT;
    if (l0 + (j >> 4) < L) {
      float f[8];
      value(raw[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) am = fmaxf(am, fabsf(f[e]));
    }
  }
  am = warp_max(am);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
  __syncthreads();
  am = red[0];
#pragma unroll
  for (int i = 1; i < NT / 32; ++i) am = fmaxf(am, red[i]);
  const float sc = (am > 0.f) ? __fdiv_rn(am, 127.f) : 1.f;
  const float inv = (am > 0.f) ? __fdiv_rn(127.f, am) : 1.f;
  if (threadIdx.x == 0) scale[(int64_t)h * (Lpad / BLOCK) + b] = sc;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int j = threadIdx.x + i * NT;
    const int r = j >> 4;
    float f[8];
    if (l0 + r < L) {
      value(raw[i], f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;  // padding rows quantise to 0 whatever the mean
    }
    // round-half-even to an integer without a conversion instruction: adding 1.5 * 2^23 leaves the two's
    // complement integer in the low mantissa bits (|x * inv| <= 127 * (1 + 2^-23) by construction, so the
    // clamp to +-127 can never bind); the low bytes of four sums are gathered with byte permutes
    uint32_t t[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) t[e] = __float_as_uint(__fadd_rn(__fmul_rn(f[e], inv), 12582912.f));
    uint32_t w[2];
#pragma unroll
    for (int g = 0; g < 2; ++g)
      w[g] = __byte_perm(__byte_perm(t[4 * g], t[4 * g + 1], 0x0040), __byte_perm(t[4 * g + 2], t[4 * g + 3], 0x0040), 0x5410);
    *reinterpret_cast<uint2*>(out + ((int64_t)h * Lpad + l0 + r) * D + c) = make_uint2(w[0], w[1]);
  }
}

// ---------------------------------------------------------------------------------- V quantiser + transpose
// grid (Lpad / 128, H): tile of 128 tokens x 128 channels -> vt[h][d][l0 .. l0+127] e4m3.
// A thread quantises 4 consecutive tokens of 8 channels and writes one 32-bit word per channel into a
// [channel][token] tile in shared memory whose 16-byte groups are XOR-swizzled by the channel group, so that
// both the word writes and the 128-bit row reads are (almost) conflict free.
template <typename T>
__global__ void __launch_bounds__(THREADS) v_quant_transpose_kernel(const T* __restrict__ v, int64_t L, int64_t ts, int64_t hs,
                                                                     const float* __restrict__ amax, uint8_t* __restrict__ vt,
                                                                     float* __restrict__ vs, int64_t Lpad) {
  __shared__ __align__(16) uint32_t tile[D][32];  // [d][token / 4]
  __shared__ float s_inv[D];
  const int h = blockIdx.y;
  const int64_t l0 = (int64_t)blockIdx.x * 128;
  if (threadIdx.x < D) {
    const float a = amax[h * D + threadIdx.x];
    s_inv[threadIdx.x] = (a > 0.f) ? __fdiv_rn(448.f, a) : 1.f;
    if (blockIdx.x == 0) vs[h * D + threadIdx.x] = (a > 0.f) ? __fdiv_rn(a, 448.f) : 1.f;
  }
  __syncthreads();
  const int cg = threadIdx.x & 15, tq0 = threadIdx.x >> 4;  // 16 channel groups x 16 token quads per pass
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int tq = tq0 + 16 * pass;
    float f[4][8];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t l = l0 + tq * 4 + r;
      if (l < L) {
        load8<T>(v + l * ts + (int64_t)h * hs + cg * 8, f[r]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[r][e] = 0.f;
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float inv = s_inv[cg * 8 + e];
      const uint32_t w = cvt_e4m3x4(__fmul_rn(f[0][e], inv), __fmul_rn(f[1][e], inv), __fmul_rn(f[2][e], inv), __fmul_rn(f[3][e], inv));
      tile[cg * 8 + e][tq ^ ((cg & 7) << 2)] = w;
    }
  }
  __syncthreads();
  // 128 rows (d) x 128 bytes: 8 x 16-byte stores per row
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int j = threadIdx.x + i * THREADS;
    const int d = j >> 3, c = j & 7;
    const uint4 val = *reinterpret_cast<const uint4*>(&tile[d][(c ^ ((d >> 3) & 7)) << 2]);
    *reinterpret_cast<uint4*>(vt + ((int64_t)h * D + d) * Lpad + l0 + c * 16) = val;
  }
}

// ---------------------------------------------------------------------------------- RMSNorm (+ RoPE) in place
// RMSNorm over all C = H*128 channels (or over each head's 128) with an fp32 weight, optionally followed by
// the 3-axis rotary embedding, applied in place to a [L, C] half view (row stride ld).  A row is owned by
// the 4 warps of a CTA (one 128-bit vector of 8 channels per thread and step), read once, held in registers
// in packed form across the sum-of-squares reduction, and written once; many CTAs share an SM.
// Rounding points follow the eager sequence: norm output rounded to half, rotation computed in fp32
// (the eager path uses fp64) and rounded to half.
constexpr int NR_THREADS = 128;
constexpr int NR_MAX_VEC = 8;  // C <= 128 * 8 * 8 = 8192

struct RopeGrid {
  const float2* table;  // [table_len][64] (cos, sin); pair p of a head uses axis f for p < nf, then h, then w
  int table_len, nf, nh;
  int F, Hh, Ww;
  int64_t pos0;  // global index of row 0 (sequence-parallel shard offset)
  int diag;      // 1: one running position drives all three axes (text tokens of the Qwen-Image block)
};

struct PeerTables {
  float* p[KSB_MAX_PEERS];
};

// rstd[which][rank * M + m] = rsqrt(sum over the tiles of `which` of tile_sumsq[tile][m] / C + eps), written into
// every peer's table (plain peer stores).
__global__ void rstd_scatter_kernel(const float* __restrict__ tile_sumsq, int tiles_per_which, int M, int C, float eps,
                                    PeerTables peers, int n_peers, int rank) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * M) return;
  const int which = i / M, m = i - which * M;
  float s = 0.f;
  for (int t = 0; t < tiles_per_which; ++t) s += tile_sumsq[(int64_t)(which * tiles_per_which + t) * M + m];
  const float r = rsqrtf(s / (float)C + eps);
  const int64_t L_all = (int64_t)n_peers * M;
  for (int d = 0; d < n_peers; ++d) peers.p[d][which * L_all + (int64_t)rank * M + m] = r;
}

// x = q * d + r for 0 <= x < 2^24 (exact in fp32): the estimate from the reciprocal is within one of the quotient
__device__ __forceinline__ void divmod_small(int x, int d, float inv_d, int& q, int& r) {
  q = static_cast<int>(static_cast<float>(x) * inv_d);
  r = x - q * d;
  if (r < 0) { r += d; --q; } else if (r >= d) { r -= d; ++q; }
}

// (a, b) rotated by (cos, sin): the operation order both norm/RoPE kernels share, so that their results are the same bits
__device__ __forceinline__ float2 rope_pair(float a, float b, float2 cs) {
  return __ffma2_rn(make_float2(-b, b), make_float2(cs.y, cs.x), __fmul2_rn(make_float2(a, a), cs));
}

template <typename T, bool ROPE, bool PER_HEAD, int NV>
__global__ void __launch_bounds__(NR_THREADS, NV <= 5 ? 6 : 4) rmsnorm_rope_kernel(T* __restrict__ x, int64_t L, int C, int64_t ld,
                                                                     const float* __restrict__ w, float eps, RopeGrid rg,
                                                                     const float* __restrict__ row_rstd) {
  __shared__ float red[2][NR_THREADS / 32];
  const int nvec = C / 8;
  int par = 0;
  for (int64_t l = blockIdx.x; l < L; l += gridDim.x, par ^= 1) {
    T* row = x + l * ld;
    uint4 cur[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int j = threadIdx.x + i * NR_THREADS;
      cur[i] = (j < nvec) ? *reinterpret_cast<const uint4*>(row + j * 8) : make_uint4(0, 0, 0, 0);
    }
    float rstd_v[NV];
    if (PER_HEAD) {
      // each head's 128 channels = 16 consecutive 8-channel vectors = 16 consecutive lanes
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const T* t = reinterpret_cast<const T*>(&cur[i]);
        float hs = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float f = HalfOps<T>::to_f(t[e]);
          hs = __fmaf_rn(f, f, hs);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) hs += __shfl_xor_sync(0xffffffffu, hs, o);
        rstd_v[i] = rsqrtf(hs / (float)D + eps);
      }
    } else if (row_rstd) {
      const float r = row_rstd[l];
#pragma unroll
      for (int i = 0; i < NV; ++i) rstd_v[i] = r;
    } else {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const T* t = reinterpret_cast<const T*>(&cur[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float f = HalfOps<T>::to_f(t[e]);
          ss += f * f;
        }
      }
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red[par][threadIdx.x >> 5] = ss;
      __syncthreads();
      const float r = rsqrtf((red[par][0] + red[par][1] + red[par][2] + red[par][3]) / (float)C + eps);
#pragma unroll
      for (int i = 0; i < NV; ++i) rstd_v[i] = r;
    }
    int cf = 0, ch = 0, cw = 0;
    bool rotate = false;
    if (ROPE) {
      const int64_t pos = rg.pos0 + l;
      const int64_t per_frame = (int64_t)rg.Hh * rg.Ww;
      if (pos < (int64_t)rg.F * per_frame) {
        rotate = true;
        cf = (int)(pos / per_frame);
        const int rem = (int)(pos - (int64_t)cf * per_frame);
        ch = rem / rg.Ww;
        cw = rem - ch * rg.Ww;
        if (rg.diag) ch = cw = cf;
      }
    }
    // A thread's vectors are 1024 channels (8 heads) apart, so they all cover the same four rotation pairs of
    // their heads: the (cos, sin) entries -- and a per-head weight -- are fetched once per row, not per vector.
    static_assert((NR_THREADS * 8) % D == 0, "a thread's vectors must fall on the same channels of their heads");
    const int p0 = ((threadIdx.x * 8) & (D - 1)) >> 1;
    float2 rot[4];
    if (ROPE && rotate) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int pr = p0 + q;
        const int coord = pr < rg.nf ? cf : (pr < rg.nf + rg.nh ? ch : cw);
        rot[q] = rg.table[(int64_t)coord * 64 + pr];
      }
    }
    float wh[8];
    if (PER_HEAD) {
      const float4 w0 = *reinterpret_cast<const float4*>(w + 2 * p0), w1 = *reinterpret_cast<const float4*>(w + 2 * p0 + 4);
      wh[0] = w0.x; wh[1] = w0.y; wh[2] = w0.z; wh[3] = w0.w; wh[4] = w1.x; wh[5] = w1.y; wh[6] = w1.z; wh[7] = w1.w;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int j = threadIdx.x + i * NR_THREADS;
      if (j < nvec) {
        const T* t = reinterpret_cast<const T*>(&cur[i]);
        float wv[8];
        if (PER_HEAD) {
#pragma unroll
          for (int e = 0; e < 8; ++e) wv[e] = wh[e];
        } else {
          const float4 w0 = *reinterpret_cast<const float4*>(w + j * 8), w1 = *reinterpret_cast<const float4*>(w + j * 8 + 4);
          wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
        }
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = HalfOps<T>::to_f(HalfOps<T>::from_f(HalfOps<T>::to_f(t[e]) * rstd_v[i] * wv[e]));
        if (ROPE && rotate) {
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float2 yr = rope_pair(y[e], y[e + 1], rot[e >> 1]);
            y[e] = yr.x;
            y[e + 1] = yr.y;
          }
        }
        uint4 o;
        T* ot = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int e = 0; e < 8; ++e) ot[e] = HalfOps<T>::from_f(y[e]);
        *reinterpret_cast<uint4*>(row + j * 8) = o;
      }
    }
  }
}

// ---------------------------------------------------------------------------------- norm + RoPE inside the quantisers
// The same RMSNorm (+ rotary embedding) as rmsnorm_rope_kernel, applied to a tile of 128 tokens x one head as it is
// read by a quantiser, so that the normalised tensor is never written: Q is read once, K twice (its column means
// first).  The 1 / rms of a token over all heads comes from a table (written from the producing GEMM's per-tile sums
// of squares, or by another rank under the fused exchange); with PER_HEAD it is taken over the head's own 128
// channels, which the 16 lanes holding a token's vectors reduce among themselves.  The rounding points are those of
// the in-place kernel (norm output rounded to half, rotation in fp32, rounded to half), so the bytes are the same as
// running that kernel and then the plain quantiser with the same table.
struct NormSpec {
  const float* w;         // norm weight: [H * 128], or [128] with per_head
  const float* row_rstd;  // [L]; unused with per_head
  float eps;
  RopeGrid rg;            // rg.table == nullptr: no rotation
  int per_frame;          // rg.Hh * rg.Ww, with the reciprocals the position decoding uses
  float inv_per_frame, inv_w;
};

constexpr int NQ_THREADS = 512;  // 32 token lanes x 16 column groups of 8 channels; 4 vectors per thread

// Loads the thread's four vectors of tile (l0, h) and replaces them by the normalised (and rotated) values; rows
// at or past nvalid (the tile's share of L) come back as zeros.  VIS(i, q, v) is called with every pair of final
// values (as fp32, already rounded to half) of valid rows, while they are still in registers.
template <typename T, bool PER_HEAD, typename Visitor>
__device__ __forceinline__ void load_normed_tile(const T* __restrict__ x, int nvalid, int64_t ts, int64_t hs, int h, int64_t l0,
                                                 const NormSpec& ns, uint4 (&raw)[4], Visitor&& vis) {
  const int lane = threadIdx.x & 31;
  const int cg = threadIdx.x & 15, tl = threadIdx.x >> 4;
  const int c = cg * 8;
  const T* xp = x + (l0 + tl) * ts + (int64_t)h * hs + c;
#pragma unroll
  for (int i = 0; i < 4; ++i) raw[i] = (tl + 32 * i < nvalid) ? *reinterpret_cast<const uint4*>(xp + 32 * i * ts) : make_uint4(0, 0, 0, 0);
  float rstd[4];
  if (!PER_HEAD) {
#pragma unroll
    for (int i = 0; i < 4; ++i) rstd[i] = (tl + 32 * i < nvalid) ? ns.row_rstd[l0 + tl + 32 * i] : 0.f;
  }
  float2 w2[4];
  {
    const float* wp = ns.w + (PER_HEAD ? 0 : h * D) + c;
    const float4 w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + 4);
    w2[0] = make_float2(w0.x, w0.y); w2[1] = make_float2(w0.z, w0.w); w2[2] = make_float2(w1.x, w1.y); w2[3] = make_float2(w1.z, w1.w);
  }
  // Grid coordinates of the four tokens: the 16 lanes that share a token would all decode the same position, so lane
  // cg decodes the token of vector (cg & 3) and the group exchanges the results (packed 10 bits per axis; -1: the
  // token lies past the grid and is not rotated).
  const int p0 = c >> 1;  // first of the four rotation pairs of these 8 channels
  int packed = -1;
  bool ax_f[4], ax_h[4];  // which axis drives pair p0 + q: fixed per thread
  if (ns.rg.table) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      ax_f[q] = p0 + q < ns.rg.nf;
      ax_h[q] = p0 + q < ns.rg.nf + ns.rg.nh;
    }
    const int pos = static_cast<int>(ns.rg.pos0 + l0) + tl + 32 * (cg & 3);
    int cf, rem, ch, cw;
    divmod_small(pos, ns.per_frame, ns.inv_per_frame, cf, rem);
    divmod_small(rem, ns.rg.Ww, ns.inv_w, ch, cw);
    if (ns.rg.diag) ch = cw = cf;
    if (cf < ns.rg.F) packed = cf | (ch << 10) | (cw << 20);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t* wd = reinterpret_cast<const uint32_t*>(&raw[i]);
    float2 f[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) f[q] = HalfOps<T>::unpack2(wd[q]);
    float r;
    if (PER_HEAD) {
      float hsum = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        hsum = __fmaf_rn(f[q].x, f[q].x, hsum);
        hsum = __fmaf_rn(f[q].y, f[q].y, hsum);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) hsum += __shfl_xor_sync(0xffffffffu, hsum, o);  // every lane takes part, also past L
      r = rsqrtf(hsum / (float)D + ns.eps);
    } else {
      r = rstd[i];
    }
    int coords = -1;
    if (ns.rg.table) coords = __shfl_sync(0xffffffffu, packed, (lane & 16) | i);  // uniform branch: every lane takes part
    if (tl + 32 * i >= nvalid) continue;
    const float2 r2 = make_float2(r, r);
    float2 y[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) y[q] = HalfOps<T>::unpack2(HalfOps<T>::pack2(__fmul2_rn(__fmul2_rn(f[q], r2), w2[q])));  // norm output, rounded to half
    if (coords >= 0) {
      const int cf = coords & 1023, ch = (coords >> 10) & 1023, cw = coords >> 20;
      // pairs p0 .. p0+3 as two 16-byte table reads; a pair whose axis differs from its neighbour's is fetched on its own
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int pr = p0 + 2 * hf;
        const int c0 = ax_f[2 * hf] ? cf : (ax_h[2 * hf] ? ch : cw);
        const int c1 = ax_f[2 * hf + 1] ? cf : (ax_h[2 * hf + 1] ? ch : cw);
        const float4 t4 = *reinterpret_cast<const float4*>(ns.rg.table + c0 * 64 + pr);
        float2 cs1 = make_float2(t4.z, t4.w);
        if (c1 != c0) cs1 = ns.rg.table[c1 * 64 + pr + 1];
        y[2 * hf] = HalfOps<T>::unpack2(HalfOps<T>::pack2(rope_pair(y[2 * hf].x, y[2 * hf].y, make_float2(t4.x, t4.y))));
        y[2 * hf + 1] = HalfOps<T>::unpack2(HalfOps<T>::pack2(rope_pair(y[2 * hf + 1].x, y[2 * hf + 1].y, cs1)));
      }
    }
    uint32_t nw[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      nw[q] = HalfOps<T>::pack2(y[q]);  // exact: y is already rounded
      vis(i, q, y[q]);
    }
    raw[i] = make_uint4(nw[0], nw[1], nw[2], nw[3]);
  }
}

// Column sums of the normalised K over chunks of MEAN_CHUNK tokens: grid (chunks, H), partial[chunk][h][d].
template <typename T, bool PER_HEAD>
__global__ void __launch_bounds__(NQ_THREADS, 2) normed_colsum_kernel(const T* __restrict__ x, int64_t L, int64_t ts, int64_t hs, NormSpec ns,
                                                                       float* __restrict__ partial, int H) {
  __shared__ float red[32][D + 1];
  const int h = blockIdx.y, chunk = blockIdx.x;
  const int cg = threadIdx.x & 15, tl = threadIdx.x >> 4;
  float2 acc[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) acc[q] = make_float2(0.f, 0.f);
  for (int tile = 0; tile < MEAN_CHUNK / 128; ++tile) {
    const int64_t l0 = (int64_t)chunk * MEAN_CHUNK + tile * 128;
    if (l0 >= L) break;
    const int nvalid = (int)min((int64_t)128, L - l0);
    uint4 raw[4];
    load_normed_tile<T, PER_HEAD>(x, nvalid, ts, hs, h, l0, ns, raw, [&](int, int q, float2 v) { acc[q] = __fadd2_rn(acc[q], v); });
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    red[tl][cg * 8 + 2 * q] = acc[q].x;
    red[tl][cg * 8 + 2 * q + 1] = acc[q].y;
  }
  __syncthreads();
  if (threadIdx.x < D) {
    float r = red[0][threadIdx.x];
#pragma unroll
    for (int j = 1; j < 32; ++j) r += red[j][threadIdx.x];
    partial[((int64_t)chunk * H + h) * D + threadIdx.x] = r;
  }
}

// Norm (+ RoPE) + INT8 block quantiser over a tile of 128 tokens x one head: grid (Lpad / 128, H).
// NB = 1: one 128-token block (Q: premul, no mean); NB = 2: two 64-token blocks (K: mean subtracted).
template <typename T, int NB, bool PER_HEAD>
__global__ void __launch_bounds__(NQ_THREADS, 2) normed_int8_quant_kernel(const T* __restrict__ x, int64_t L, int64_t ts, int64_t hs, NormSpec ns,
                                                                           float premul, const float* __restrict__ mean,
                                                                           int8_t* __restrict__ out, float* __restrict__ scale, int64_t Lpad) {
  __shared__ float red[NB][NQ_THREADS / 32];
  const int h = blockIdx.y;
  const int64_t l0 = (int64_t)blockIdx.x * 128;
  const int nvalid = (int)min((int64_t)128, L - l0);
  const int cg = threadIdx.x & 15, tl = threadIdx.x >> 4;
  const int c = cg * 8;
  float2 nmu[4];  // minus the mean: x - mu and x + (-mu) are the same number
#pragma unroll
  for (int q = 0; q < 4; ++q) nmu[q] = mean ? make_float2(-mean[h * D + c + 2 * q], -mean[h * D + c + 2 * q + 1]) : make_float2(0.f, 0.f);
  const float2 pm2 = make_float2(premul, premul);
  auto value = [&](float2 v, int q) -> float2 {
    if (mean) v = __fadd2_rn(v, nmu[q]);
    if (premul != 0.f) v = __fmul2_rn(v, pm2);
    return v;
  };
  float am[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) am[b] = 0.f;
  uint4 raw[4];
  load_normed_tile<T, PER_HEAD>(x, nvalid, ts, hs, h, l0, ns, raw, [&](int i, int q, float2 y) {
    const float2 v = value(y, q);
    const int b = NB == 2 ? (i >> 1) : 0;  // tokens tl + 32 i: i = 0, 1 are the first 64
    am[b] = fmax3(am[b], fabsf(v.x), fabsf(v.y));
  });
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    am[b] = warp_max(am[b]);
    if ((threadIdx.x & 31) == 0) red[b][threadIdx.x >> 5] = am[b];
  }
  __syncthreads();
  float inv[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    float a = red[b][0];
#pragma unroll
    for (int i = 1; i < NQ_THREADS / 32; ++i) a = fmaxf(a, red[b][i]);
    inv[b] = (a > 0.f) ? __fdiv_rn(127.f, a) : 1.f;
    if (threadIdx.x == 0) scale[(int64_t)h * (Lpad / 128 * NB) + (int64_t)blockIdx.x * NB + b] = (a > 0.f) ? __fdiv_rn(a, 127.f) : 1.f;
  }
  // rounding by the magic addend: see int8_block_quant_kernel
  int8_t* op = out + ((int64_t)h * Lpad + l0 + tl) * D + c;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t* wd = reinterpret_cast<const uint32_t*>(&raw[i]);
    const float iv = inv[NB == 2 ? (i >> 1) : 0];
    uint32_t t[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 v = make_float2(0.f, 0.f);  // padding rows quantise to 0 whatever the mean
      if (tl + 32 * i < nvalid) v = value(HalfOps<T>::unpack2(wd[q]), q);
      // scalar on purpose: the product must be rounded before the addition (a packed multiply followed by a packed
      // add was observed to round like one fused operation, which breaks ties such as 63.5 the other way)
      t[2 * q] = __float_as_uint(__fadd_rn(__fmul_rn(v.x, iv), 12582912.f));
      t[2 * q + 1] = __float_as_uint(__fadd_rn(__fmul_rn(v.y, iv), 12582912.f));
    }
    uint32_t w[2];
#pragma unroll
    for (int g = 0; g < 2; ++g)
      w[g] = __byte_perm(__byte_perm(t[4 * g], t[4 * g + 1], 0x0040), __byte_perm(t[4 * g + 2], t[4 * g + 3], 0x0040), 0x5410);
    *reinterpret_cast<uint2*>(op + 32 * i * D) = make_uint2(w[0], w[1]);
  }
}

// rstd[g][m] = rsqrt(sum over the tiles of column group g of tile_sumsq[tile][m] / C + eps)
__global__ void rstd_finish_kernel(const float* __restrict__ tile_sumsq, int tiles_per_group, int groups, int M, int C, float eps,
                                   float* __restrict__ rstd) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= groups * M) return;
  const int g = i / M, m = i - g * M;
  float s = 0.f;
  for (int t = 0; t < tiles_per_group; ++t) s += tile_sumsq[(int64_t)(g * tiles_per_group + t) * M + m];
  rstd[i] = rsqrtf(s / (float)C + eps);
}

// ---------------------------------------------------------------------------------- built-in scratch
// Scratch of the allocation-free V quantiser entry point: per-(head, channel) absmax words.  It lives in
// the library image, so every GPU that loads the library holds these 256 KB until the process exits.
constexpr int64_t NOALLOC_MAX_HD = 65536;  // heads * 128 <= 65536, i.e. at most 512 heads
static __device__ __align__(256) float g_v_amax_scratch[NOALLOC_MAX_HD];

// In host code the array's name is only a handle: the device address has to be asked for, once per device,
// with that device current.  Returns nullptr (with the error text set) if the runtime refuses.
static float* v_amax_scratch_address() {
  static float* cached[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    fail(KSB_ERR_CUDA, "cudaGetDevice failed or device index out of range: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (!cached[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_v_amax_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fail(KSB_ERR_CUDA, "cudaGetSymbolAddress(built-in scratch) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = ptr;
  }
  return cached[dev];
}

int validate(const void* x, int dtype, int64_t L, int64_t H, int64_t Dh, int64_t ts, int64_t hs) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (Dh != D) return fail(KSB_ERR_UNSUPPORTED, "head size %lld is not supported (only 128)", (long long)Dh);
  if (L <= 0 || H <= 0 || H > 65535) return fail(KSB_ERR_INVALID, "bad shape L=%lld H=%lld", (long long)L, (long long)H);
  if (!x || !aligned16(x) || ts % 8 != 0 || hs % 8 != 0) return fail(KSB_ERR_INVALID, "input must be 16-byte aligned with strides multiple of 8 elements");
  return 0;
}

// Fills a RopeGrid from the C-ABI arguments (rope_table == nullptr: no rotation).
int make_rope_grid(RopeGrid& rg, const float* rope_table, int table_len, int nf, int nh, int F, int Hh, int Ww, int64_t pos0, int diag) {
  rg = RopeGrid{};
  if (!rope_table) return 0;
  if (nf < 0 || nh < 0 || nf + nh > 64 || F <= 0 || Hh <= 0 || Ww <= 0) return fail(KSB_ERR_INVALID, "bad rope grid");
  if (F > table_len || (!diag && (Hh > table_len || Ww > table_len))) return fail(KSB_ERR_INVALID, "rope table too short for the grid");
  if (diag && (Hh != 1 || Ww != 1)) return fail(KSB_ERR_INVALID, "diag positions need a grid of (F, 1, 1)");
  if (!aligned16(rope_table)) return fail(KSB_ERR_INVALID, "rope table must be 16-byte aligned");
  rg.table = reinterpret_cast<const float2*>(rope_table); rg.table_len = table_len; rg.nf = nf; rg.nh = nh;
  rg.F = F; rg.Hh = Hh; rg.Ww = Ww; rg.pos0 = pos0; rg.diag = diag ? 1 : 0;
  return 0;
}

int make_norm_spec(NormSpec& ns, int64_t L, const float* norm_w, int per_head, const float* row_rstd, float eps, const float* rope_table,
                   int table_len, int nf, int nh, int F, int Hh, int Ww, int64_t pos0, int diag) {
  if (!norm_w || !aligned16(norm_w)) return fail(KSB_ERR_INVALID, "norm weight null or unaligned");
  if (!per_head && !row_rstd) return fail(KSB_ERR_INVALID, "a norm over all heads needs the row_rstd table");
  ns.w = norm_w; ns.row_rstd = per_head ? nullptr : row_rstd; ns.eps = eps;
  if (int rc = make_rope_grid(ns.rg, rope_table, table_len, nf, nh, F, Hh, Ww, pos0, diag)) return rc;
  if (rope_table) {
    if (pos0 < 0 || pos0 + L > (1 << 24)) return fail(KSB_ERR_INVALID, "token positions must stay below 2^24");
    ns.per_frame = Hh * Ww;
    ns.inv_per_frame = 1.0f / (float)ns.per_frame;
    ns.inv_w = 1.0f / (float)Ww;
  }
  return 0;
}

inline int64_t pad128(int64_t L) { return (L + 127) / 128 * 128; }

}  // namespace prep
}  // namespace ksb

using namespace ksb;

extern "C" {

int64_t ksb_sage_kmean_scratch_floats(int64_t L, int64_t H, int64_t D) {
  return ((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK) * H * D;
}

int ksb_sage_kmean(const void* k, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride, int64_t head_stride,
                   float* partial, float* km, ksb_stream_t stream) {
  if (int rc = prep::validate(k, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (!partial || !km) return fail(KSB_ERR_INVALID, "null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunks = (int)((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK);
  dim3 grid(chunks, (unsigned)H);
  if (dtype == KSB_BF16)
    prep::column_reduce_kernel<__nv_bfloat16, false><<<grid, prep::THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(k), L, token_stride, head_stride, partial, (int)H);
  else
    prep::column_reduce_kernel<__half, false><<<grid, prep::THREADS, 0, st>>>(static_cast<const __half*>(k), L, token_stride, head_stride, partial, (int)H);
  if (int rc = check_launch("k mean (partial)")) return rc;
  const int HD = (int)(H * D);
  prep::mean_finish_kernel<<<(HD + 255) / 256, 256, 0, st>>>(partial, chunks, HD, 1.0f / (float)L, km);
  return check_launch("k mean (finish)");
}


int64_t ksb_rmsnorm_rope_scratch_floats(int64_t L, int64_t C) {
  return ((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK) * C;
}

int ksb_rowsumsq_to_rstd_scatter(const float* tile_sumsq, int64_t M, int64_t C, float eps, float* const* peer_rstd,
                                 int n_peers, int rank, ksb_stream_t stream) {
  if (!tile_sumsq || !peer_rstd || M <= 0 || C <= 0 || C % 256 != 0) return fail(KSB_ERR_INVALID, "bad arguments");
  if (n_peers < 1 || n_peers > KSB_MAX_PEERS || rank < 0 || rank >= n_peers) return fail(KSB_ERR_INVALID, "bad peer count / rank");
  prep::PeerTables pt{};
  for (int i = 0; i < n_peers; ++i) {
    if (!peer_rstd[i]) return fail(KSB_ERR_INVALID, "peer table %d is null", i);
    pt.p[i] = peer_rstd[i];
  }
  const int n = (int)(2 * M);
  prep::rstd_scatter_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(tile_sumsq, (int)(C / 256), (int)M, (int)C, eps, pt, n_peers, rank);
  return check_launch("rstd scatter");
}

int ksb_rmsnorm_rope_inplace(void* x, int dtype, int64_t L, int64_t C, int64_t ld, const float* w, int per_head,
                             const float* row_rstd, float eps, const float* rope_table, int table_len, int nf, int nh, int F, int Hh, int Ww, int64_t pos0,
                             int diag, float* colsum_partial, float* colmean, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (L <= 0 || C <= 0 || C % 128 != 0 || C > prep::NR_THREADS * 8 * prep::NR_MAX_VEC) return fail(KSB_ERR_INVALID, "C=%lld must be a multiple of 128 and <= 8192", (long long)C);
  if (!x || !w || !aligned16(x) || !aligned16(w) || ld < C || ld % 8 != 0) return fail(KSB_ERR_INVALID, "x/w null, unaligned or bad row stride");
  if ((colsum_partial == nullptr) != (colmean == nullptr)) return fail(KSB_ERR_INVALID, "colsum_partial and colmean go together");
  if (row_rstd && per_head) return fail(KSB_ERR_INVALID, "row_rstd and per_head exclude each other");
  prep::RopeGrid rg{};
  if (int rc = prep::make_rope_grid(rg, rope_table, table_len, nf, nh, F, Hh, Ww, pos0, diag)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t cap = (int64_t)sm_count() * 16;
  const int blocks = (int)(L < cap ? L : cap);
  const bool wide = C > prep::NR_THREADS * 8 * 4;  // more than 4 vectors per thread
#define KSB_LAUNCH_NR(T, R, P, NV) prep::rmsnorm_rope_kernel<T, R, P, NV><<<blocks, prep::NR_THREADS, 0, st>>>(static_cast<T*>(x), L, (int)C, ld, w, eps, rg, row_rstd)
  const bool five = C > prep::NR_THREADS * 8 * 4 && C <= prep::NR_THREADS * 8 * 5;  // e.g. 5120: five vectors per thread, six CTAs per SM
#define KSB_LAUNCH_NR3(T, R, P) do { if (five) KSB_LAUNCH_NR(T, R, P, 5); else if (wide) KSB_LAUNCH_NR(T, R, P, 8); else KSB_LAUNCH_NR(T, R, P, 4); } while (0)
#define KSB_LAUNCH_NR2(T)                                                          \
  do {                                                                             \
    if (rope_table) { if (per_head) KSB_LAUNCH_NR3(T, true, true); else KSB_LAUNCH_NR3(T, true, false); } \
    else { if (per_head) KSB_LAUNCH_NR3(T, false, true); else KSB_LAUNCH_NR3(T, false, false); }           \
  } while (0)
  if (dtype == KSB_BF16) KSB_LAUNCH_NR2(__nv_bfloat16); else KSB_LAUNCH_NR2(__half);
#undef KSB_LAUNCH_NR2
#undef KSB_LAUNCH_NR3
#undef KSB_LAUNCH_NR
  if (int rc = check_launch("rmsnorm/rope")) return rc;
  if (colmean) {
    // per-channel mean of the values just written (the K smoothing vector): the column-reduction pass over x
    // seen as [L, C/128, 128]
    const int chunks = (int)((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK);
    dim3 grid(chunks, (unsigned)(C / 128));
    if (dtype == KSB_BF16)
      prep::column_reduce_kernel<__nv_bfloat16, false><<<grid, prep::THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(x), L, ld, 128, colsum_partial, (int)(C / 128));
    else
      prep::column_reduce_kernel<__half, false><<<grid, prep::THREADS, 0, st>>>(static_cast<const __half*>(x), L, ld, 128, colsum_partial, (int)(C / 128));
    if (int rc = check_launch("column sums")) return rc;
    prep::mean_finish_kernel<<<(int)((C + 255) / 256), 256, 0, st>>>(colsum_partial, chunks, (int)C, 1.0f / (float)L, colmean);
    return check_launch("column mean");
  }
  return 0;
}

int ksb_sage_quant_int8(const void* x, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride, int64_t head_stride,
                        int block, float premul, const float* mean, void* out, float* scale, ksb_stream_t stream) {
  if (int rc = prep::validate(x, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (block != 128 && block != 64) return fail(KSB_ERR_INVALID, "block must be 128 or 64");
  if (!out || !scale || !aligned16(out)) return fail(KSB_ERR_INVALID, "null or unaligned output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t Lpad = prep::pad128(L);
  dim3 grid((unsigned)(Lpad / block), (unsigned)H);
  int8_t* o = static_cast<int8_t*>(out);
#define KSB_LAUNCH_Q(T, B) prep::int8_block_quant_kernel<T, B><<<grid, B * 4, 0, st>>>(static_cast<const T*>(x), L, token_stride, head_stride, premul, mean, o, scale, Lpad)
  if (dtype == KSB_BF16) {
    if (block == 128) KSB_LAUNCH_Q(__nv_bfloat16, 128); else KSB_LAUNCH_Q(__nv_bfloat16, 64);
  } else {
    if (block == 128) KSB_LAUNCH_Q(__half, 128); else KSB_LAUNCH_Q(__half, 64);
  }
#undef KSB_LAUNCH_Q
  return check_launch("int8 block quantiser");
}

int ksb_rowsumsq_to_rstd(const float* tile_sumsq, int64_t M, int64_t C, int groups, float eps, float* rstd, ksb_stream_t stream) {
  if (!tile_sumsq || !rstd || M <= 0 || C <= 0 || C % 256 != 0 || groups < 1 || groups * M > INT32_MAX) return fail(KSB_ERR_INVALID, "bad arguments");
  const int n = (int)(groups * M);
  prep::rstd_finish_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(tile_sumsq, (int)(C / 256), groups, (int)M, (int)C, eps, rstd);
  return check_launch("rstd from tile sums");
}

int ksb_sage_kmean_normed(const void* k, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride, int64_t head_stride,
                          const float* norm_w, int per_head, const float* row_rstd, float eps, const float* rope_table, int table_len,
                          int nf, int nh, int F, int Hh, int Ww, int64_t pos0, int diag, float* partial, float* km, ksb_stream_t stream) {
  if (int rc = prep::validate(k, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (!partial || !km) return fail(KSB_ERR_INVALID, "null pointer");
  prep::NormSpec ns{};
  if (int rc = prep::make_norm_spec(ns, L, norm_w, per_head, row_rstd, eps, rope_table, table_len, nf, nh, F, Hh, Ww, pos0, diag)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunks = (int)((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK);
  dim3 grid(chunks, (unsigned)H);
#define KSB_LAUNCH_CS(T, P) prep::normed_colsum_kernel<T, P><<<grid, prep::NQ_THREADS, 0, st>>>(static_cast<const T*>(k), L, token_stride, head_stride, ns, partial, (int)H)
  if (dtype == KSB_BF16) { if (per_head) KSB_LAUNCH_CS(__nv_bfloat16, true); else KSB_LAUNCH_CS(__nv_bfloat16, false); }
  else { if (per_head) KSB_LAUNCH_CS(__half, true); else KSB_LAUNCH_CS(__half, false); }
#undef KSB_LAUNCH_CS
  if (int rc = check_launch("normed k column sums")) return rc;
  const int HD = (int)(H * D);
  prep::mean_finish_kernel<<<(HD + 255) / 256, 256, 0, st>>>(partial, chunks, HD, 1.0f / (float)L, km);
  return check_launch("k mean (finish)");
}

int ksb_sage_quant_int8_normed(const void* x, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride, int64_t head_stride,
                               int block, float premul, const float* mean, const float* norm_w, int per_head, const float* row_rstd,
                               float eps, const float* rope_table, int table_len, int nf, int nh, int F, int Hh, int Ww, int64_t pos0,
                               int diag, void* out, float* scale, ksb_stream_t stream) {
  if (int rc = prep::validate(x, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (block != 128 && block != 64) return fail(KSB_ERR_INVALID, "block must be 128 or 64");
  if (!out || !scale || !aligned16(out)) return fail(KSB_ERR_INVALID, "null or unaligned output");
  prep::NormSpec ns{};
  if (int rc = prep::make_norm_spec(ns, L, norm_w, per_head, row_rstd, eps, rope_table, table_len, nf, nh, F, Hh, Ww, pos0, diag)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t Lpad = prep::pad128(L);
  dim3 grid((unsigned)(Lpad / 128), (unsigned)H);
  int8_t* o = static_cast<int8_t*>(out);
#define KSB_LAUNCH_NQ(T, NB, P) prep::normed_int8_quant_kernel<T, NB, P><<<grid, prep::NQ_THREADS, 0, st>>>(static_cast<const T*>(x), L, token_stride, head_stride, ns, premul, mean, o, scale, Lpad)
#define KSB_LAUNCH_NQ2(T) do { if (block == 128) { if (per_head) KSB_LAUNCH_NQ(T, 1, true); else KSB_LAUNCH_NQ(T, 1, false); } \
                               else { if (per_head) KSB_LAUNCH_NQ(T, 2, true); else KSB_LAUNCH_NQ(T, 2, false); } } while (0)
  if (dtype == KSB_BF16) KSB_LAUNCH_NQ2(__nv_bfloat16); else KSB_LAUNCH_NQ2(__half);
#undef KSB_LAUNCH_NQ2
#undef KSB_LAUNCH_NQ
  return check_launch("normed int8 block quantiser");
}

int ksb_sage_quant_v_fp8(const void* v, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride, int64_t head_stride,
                         float* amax, void* vt, float* vs, ksb_stream_t stream) {
  if (int rc = prep::validate(v, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (!amax || !vt || !vs || !aligned16(vt)) return fail(KSB_ERR_INVALID, "null or unaligned output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(amax, 0, sizeof(float) * H * D, st) != cudaSuccess) return fail(KSB_ERR_CUDA, "memset failed");
  const int chunks = (int)((L + prep::MEAN_CHUNK - 1) / prep::MEAN_CHUNK);
  dim3 g1(chunks, (unsigned)H);
  const int64_t Lpad = prep::pad128(L);
  dim3 g2((unsigned)(Lpad / 128), (unsigned)H);
  if (dtype == KSB_BF16) {
    prep::column_reduce_kernel<__nv_bfloat16, true><<<g1, prep::THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(v), L, token_stride, head_stride, amax, (int)H);
    if (int rc = check_launch("v absmax")) return rc;
    prep::v_quant_transpose_kernel<__nv_bfloat16><<<g2, prep::THREADS, 0, st>>>(static_cast<const __nv_bfloat16*>(v), L, token_stride, head_stride, amax, static_cast<uint8_t*>(vt), vs, Lpad);
  } else {
    prep::column_reduce_kernel<__half, true><<<g1, prep::THREADS, 0, st>>>(static_cast<const __half*>(v), L, token_stride, head_stride, amax, (int)H);
    if (int rc = check_launch("v absmax")) return rc;
    prep::v_quant_transpose_kernel<__half><<<g2, prep::THREADS, 0, st>>>(static_cast<const __half*>(v), L, token_stride, head_stride, amax, static_cast<uint8_t*>(vt), vs, Lpad);
  }
  return check_launch("v quantiser");
}

int ksb_sage_quant_v_fp8_noalloc(const void* v, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                                 int64_t head_stride, void* vt, float* vs, ksb_stream_t stream) {
  if (int rc = prep::validate(v, dtype, L, H, D, token_stride, head_stride)) return rc;
  if (H * D > prep::NOALLOC_MAX_HD)
    return fail(KSB_ERR_INVALID, "ksb_sage_quant_v_fp8_noalloc: heads * head_size = %lld exceeds the built-in scratch of %lld words; "
                "use ksb_sage_quant_v_fp8 with caller-provided scratch", (long long)(H * D), (long long)prep::NOALLOC_MAX_HD);
  float* amax = prep::v_amax_scratch_address();  // first call on a device resolves the address
  if (!amax) return KSB_ERR_CUDA;
  // same two passes as ksb_sage_quant_v_fp8; the absmax words are cleared first because the array keeps
  // whatever the previous call left in it
  return ksb_sage_quant_v_fp8(v, dtype, L, H, D, token_stride, head_stride, amax, vt, vs, stream);
}

}  // extern "C"
