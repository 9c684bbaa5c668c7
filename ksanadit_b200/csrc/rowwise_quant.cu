// HBM-bound row kernels: per-token FP8 (e4m3) activation quantiser, alone or fused behind
// LayerNorm + adaLN modulate / affine LayerNorm.  A row is owned by 1, 2 or 4 warps (by its width), read
// once from HBM with 2 x 128-bit loads per 16 elements, held in registers across the reductions, and
// written once (16 e4m3 bytes per 128-bit store); a CTA of 4 warps keeps up to 4 rows in flight and many
// CTAs share an SM.  Algorithmic bytes per row: 2K (read) + K (write) + 4 (scale).
//
// Rounding points follow the eager PyTorch sequence this replaces, so the FP8 bytes match it bit for
// bit: s = amax/448 (fp32 divide), inv = half(1/s), q = e4m3(half(x * inv)).
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace rq {

constexpr int THREADS = 128;   // 4 warps per CTA; a row is owned by 1, 2 or 4 of them
constexpr int CHUNK = 16;      // elements per thread-chunk: two 128-bit loads, one 128-bit e4m3 store
// chunks per thread (NC) is 4 or 8: K <= warps_per_row * 32 * 16 * NC

enum Mode : int { PLAIN = 0, ADALN = 1, LN_AFFINE = 2, STATIC = 3 };

struct Params {
  const void* x;
  int64_t M, K, ldx;
  const void* shift;  // ADALN
  const void* scale;  // ADALN
  int64_t mod_rows;
  int round_product;  // ADALN: 0 = addcmul(shift, ln, 1+scale) (one rounding), 1 = ln * (1+scale) rounded, then + shift
  const float* w;  // LN_AFFINE
  const float* b;
  float eps;
  const float* scale_input;  // STATIC (may be null = clamp only)
  void* h_out;               // optional half copy of the transformed row
  uint8_t* q;
  float* qscale;
};

template <typename T> __device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float (&f)[16]) {
  const T* ta = reinterpret_cast<const T*>(&a);
  const T* tb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[i] = HalfOps<T>::to_f(ta[i]);
    f[8 + i] = HalfOps<T>::to_f(tb[i]);
  }
}
template <typename T> __device__ __forceinline__ void pack16(const float (&f)[16], uint4& a, uint4& b) {
  T* ta = reinterpret_cast<T*>(&a);
  T* tb = reinterpret_cast<T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ta[i] = HalfOps<T>::from_f(f[i]);
    tb[i] = HalfOps<T>::from_f(f[8 + i]);
  }
}
template <typename T> __device__ __forceinline__ float round_half(float v) { return HalfOps<T>::to_f(HalfOps<T>::from_f(v)); }

// Reduction over the WPR warps that own one row.  `red` is [2][4] floats per CTA, double-buffered by `par`.
template <int WPR, bool IS_MAX> __device__ __forceinline__ float row_reduce(float v, float* red, int par, int warp) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (WPR == 1) return v;
  if ((threadIdx.x & 31) == 0) red[par * 4 + warp] = v;
  __syncthreads();
  const int g0 = (warp / WPR) * WPR;
  float r = red[par * 4 + g0];
#pragma unroll
  for (int i = 1; i < WPR; ++i) r = IS_MAX ? fmaxf(r, red[par * 4 + g0 + i]) : r + red[par * 4 + g0 + i];
  return r;
}

// Rows are kept in registers in their packed half form between the HBM read and the HBM write.  With a
// broadcast modulation (mod_rows == 1) the shift and (1 + scale) vectors, or the affine weight and bias, are
// staged once per CTA in shared memory.
template <typename T, int MODE, int WPR, int MAX_CHUNKS>
__global__ void __launch_bounds__(THREADS, 4) rowwise_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[3][2][4];
  constexpr int RPC = 4 / WPR;          // rows per CTA per iteration
  constexpr int GT = WPR * 32;          // threads per row
  const int warp = threadIdx.x >> 5;
  const int rg = warp / WPR;            // row slot of this warp
  const int t = threadIdx.x - rg * GT;  // thread index inside the row group
  const int nchunks = static_cast<int>(p.K / CHUNK);
  const T* x = static_cast<const T*>(p.x);
  const bool staged = (MODE == ADALN && p.mod_rows == 1) || MODE == LN_AFFINE;
  // Staged vectors are stored as 16-byte units in unit-major order (unit u of chunk ch at index u * nchunks + ch),
  // so that consecutive threads, which own consecutive chunks, read consecutive 16-byte units: no bank conflicts.
  if (MODE == ADALN && staged) {
    uint4* s_shift = reinterpret_cast<uint4*>(smem);       // [2][nchunks] units of 8 halves
    uint4* s_tsc = s_shift + 2 * nchunks;
    for (int i = threadIdx.x; i < 2 * nchunks; i += THREADS) {
      const int ch = i >> 1, u = i & 1;
      const uint4 sh = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.shift) + ch * CHUNK + u * 8);
      uint4 sc = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.scale) + ch * CHUNK + u * 8);
      T* st = reinterpret_cast<T*>(&sc);
#pragma unroll
      for (int e = 0; e < 8; ++e) st[e] = HalfOps<T>::from_f(1.f + HalfOps<T>::to_f(st[e]));  // (1 + scale) in half
      s_shift[u * nchunks + ch] = sh;
      s_tsc[u * nchunks + ch] = sc;
    }
    __syncthreads();
  }
  if (MODE == LN_AFFINE) {
    float4* s_w = reinterpret_cast<float4*>(smem);  // [4][nchunks] units of 4 floats
    float4* s_b = s_w + 4 * nchunks;
    for (int i = threadIdx.x; i < 4 * nchunks; i += THREADS) {
      const int ch = i >> 2, u = i & 3;
      s_w[u * nchunks + ch] = *reinterpret_cast<const float4*>(p.w + ch * CHUNK + u * 4);
      s_b[u * nchunks + ch] = p.b ? *reinterpret_cast<const float4*>(p.b + ch * CHUNK + u * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
  }
  int par = 0;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * RPC; base < p.M; base += static_cast<int64_t>(gridDim.x) * RPC, par ^= 1) {
    const int64_t row = base + rg;
    const bool live = row < p.M;
    uint4 va[MAX_CHUNKS], vb[MAX_CHUNKS];
    const T* xr = x + row * p.ldx;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
      const int ch = t + c * GT;
      if (live && ch < nchunks) {
        va[c] = *reinterpret_cast<const uint4*>(xr + ch * CHUNK);
        vb[c] = *reinterpret_cast<const uint4*>(xr + ch * CHUNK + 8);
      } else {
        va[c] = make_uint4(0, 0, 0, 0);
        vb[c] = make_uint4(0, 0, 0, 0);
      }
    }
    if (MODE == ADALN || MODE == LN_AFFINE) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        float f[16];
        unpack16<T>(va[c], vb[c], f);
#pragma unroll
        for (int i = 0; i < 16; ++i) s += f[i];
      }
      const float mean = row_reduce<WPR, false>(s, &red[0][0][0], par, warp) / static_cast<float>(p.K);
      float s2 = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        if (t + c * GT < nchunks) {
          float f[16];
          unpack16<T>(va[c], vb[c], f);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float d = f[i] - mean;
            s2 += d * d;
          }
        }
      }
      const float var = row_reduce<WPR, false>(s2, &red[1][0][0], par, warp) / static_cast<float>(p.K);
      const float rstd = rsqrtf(var + p.eps);
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        const int ch = t + c * GT;
        if (live && ch < nchunks) {
          float f[16];
          unpack16<T>(va[c], vb[c], f);
          if (MODE == ADALN) {
            float sh[16], ts[16];
            if (staged) {
              const uint4* s_shift = reinterpret_cast<const uint4*>(smem);
              const uint4* s_tsc = s_shift + 2 * nchunks;
              unpack16<T>(s_shift[ch], s_shift[nchunks + ch], sh);
              unpack16<T>(s_tsc[ch], s_tsc[nchunks + ch], ts);
            } else {
              const T* gs = static_cast<const T*>(p.shift) + row * p.K + ch * CHUNK;
              const T* gc = static_cast<const T*>(p.scale) + row * p.K + ch * CHUNK;
              unpack16<T>(*reinterpret_cast<const uint4*>(gs), *reinterpret_cast<const uint4*>(gs + 8), sh);
              unpack16<T>(*reinterpret_cast<const uint4*>(gc), *reinterpret_cast<const uint4*>(gc + 8), ts);
#pragma unroll
              for (int i = 0; i < 16; ++i) ts[i] = round_half<T>(1.f + ts[i]);  // (1 + scale) in half
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float ln = round_half<T>((f[i] - mean) * rstd);  // F.layer_norm output in half
              f[i] = p.round_product ? (round_half<T>(ln * ts[i]) + sh[i]) : fmaf(ln, ts[i], sh[i]);  // rounded once more by pack16
            }
          } else {
            const float4* s_w = reinterpret_cast<const float4*>(smem);
            const float4* s_b = s_w + 4 * nchunks;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float4 wv = s_w[u * nchunks + ch], bv = s_b[u * nchunks + ch];
              f[4 * u + 0] = (f[4 * u + 0] - mean) * rstd * wv.x + bv.x;
              f[4 * u + 1] = (f[4 * u + 1] - mean) * rstd * wv.y + bv.y;
              f[4 * u + 2] = (f[4 * u + 2] - mean) * rstd * wv.z + bv.z;
              f[4 * u + 3] = (f[4 * u + 3] - mean) * rstd * wv.w + bv.w;
            }
          }
          pack16<T>(f, va[c], vb[c]);
          if (p.h_out) {
            T* ho = static_cast<T*>(p.h_out) + row * p.K + ch * CHUNK;
            *reinterpret_cast<uint4*>(ho) = va[c];
            *reinterpret_cast<uint4*>(ho + 8) = vb[c];
          }
        }
      }
    }
    float inv_h;  // multiplier already rounded to half precision
    float row_scale;
    if (MODE == STATIC) {
      if (p.scale_input) {
        row_scale = *p.scale_input;
        inv_h = round_half<T>(__frcp_rn(row_scale));
      } else {
        row_scale = 1.f;
        inv_h = 1.f;
      }
    } else {
      float am = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        float f[16];
        unpack16<T>(va[c], vb[c], f);
#pragma unroll
        for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(f[i]));
      }
      am = row_reduce<WPR, true>(am, &red[2][0][0], par, warp);
      row_scale = (am > 0.f) ? __fdiv_rn(am, 448.f) : 1.f;
      inv_h = round_half<T>(__frcp_rn(row_scale));
    }
    if (live) {
      if (t == 0) p.qscale[row] = row_scale;
      uint8_t* qr = p.q + row * p.K;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        const int ch = t + c * GT;
        if (ch < nchunks) {
          float f[16];
          unpack16<T>(va[c], vb[c], f);
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = round_half<T>(f[i] * inv_h);  // product formed in half precision
          uint4 o;
          o.x = cvt_e4m3x4(f[0], f[1], f[2], f[3]);
          o.y = cvt_e4m3x4(f[4], f[5], f[6], f[7]);
          o.z = cvt_e4m3x4(f[8], f[9], f[10], f[11]);
          o.w = cvt_e4m3x4(f[12], f[13], f[14], f[15]);
          *reinterpret_cast<uint4*>(qr + ch * CHUNK) = o;
        }
      }
    }
  }
}

// Pair conversions: two fp32 values <-> one packed word of two halves (one conversion instruction per pair).
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float2 v) {
    __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
};
template <> struct Pair<__half> {
  static __device__ __forceinline__ uint32_t pack(float2 v) {
    __half2 h = __floats2half2_rn(v.x, v.y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
};
template <typename T> __device__ __forceinline__ float2 round_half2(float2 v) { return Pair<T>::unpack(Pair<T>::pack(v)); }
// Pair arithmetic, written as two scalar instructions: the packed fp32x2 forms were measured here and bring
// nothing (same instruction count and time; the values do not sit in aligned register pairs) and make the
// affine-LayerNorm variant spill.
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }

// Rows of up to 48 (NC = 3: six CTAs per SM) or 64 (NC = 4: four) elements per thread: the thread's part of the row is unpacked to fp32
// once and stays in fp32 registers through the statistics, the modulation, the absmax and the quantiser
// (two-at-a-time conversions between halves and fp32).  The fused LayerNorm variants are bound by instruction
// issue (66 % issue-active, ALU pipe 55 %: the half <-> fp32 conversions) as much as by HBM; every pass
// re-unpacking packed registers cost a quarter more.  Rounding points are unchanged.
template <typename T, int MODE, int WPR, int NC>
__global__ void __launch_bounds__(THREADS, NC == 3 ? 6 : 4) rowwise_f32_kernel(const Params p) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[3][2][4];
  constexpr int RPC = 4 / WPR;          // rows per CTA per iteration
  constexpr int GT = WPR * 32;          // threads per row
  const int warp = threadIdx.x >> 5;
  const int rg = warp / WPR;            // row slot of this warp
  const int t = threadIdx.x - rg * GT;  // thread index inside the row group
  const int nchunks = static_cast<int>(p.K / CHUNK);
  const T* x = static_cast<const T*>(p.x);
  const bool staged = (MODE == ADALN && p.mod_rows == 1) || MODE == LN_AFFINE;
  // Staged vectors (adaLN: 1 + scale rounded to half, and shift; affine LN: weight and bias) are kept as units of
  // 4 elements in unit-major order (unit u of chunk ch at index u * nchunks + ch): consecutive threads own
  // consecutive chunks and read consecutive units, no bank conflicts.
  // adaLN keeps them as halves (8-byte units of 4), affine LN as fp32 (16-byte units of 4).
  float4* s_mul = reinterpret_cast<float4*>(smem);  // LN_AFFINE: [4][nchunks] float4
  float4* s_add = s_mul + 4 * nchunks;
  uint2* h_mul = reinterpret_cast<uint2*>(smem);    // ADALN: [4][nchunks] uint2
  uint2* h_add = h_mul + 4 * nchunks;
  if (staged) {
    for (int i = threadIdx.x; i < 4 * nchunks; i += THREADS) {
      const int ch = i >> 2, u = i & 3;
      if (MODE == ADALN) {
        const uint2 cw = *reinterpret_cast<const uint2*>(static_cast<const T*>(p.scale) + ch * CHUNK + u * 4);
        const float2 one = make_float2(1.f, 1.f);
        uint2 m;  // (1 + scale) in half
        m.x = Pair<T>::pack(add2(one, Pair<T>::unpack(cw.x)));
        m.y = Pair<T>::pack(add2(one, Pair<T>::unpack(cw.y)));
        h_mul[u * nchunks + ch] = m;
        h_add[u * nchunks + ch] = *reinterpret_cast<const uint2*>(static_cast<const T*>(p.shift) + ch * CHUNK + u * 4);
      } else {
        s_mul[u * nchunks + ch] = *reinterpret_cast<const float4*>(p.w + ch * CHUNK + u * 4);
        s_add[u * nchunks + ch] = p.b ? *reinterpret_cast<const float4*>(p.b + ch * CHUNK + u * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    __syncthreads();
  }
  int par = 0;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * RPC; base < p.M; base += static_cast<int64_t>(gridDim.x) * RPC, par ^= 1) {
    const int64_t row = base + rg;
    const bool live = row < p.M;
    float f[NC][16];
    const T* xr = x + row * p.ldx;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int ch = t + c * GT;
      uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
      if (live && ch < nchunks) {
        a = *reinterpret_cast<const uint4*>(xr + ch * CHUNK);
        b = *reinterpret_cast<const uint4*>(xr + ch * CHUNK + 8);
      }
      const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 v = Pair<T>::unpack(w[i]);
        f[c][2 * i] = v.x;
        f[c][2 * i + 1] = v.y;
      }
    }
    if (MODE == ADALN || MODE == LN_AFFINE) {
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < 16; i += 2) acc = add2(acc, make_float2(f[c][i], f[c][i + 1]));
      const float mean = row_reduce<WPR, false>(acc.x + acc.y, &red[0][0][0], par, warp) / static_cast<float>(p.K);
      const float2 nm2 = make_float2(-mean, -mean);
      acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        if (t + c * GT < nchunks) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 d = add2(make_float2(f[c][i], f[c][i + 1]), nm2);
            acc = fma2(d, d, acc);
          }
        }
      }
      const float var = row_reduce<WPR, false>(acc.x + acc.y, &red[1][0][0], par, warp) / static_cast<float>(p.K);
      const float rstd = rsqrtf(var + p.eps);
      const float2 r2 = make_float2(rstd, rstd);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int ch = t + c * GT;
        if (live && ch < nchunks) {
          uint32_t hw[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float4 mu, ad;
            if (staged && MODE == LN_AFFINE) {
              mu = s_mul[u * nchunks + ch];
              ad = s_add[u * nchunks + ch];
            } else if (staged) {
              const uint2 mw = h_mul[u * nchunks + ch], aw = h_add[u * nchunks + ch];
              const float2 m01 = Pair<T>::unpack(mw.x), m23 = Pair<T>::unpack(mw.y), a01 = Pair<T>::unpack(aw.x), a23 = Pair<T>::unpack(aw.y);
              mu = make_float4(m01.x, m01.y, m23.x, m23.y);
              ad = make_float4(a01.x, a01.y, a23.x, a23.y);
            } else {  // per-row modulation (ADALN only)
              const T* gc = static_cast<const T*>(p.scale) + row * p.K + ch * CHUNK + u * 4;
              const T* gs = static_cast<const T*>(p.shift) + row * p.K + ch * CHUNK + u * 4;
              const uint2 cw = *reinterpret_cast<const uint2*>(gc), sw = *reinterpret_cast<const uint2*>(gs);
              const float2 c01 = Pair<T>::unpack(cw.x), c23 = Pair<T>::unpack(cw.y), s01 = Pair<T>::unpack(sw.x), s23 = Pair<T>::unpack(sw.y);
              const float2 one = make_float2(1.f, 1.f);
              const float2 t01 = round_half2<T>(add2(one, c01)), t23 = round_half2<T>(add2(one, c23));  // (1 + scale) in half
              mu = make_float4(t01.x, t01.y, t23.x, t23.y);
              ad = make_float4(s01.x, s01.y, s23.x, s23.y);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int i = 4 * u + 2 * j;
              const float2 m2 = j ? make_float2(mu.z, mu.w) : make_float2(mu.x, mu.y);
              const float2 a2 = j ? make_float2(ad.z, ad.w) : make_float2(ad.x, ad.y);
              float2 ln = mul2(add2(make_float2(f[c][i], f[c][i + 1]), nm2), r2);
              float2 v;
              if (MODE == ADALN) {
                ln = round_half2<T>(ln);  // F.layer_norm output in half
                v = p.round_product ? add2(round_half2<T>(mul2(ln, m2)), a2) : fma2(ln, m2, a2);
              } else {
                v = fma2(ln, m2, a2);
              }
              hw[2 * u + j] = Pair<T>::pack(v);  // the transformed row in half: what is quantised (and optionally stored)
              const float2 vr = Pair<T>::unpack(hw[2 * u + j]);
              f[c][i] = vr.x;
              f[c][i + 1] = vr.y;
            }
          }
          if (p.h_out) {
            T* ho = static_cast<T*>(p.h_out) + row * p.K + ch * CHUNK;
            *reinterpret_cast<uint4*>(ho) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4*>(ho + 8) = make_uint4(hw[4], hw[5], hw[6], hw[7]);
          }
        }
      }
    }
    float inv_h;  // multiplier already rounded to half precision
    float row_scale;
    if (MODE == STATIC) {
      if (p.scale_input) {
        row_scale = *p.scale_input;
        inv_h = round_half<T>(__frcp_rn(row_scale));
      } else {
        row_scale = 1.f;
        inv_h = 1.f;
      }
    } else {
      float am0 = 0.f, am1 = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          am0 = fmax3(am0, fabsf(f[c][i]), fabsf(f[c][i + 1]));
          am1 = fmax3(am1, fabsf(f[c][i + 2]), fabsf(f[c][i + 3]));
        }
      const float am = row_reduce<WPR, true>(fmaxf(am0, am1), &red[2][0][0], par, warp);
      row_scale = (am > 0.f) ? __fdiv_rn(am, 448.f) : 1.f;
      inv_h = round_half<T>(__frcp_rn(row_scale));
    }
    if (live) {
      if (t == 0) p.qscale[row] = row_scale;
      uint8_t* qr = p.q + row * p.K;
      const float2 i2 = make_float2(inv_h, inv_h);
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int ch = t + c * GT;
        if (ch < nchunks) {
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            // product formed in half precision, then rounded to e4m3
            const float2 p01 = round_half2<T>(mul2(make_float2(f[c][i], f[c][i + 1]), i2));
            const float2 p23 = round_half2<T>(mul2(make_float2(f[c][i + 2], f[c][i + 3]), i2));
            o[i >> 2] = cvt_e4m3x4(p01.x, p01.y, p23.x, p23.y);
          }
          *reinterpret_cast<uint4*>(qr + ch * CHUNK) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
  }
}

template <typename T, int MODE> int launch_t(const Params& p, cudaStream_t st) {
  const bool wide = p.K > 8192;
  size_t smem = 0;
  if (MODE == ADALN && p.mod_rows == 1) smem = 2 * p.K * sizeof(T);
  if (MODE == LN_AFFINE) smem = 2 * p.K * sizeof(float);
  // narrow rows: 1 or 2 warps per row and 4 chunks per thread; wide rows: all 4 warps on one row
  const int wpr = p.K <= 2048 ? 1 : (p.K <= 4096 ? 2 : 4);
  const int rpc = 4 / wpr;
  const int64_t want = (p.M + rpc - 1) / rpc;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
#define KSB_RQ_LAUNCH(W, NC)                                                                                                     \
  do {                                                                                                                           \
    if (smem > 48 * 1024 &&                                                                                                      \
        cudaFuncSetAttribute(rowwise_kernel<T, MODE, W, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");                                                     \
    rowwise_kernel<T, MODE, W, NC><<<grid, THREADS, smem, st>>>(p);                                                              \
  } while (0)
#define KSB_RQ_LAUNCH_F32(W, NC)                                                                                                  \
  do {                                                                                                                           \
    if (smem > 48 * 1024 &&                                                                                                      \
        cudaFuncSetAttribute(rowwise_f32_kernel<T, MODE, W, NC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");                                                     \
    rowwise_f32_kernel<T, MODE, W, NC><<<grid, THREADS, smem, st>>>(p);                                                          \
  } while (0)
  const bool three = p.K <= static_cast<int64_t>(wpr) * 32 * CHUNK * 3;  // three chunks per thread are enough
  if (wide) KSB_RQ_LAUNCH(4, 8);
  else if (wpr == 1) { if (three) KSB_RQ_LAUNCH_F32(1, 3); else KSB_RQ_LAUNCH_F32(1, 4); }
  else if (wpr == 2) { if (three) KSB_RQ_LAUNCH_F32(2, 3); else KSB_RQ_LAUNCH_F32(2, 4); }
  else { if (three) KSB_RQ_LAUNCH_F32(4, 3); else KSB_RQ_LAUNCH_F32(4, 4); }
#undef KSB_RQ_LAUNCH_F32
#undef KSB_RQ_LAUNCH
  return check_launch("rowwise quantiser");
}

template <int MODE> int launch(const Params& p, int dtype, cudaStream_t st) {
  if (p.M == 0) return 0;
  return dtype == KSB_BF16 ? launch_t<__nv_bfloat16, MODE>(p, st) : launch_t<__half, MODE>(p, st);
}

int validate(const Params& p, int dtype) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (p.M < 0 || p.K <= 0) return fail(KSB_ERR_INVALID, "bad shape M=%lld K=%lld", (long long)p.M, (long long)p.K);
  if (p.K % CHUNK != 0 || p.K > (int64_t)16384)
    return fail(KSB_ERR_INVALID, "K=%lld must be a multiple of 16 and <= 16384", (long long)p.K);
  if (p.ldx < p.K || p.ldx % 8 != 0) return fail(KSB_ERR_INVALID, "ldx=%lld must be >= K and a multiple of 8", (long long)p.ldx);
  if (p.M > 0 && (!p.x || !p.q || !p.qscale)) return fail(KSB_ERR_INVALID, "null pointer");
  if (!aligned16(p.x) || !aligned16(p.q) || (p.h_out && !aligned16(p.h_out)))
    return fail(KSB_ERR_INVALID, "pointers must be 16-byte aligned");
  return 0;
}

}  // namespace rq
}  // namespace ksb

using namespace ksb;

extern "C" {

int ksb_quant_fp8_rowwise(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, void* q, float* scale,
                          ksb_stream_t stream) {
  rq::Params p{};
  p.x = x; p.M = M; p.K = K; p.ldx = ldx; p.q = static_cast<uint8_t*>(q); p.qscale = scale;
  if (int rc = rq::validate(p, dtype)) return rc;
  return rq::launch<rq::PLAIN>(p, dtype, static_cast<cudaStream_t>(stream));
}

int ksb_quant_fp8_static(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const float* scale_input,
                         void* q, float* scale_out, ksb_stream_t stream) {
  rq::Params p{};
  p.x = x; p.M = M; p.K = K; p.ldx = ldx; p.q = static_cast<uint8_t*>(q); p.qscale = scale_out;
  p.scale_input = scale_input;
  if (int rc = rq::validate(p, dtype)) return rc;
  return rq::launch<rq::STATIC>(p, dtype, static_cast<cudaStream_t>(stream));
}

int ksb_adaln_quant_fp8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const void* shift,
                        const void* scale, int64_t mod_rows, int round_product, float eps, void* h_out, void* q,
                        float* qscale, ksb_stream_t stream) {
  rq::Params p{};
  p.round_product = round_product ? 1 : 0;
  p.x = x; p.M = M; p.K = K; p.ldx = ldx; p.shift = shift; p.scale = scale; p.mod_rows = mod_rows; p.eps = eps;
  p.h_out = h_out; p.q = static_cast<uint8_t*>(q); p.qscale = qscale;
  if (int rc = rq::validate(p, dtype)) return rc;
  if (!shift || !scale || !aligned16(shift) || !aligned16(scale)) return fail(KSB_ERR_INVALID, "shift/scale null or unaligned");
  if (mod_rows != 1 && mod_rows != M) return fail(KSB_ERR_INVALID, "mod_rows must be 1 or M");
  return rq::launch<rq::ADALN>(p, dtype, static_cast<cudaStream_t>(stream));
}

int ksb_layernorm_quant_fp8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const float* w,
                            const float* b, float eps, void* h_out, void* q, float* qscale, ksb_stream_t stream) {
  rq::Params p{};
  p.x = x; p.M = M; p.K = K; p.ldx = ldx; p.w = w; p.b = b; p.eps = eps; p.mod_rows = 1;
  p.h_out = h_out; p.q = static_cast<uint8_t*>(q); p.qscale = qscale;
  if (int rc = rq::validate(p, dtype)) return rc;
  if (!w || !aligned16(w) || (b && !aligned16(b))) return fail(KSB_ERR_INVALID, "weight / bias null or not 16-byte aligned");
  return rq::launch<rq::LN_AFFINE>(p, dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
