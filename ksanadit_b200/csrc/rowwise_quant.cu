// HBM-bound row kernels: per-token FP8 (e4m3) activation quantiser, alone or fused behind
// LayerNorm + adaLN modulate / affine LayerNorm.  One CTA walks rows; a row is read once from HBM
// with 2 x 128-bit loads per 16 elements, held in registers across the reductions, and written once
// (16 e4m3 bytes per 128-bit store).  Algorithmic bytes per row: 2K (read) + K (write) + 4 (scale).
//
// Rounding points follow the eager PyTorch sequence this replaces, so the FP8 bytes match it bit for
// bit: s = amax/448 (fp32 divide), inv = half(1/s), q = e4m3(half(x * inv)).
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace rq {

constexpr int THREADS = 256;
constexpr int CHUNK = 16;     // elements per thread-chunk
constexpr int MAX_CHUNKS = 4;  // K <= THREADS * CHUNK * MAX_CHUNKS = 16384

enum Mode : int { PLAIN = 0, ADALN = 1, LN_AFFINE = 2, STATIC = 3 };

struct Params {
  const void* x;
  int64_t M, K, ldx;
  const void* shift;  // ADALN
  const void* scale;  // ADALN
  int64_t mod_rows;
  const float* w;  // LN_AFFINE
  const float* b;
  float eps;
  const float* scale_input;  // STATIC (may be null = clamp only)
  void* h_out;               // optional half copy of the transformed row
  uint8_t* q;
  float* qscale;
};

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* red) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < THREADS / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

template <typename T> __device__ __forceinline__ void load16(const T* p, float (&f)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const T* ta = reinterpret_cast<const T*>(&a);
  const T* tb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[i] = HalfOps<T>::to_f(ta[i]);
    f[8 + i] = HalfOps<T>::to_f(tb[i]);
  }
}
template <typename T> __device__ __forceinline__ void store16(T* p, const float (&f)[16]) {
  uint4 a, b;
  T* ta = reinterpret_cast<T*>(&a);
  T* tb = reinterpret_cast<T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    ta[i] = HalfOps<T>::from_f(f[i]);
    tb[i] = HalfOps<T>::from_f(f[8 + i]);
  }
  *reinterpret_cast<uint4*>(p) = a;
  *reinterpret_cast<uint4*>(p + 8) = b;
}
template <typename T> __device__ __forceinline__ float round_half(float v) { return HalfOps<T>::to_f(HalfOps<T>::from_f(v)); }

template <typename T, int MODE> __global__ void __launch_bounds__(THREADS) rowwise_kernel(const Params p) {
  __shared__ float red[THREADS / 32];
  const int nchunks = static_cast<int>(p.K / CHUNK);
  const T* x = static_cast<const T*>(p.x);
  for (int64_t row = blockIdx.x; row < p.M; row += gridDim.x) {
    float v[MAX_CHUNKS][16];
    const T* xr = x + row * p.ldx;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < nchunks) load16<T>(xr + ch * CHUNK, v[c]);
    }
    if (MODE == ADALN || MODE == LN_AFFINE) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c)
        if (threadIdx.x + c * THREADS < nchunks)
#pragma unroll
          for (int i = 0; i < 16; ++i) s += v[c][i];
      const float mean = block_reduce(s, false, red) / static_cast<float>(p.K);
      float s2 = 0.f;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c)
        if (threadIdx.x + c * THREADS < nchunks)
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float d = v[c][i] - mean;
            s2 += d * d;
          }
      const float var = block_reduce(s2, false, red) / static_cast<float>(p.K);
      const float rstd = rsqrtf(var + p.eps);
      const int64_t mrow = (p.mod_rows == 1) ? 0 : row;
#pragma unroll
      for (int c = 0; c < MAX_CHUNKS; ++c) {
        const int ch = threadIdx.x + c * THREADS;
        if (ch < nchunks) {
          if (MODE == ADALN) {
            float sh[16], sc[16];
            load16<T>(static_cast<const T*>(p.shift) + mrow * p.K + ch * CHUNK, sh);
            load16<T>(static_cast<const T*>(p.scale) + mrow * p.K + ch * CHUNK, sc);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float ln = round_half<T>((v[c][i] - mean) * rstd);  // F.layer_norm output in half
              const float t = round_half<T>(1.f + sc[i]);               // (1 + scale) in half
              v[c][i] = round_half<T>(fmaf(ln, t, sh[i]));              // addcmul, one rounding
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float y = (v[c][i] - mean) * rstd * p.w[ch * CHUNK + i];
              if (p.b) y += p.b[ch * CHUNK + i];
              v[c][i] = round_half<T>(y);
            }
          }
          if (p.h_out) store16<T>(static_cast<T*>(p.h_out) + row * p.K + ch * CHUNK, v[c]);
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
      for (int c = 0; c < MAX_CHUNKS; ++c)
        if (threadIdx.x + c * THREADS < nchunks)
#pragma unroll
          for (int i = 0; i < 16; ++i) am = fmaxf(am, fabsf(v[c][i]));
      am = block_reduce(am, true, red);
      row_scale = (am > 0.f) ? __fdiv_rn(am, 448.f) : 1.f;
      inv_h = round_half<T>(__frcp_rn(row_scale));
    }
    if (threadIdx.x == 0) p.qscale[row] = row_scale;
    uint8_t* qr = p.q + row * p.K;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
      const int ch = threadIdx.x + c * THREADS;
      if (ch < nchunks) {
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) t[i] = round_half<T>(v[c][i] * inv_h);  // product formed in half precision
        uint4 o;
        o.x = cvt_e4m3x4(t[0], t[1], t[2], t[3]);
        o.y = cvt_e4m3x4(t[4], t[5], t[6], t[7]);
        o.z = cvt_e4m3x4(t[8], t[9], t[10], t[11]);
        o.w = cvt_e4m3x4(t[12], t[13], t[14], t[15]);
        *reinterpret_cast<uint4*>(qr + ch * CHUNK) = o;
      }
    }
  }
}

template <int MODE> int launch(const Params& p, int dtype, cudaStream_t st) {
  if (p.M == 0) return 0;
  const int64_t grid = p.M < (int64_t)sm_count() * 16 ? p.M : (int64_t)sm_count() * 16;
  if (dtype == KSB_BF16)
    rowwise_kernel<__nv_bfloat16, MODE><<<(unsigned)grid, THREADS, 0, st>>>(p);
  else
    rowwise_kernel<__half, MODE><<<(unsigned)grid, THREADS, 0, st>>>(p);
  return check_launch("rowwise quantiser");
}

int validate(const Params& p, int dtype) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (p.M < 0 || p.K <= 0) return fail(KSB_ERR_INVALID, "bad shape M=%lld K=%lld", (long long)p.M, (long long)p.K);
  if (p.K % CHUNK != 0 || p.K > (int64_t)THREADS * CHUNK * MAX_CHUNKS)
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
                        const void* scale, int64_t mod_rows, float eps, void* h_out, void* q, float* qscale,
                        ksb_stream_t stream) {
  rq::Params p{};
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
  if (!w) return fail(KSB_ERR_INVALID, "weight is null");
  return rq::launch<rq::LN_AFFINE>(p, dtype, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
