// Small HBM-bound companions of the block: gated residual where it is not fused into a GEMM epilogue, and the
// residual statistics of the block-level step cache.
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace ew {

// out[m, :] = x[m, :] + y[m, :] * gate[(gate_rows == 1 ? 0 : m), :]   (one rounding, like torch.addcmul)
template <typename T>
__global__ void __launch_bounds__(256) gate_residual_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                            const T* __restrict__ gate, int64_t gate_rows, T* __restrict__ out,
                                                            int64_t M, int64_t N) {
  const int64_t vec_per_row = N / 8;
  const int64_t total = M * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / vec_per_row, c = (i - m * vec_per_row) * 8;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + m * N + c);
    const uint4 yv = *reinterpret_cast<const uint4*>(y + m * N + c);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + (gate_rows == 1 ? 0 : m) * N + c);
    const T* xt = reinterpret_cast<const T*>(&xv);
    const T* yt = reinterpret_cast<const T*>(&yv);
    const T* gt = reinterpret_cast<const T*>(&gv);
    uint4 ov;
    T* ot = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      ot[k] = HalfOps<T>::from_f(fmaf(HalfOps<T>::to_f(yt[k]), HalfOps<T>::to_f(gt[k]), HalfOps<T>::to_f(xt[k])));
    *reinterpret_cast<uint4*>(out + m * N + c) = ov;
  }
}

// Residual of a group of blocks and its distance to the residual kept from an earlier step, in one pass:
//   r = round(x_new - x_old)             (the eager `x - x_ori` in the activation dtype)
//   sums[0] += round(|r - prev|)          sums[1] += |r|          sums[2] += |prev|
// r is written to res_out when given (it becomes the next step's `prev`).  prev may be NULL (sums[0], sums[2] stay 0).
// Per-thread fp32 partial sums, warp shuffle, one atomicAdd per warp and quantity.
template <typename T>
__global__ void __launch_bounds__(256) residual_diff_kernel(const T* __restrict__ x_new, const T* __restrict__ x_old,
                                                            const T* __restrict__ prev, T* __restrict__ res_out,
                                                            float* __restrict__ sums, int64_t nvec) {
  float s_diff = 0.f, s_cur = 0.f, s_prev = 0.f;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 av = *reinterpret_cast<const uint4*>(x_new + i * 8);
    const uint4 bv = *reinterpret_cast<const uint4*>(x_old + i * 8);
    uint4 pv = make_uint4(0, 0, 0, 0);
    if (prev) pv = *reinterpret_cast<const uint4*>(prev + i * 8);
    const T* at = reinterpret_cast<const T*>(&av);
    const T* bt = reinterpret_cast<const T*>(&bv);
    const T* pt = reinterpret_cast<const T*>(&pv);
    uint4 rv;
    T* rt = reinterpret_cast<T*>(&rv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const T r = HalfOps<T>::from_f(HalfOps<T>::to_f(at[k]) - HalfOps<T>::to_f(bt[k]));
      rt[k] = r;
      const float rf = HalfOps<T>::to_f(r), pf = HalfOps<T>::to_f(pt[k]);
      s_cur += fabsf(rf);
      s_prev += fabsf(pf);
      s_diff += HalfOps<T>::to_f(HalfOps<T>::from_f(fabsf(rf - pf)));
    }
    if (res_out) *reinterpret_cast<uint4*>(res_out + i * 8) = rv;
  }
  s_diff = warp_sum(s_diff);
  s_cur = warp_sum(s_cur);
  s_prev = warp_sum(s_prev);
  if ((threadIdx.x & 31) == 0) {
    if (prev) atomicAdd(sums + 0, s_diff);
    atomicAdd(sums + 1, s_cur);
    if (prev) atomicAdd(sums + 2, s_prev);
  }
}

}  // namespace ew
}  // namespace ksb

using namespace ksb;

extern "C" int ksb_residual_diff(const void* x_new, const void* x_old, const void* prev_residual, void* residual_out,
                                 float* sums, int dtype, int64_t n, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (n < 0 || n % 8 != 0) return fail(KSB_ERR_INVALID, "element count %lld must be a multiple of 8", (long long)n);
  if (!x_new || !x_old || !sums || !aligned16(x_new) || !aligned16(x_old) || (prev_residual && !aligned16(prev_residual)) ||
      (residual_out && !aligned16(residual_out)))
    return fail(KSB_ERR_INVALID, "null or unaligned pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(sums, 0, 3 * sizeof(float), st) != cudaSuccess) return fail(KSB_ERR_CUDA, "cannot clear the sums");
  if (n == 0) return 0;
  const int grid = sm_count() * 8;
  if (dtype == KSB_BF16)
    ew::residual_diff_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x_new), static_cast<const __nv_bfloat16*>(x_old),
                                                                 static_cast<const __nv_bfloat16*>(prev_residual), static_cast<__nv_bfloat16*>(residual_out), sums, n / 8);
  else
    ew::residual_diff_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x_new), static_cast<const __half*>(x_old),
                                                          static_cast<const __half*>(prev_residual), static_cast<__half*>(residual_out), sums, n / 8);
  return check_launch("residual diff");
}

extern "C" int ksb_gate_residual(const void* x, const void* y, const void* gate, int64_t gate_rows, void* out, int dtype,
                                 int64_t M, int64_t N, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (M < 0 || N <= 0 || N % 8 != 0) return fail(KSB_ERR_INVALID, "bad shape M=%lld N=%lld (N %% 8 == 0)", (long long)M, (long long)N);
  if (M == 0) return 0;
  if (!x || !y || !gate || !out || !aligned16(x) || !aligned16(y) || !aligned16(gate) || !aligned16(out))
    return fail(KSB_ERR_INVALID, "null or unaligned pointer");
  if (gate_rows != 1 && gate_rows != M) return fail(KSB_ERR_INVALID, "gate_rows must be 1 or M");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = sm_count() * 8;
  if (dtype == KSB_BF16)
    ew::gate_residual_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(gate), gate_rows, static_cast<__nv_bfloat16*>(out), M, N);
  else
    ew::gate_residual_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(y), static_cast<const __half*>(gate), gate_rows, static_cast<__half*>(out), M, N);
  return check_launch("gate residual");
}
