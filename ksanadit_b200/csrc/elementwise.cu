// Small HBM-bound companions of the block: gated residual where it is not fused into a GEMM epilogue.
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

}  // namespace ew
}  // namespace ksb

using namespace ksb;

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
