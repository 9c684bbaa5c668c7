// Library state of the C ABI: error text, device status words, tensor-map encoding, device queries.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {

__device__ int g_status[4] = {0, 0, 0, 0};

static thread_local char t_err[512] = "";

int fail(int rc, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return rc;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(KSB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner,
                   uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(KSB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (!aligned16(base) || (row_stride_bytes & 15)) return fail(KSB_ERR_INVALID, "tensor map: base/stride not 16-byte aligned");
  if (box_inner * elem_bytes > 128 || box_outer > 256) return fail(KSB_ERR_INVALID, "tensor map: box too large");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = (box_inner * elem_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KSB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

int* status_words() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Self-test of the bounded wait: thread 0 waits for a barrier phase that nothing completes, with a short limit, and
// must come back with the time-out recorded; the other threads wait for it at a block barrier.  The kernel returns
// by itself and leaves the context usable.
constexpr int SELFTEST_KERNEL_ID = 15;
__global__ void bounded_wait_selftest_kernel(int* status, uint64_t limit_ns, int* returned) {
  __shared__ uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_limit(b, 0, status, (SELFTEST_KERNEL_ID << 16) | 1, limit_ns, 0x3u);
    *returned = ok ? 1 : 2;
  }
  __syncthreads();
}

}  // namespace ksb

extern "C" {

int ksb_selftest_bounded_wait(int64_t limit_ns, int* returned, ksb_stream_t stream) {
  if (limit_ns <= 0 || limit_ns > 1000000000ll) return ksb::fail(KSB_ERR_INVALID, "limit_ns must be in (0, 1e9]");
  if (!returned) return ksb::fail(KSB_ERR_INVALID, "null pointer");
  int* st = ksb::status_words();
  if (!st) return ksb::fail(KSB_ERR_CUDA, "status words unavailable");
  ksb::bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(st, static_cast<uint64_t>(limit_ns), returned);
  return ksb::check_launch("bounded wait self-test");
}

int ksb_version(void) { return 100; }

const char* ksb_last_error(void) { return ksb::t_err; }

int ksb_sm_count(void) { return ksb::sm_count(); }

int ksb_device_status(int* code, int* detail) {
  int h[4] = {0, 0, 0, 0};
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return ksb::fail(KSB_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
  e = cudaMemcpyFromSymbol(h, ksb::g_status, sizeof(h));
  if (e != cudaSuccess) return ksb::fail(KSB_ERR_CUDA, "status read: %s", cudaGetErrorString(e));
  if (code) *code = h[0];
  if (detail) *detail = h[1];
  if (h[0] != 0) {
    int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(ksb::g_status, z, sizeof(z));
  }
  return 0;
}

}  // extern "C"
