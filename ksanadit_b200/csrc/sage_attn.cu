// Sage-style quantised attention core on the Blackwell tensor cores, dense or block-sparse.
//
//   S = Q8 . K8^T            tcgen05.mma kind::i8   (s32 accumulator in tensor memory)
//   X = float(S) * qs * ks   fp32, exp2 domain (softmax scale and log2 e are folded into Q8's scale)
//   P = exp2(X - m + 8)      fp32 online softmax against the exact running row maximum, rounded to e4m3
//   O += P . V8              tcgen05.mma kind::f8f6f4 (f32 accumulator in tensor memory)
//   out = O / l * vs
//
// One CTA works on one (head, 128-row Q block) at a time and walks that block's list of 128-token KV
// tiles; two CTAs share an SM (256 tensor-memory columns and ~98 KB of shared memory each), so one
// CTA's softmax overlaps the other's MMAs.  Warp roles inside a CTA:
//   warp 0      TMA producer (Q block once per work item; K and V^T tiles through 2-deep rings)
//   warp 1      MMA issuer (single thread): S = Q.K^T for tile j+1 is queued before P.V of tile j
//   warps 2,3   idle (they only donate registers)
//   warps 4..7  softmax: one row per thread; tcgen05.ld S, max, exp2, e4m3 P written to shared memory
//               in the 128-byte-swizzled K-major layout the MMA reads, O rescaled in tensor memory in the
//               tiles where a row maximum of the warp grew; final normalisation and store
// Every mbarrier wait is bounded (see common.cuh).
//
// Tensor-bound: 4 * 128 * 128 * 128 flop per visited (Q block, KV tile) pair.
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace attn {

constexpr int BQ = 128, BKV = 128, D = 128;
constexpr int UMMA_K = 32;
constexpr int KST = 2, VST = 2;
constexpr int TILE_BYTES = 128 * 128;
constexpr int THREADS = 256;
constexpr int TMEM_COLS = 256;  // S: columns 0..127 (s32), O: columns 128..255 (f32)
constexpr int KERNEL_ID = 2;
constexpr float P_SHIFT = 8.0f;  // P carries a static factor 2^8 into e4m3: the row maximum maps to 256 exactly
constexpr int NUM_BARS = 12;
constexpr int SMEM_BYTES = 1024 + (2 + KST + VST) * TILE_BYTES + 8 * NUM_BARS + 64;

struct Params {
  const float* qs;
  const float* ks;
  const float* vs;
  int H, Lq, Lk, nq, nkv;
  const int32_t* offsets;
  const int32_t* entries;
  void* out;
  int64_t out_ts, out_hs;
  int* status;
};

struct Work {
  int h, qt, n;
  const int32_t* ents;
};

__device__ __forceinline__ Work get_work(const Params& p, int idx) {
  Work w;
  w.h = idx / p.nq;
  w.qt = idx - w.h * p.nq;
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

template <typename T>
__global__ void __launch_bounds__(THREADS, 2)
sage_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base, p_smem = base + TILE_BYTES;
  const uint32_t k_smem = base + 2 * TILE_BYTES, v_smem = k_smem + KST * TILE_BYTES;
  const uint32_t bars = v_smem + VST * TILE_BYTES;
  const uint32_t q_full = bars, q_empty = bars + 8, k_full = bars + 16, k_empty = bars + 32, v_full = bars + 48,
                 v_empty = bars + 64, s_full = bars + 80, s_empty = bars + 88, p_full = bars + 96, p_empty = bars + 104;
  const uint32_t tmem_slot = bars + 8 * NUM_BARS + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + (2 + KST + VST) * TILE_BYTES + 8 * NUM_BARS + 16);
  uint8_t* p_gen = gen + TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.H * p.nq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KST; ++s) { mbar_init(k_full + 8 * s, 1); mbar_init(k_empty + 8 * s, 1); }
    for (int s = 0; s < VST; ++s) { mbar_init(v_full + 8 * s, 1); mbar_init(v_empty + 8 * s, 1); }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 128);
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      uint32_t wi = 0, itk = 0, itv = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
        const Work w = get_work(p, idx);
        if (w.n == 0) continue;
        if (!mbar_wait(q_empty, (wi & 1) ^ 1, p.status, (KERNEL_ID << 16) | 1)) { ok = false; break; }
        mbar_arrive_expect_tx(q_full, TILE_BYTES);
        tma_load_2d(q_smem, &tmap_q, q_full, 0, (w.h * p.nq + w.qt) * BQ);
        for (int j = 0; j < w.n; ++j) {
          const int t = entry_at(w, j) >> 2;
          {
            const uint32_t s = itk % KST, ph = (itk / KST) & 1;
            if (!mbar_wait(k_empty + 8 * s, ph ^ 1, p.status, (KERNEL_ID << 16) | 2)) { ok = false; break; }
            mbar_arrive_expect_tx(k_full + 8 * s, TILE_BYTES);
            tma_load_2d(k_smem + s * TILE_BYTES, &tmap_k, k_full + 8 * s, 0, (w.h * p.nkv + t) * BKV);
            ++itk;
          }
          {
            const uint32_t s = itv % VST, ph = (itv / VST) & 1;
            if (!mbar_wait(v_empty + 8 * s, ph ^ 1, p.status, (KERNEL_ID << 16) | 3)) { ok = false; break; }
            mbar_arrive_expect_tx(v_full + 8 * s, TILE_BYTES);
            tma_load_2d(v_smem + s * TILE_BYTES, &tmap_v, v_full + 8 * s, t * BKV, w.h * D);
            ++itv;
          }
        }
        ++wi;
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = IDESC_S8_S32(BQ, BKV);
      constexpr uint32_t idesc_pv = IDESC_F8_E4M3_F32(BQ, D);
      const uint64_t dq = make_kmajor_sw128_desc(q_smem), dp = make_kmajor_sw128_desc(p_smem);
      uint32_t wi = 0, itk = 0, itv = 0, g = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t gg) -> bool {
        const uint32_t s = itk % KST, ph = (itk / KST) & 1;
        if (!mbar_wait(k_full + 8 * s, ph, p.status, (KERNEL_ID << 16) | 4)) return false;
        if (!mbar_wait(s_empty, (gg & 1) ^ 1, p.status, (KERNEL_ID << 16) | 5)) return false;
        tc_fence_after();
        const uint64_t dk = make_kmajor_sw128_desc(k_smem + s * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / UMMA_K; ++kk) mma_i8_ss(tmem_s, dq + 2 * kk, dk + 2 * kk, idesc_qk, kk != 0);
        mma_commit(s_full);
        mma_commit(k_empty + 8 * s);
        ++itk;
        return true;
      };
      for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
        const Work w = get_work(p, idx);
        if (w.n == 0) continue;
        if (!mbar_wait(q_full, wi & 1, p.status, (KERNEL_ID << 16) | 6)) { ok = false; break; }
        if (!issue_qk(g)) { ok = false; break; }
        for (int j = 0; j < w.n; ++j) {
          if (j + 1 < w.n) {
            if (!issue_qk(g + 1)) { ok = false; break; }
          } else {
            mma_commit(q_empty);  // every S = Q.K^T of this work item has been issued
          }
          const uint32_t s = itv % VST, ph = (itv / VST) & 1;
          if (!mbar_wait(v_full + 8 * s, ph, p.status, (KERNEL_ID << 16) | 7)) { ok = false; break; }
          if (!mbar_wait(p_full, g & 1, p.status, (KERNEL_ID << 16) | 8)) { ok = false; break; }
          tc_fence_after();
          const uint64_t dv = make_kmajor_sw128_desc(v_smem + s * TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKV / UMMA_K; ++kk) mma_f8_ss(tmem_o, dp + 2 * kk, dv + 2 * kk, idesc_pv, (j | kk) != 0);
          mma_commit(p_empty);
          mma_commit(v_empty + 8 * s);
          ++itv;
          ++g;
        }
        ++wi;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ------------------------------------------------------------------ softmax warps (one row per thread)
    const int qrt = warp & 3;
    const int row = qrt * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(qrt * 32) << 16;
    const int nk64 = p.nkv * 2;
    T* out = static_cast<T*>(p.out);
    uint32_t g = 0;
    bool ok = true;
    for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
      const Work w = get_work(p, idx);
      const int qrow = w.qt * BQ + row;
      T* orow = out + static_cast<int64_t>(qrow) * p.out_ts + static_cast<int64_t>(w.h) * p.out_hs;
      if (w.n == 0) {
        if (qrow < p.Lq) {
#pragma unroll
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const float qsc = p.qs[w.h * p.nq + w.qt];
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < w.n; ++j) {
        const int e = entry_at(w, j);
        const int t = e >> 2, halves = e & 3;
        const int valid = min(BKV, p.Lk - t * BKV);
        const bool full = (halves == 3) && (valid == BKV);
        if (!mbar_wait_warp(s_full, g & 1, p.status, (KERNEL_ID << 16) | 9)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[4][32];
        tmem_ld32(tmem_s + lane_sel + 0, s[0]);
        tmem_ld32(tmem_s + lane_sel + 32, s[1]);
        tmem_ld32(tmem_s + lane_sel + 64, s[2]);
        tmem_ld32(tmem_s + lane_sel + 96, s[3]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(s_empty);
        const float sc0 = qsc * p.ks[w.h * nk64 + 2 * t], sc1 = qsc * p.ks[w.h * nk64 + 2 * t + 1];
        if (!full) {
          // masked columns (ragged tail or dropped 64-token half) take the most negative score
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = c * 32 + i;
              const bool keep = (col < valid) && ((halves >> (col >> 6)) & 1);
              if (!keep) s[c][i] = 0x80000000u;
            }
        }
        int mx0 = INT_MIN, mx1 = INT_MIN;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          mx0 = max(mx0, max(static_cast<int>(s[0][i]), static_cast<int>(s[1][i])));
          mx1 = max(mx1, max(static_cast<int>(s[2][i]), static_cast<int>(s[3][i])));
        }
        float m_tile = -INFINITY;
        if (mx0 != INT_MIN) m_tile = __int2float_rn(mx0) * sc0;
        if (mx1 != INT_MIN) m_tile = fmaxf(m_tile, __int2float_rn(mx1) * sc1);
        // the reference point is the exact running maximum: O is rescaled in every tile in which some row
        // of the warp found a larger score (rows that did not get the factor 1)
        const bool grow = m_tile > m_used;  // also true for the first tile (m_used = -inf)
        bool waited_pv = false;
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_used, m_tile);
          const float alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
          if (j > 0) {
            // O may only be touched once the previous P.V has completed
            if (!mbar_wait_warp(p_empty, (g & 1) ^ 1, p.status, (KERNEL_ID << 16) | 10)) { ok = false; break; }
            waited_pv = true;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
              uint32_t o[32];
              tmem_ld32(tmem_o + lane_sel + c, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tmem_o + lane_sel + c, o);
            }
            tmem_wait_st();
          }
          l *= alpha;
          m_used = m_new;
        }
        // P = exp2(X - m_used) -> e4m3, packed 4 per word; masked columns give exactly 0
        const float neg_m = (m_used == -INFINITY) ? 0.f : (P_SHIFT - m_used);
        uint32_t pk[32];
        float lsum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float sc = (c < 2) ? sc0 : sc1;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float pv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int si = static_cast<int>(s[c][i + u]);
              float x = fmaf(__int2float_rn(si), sc, neg_m);
              float e2 = fast_exp2(x);
              if (!full && si == INT_MIN) e2 = 0.f;
              pv[u] = e2;
              lsum += e2;
            }
            pk[c * 8 + (i >> 2)] = cvt_e4m3x4(pv[0], pv[1], pv[2], pv[3]);
          }
        }
        l += lsum;
        if (!waited_pv) {
          // the previous P.V must have finished reading the P buffer before it is overwritten
          if (!mbar_wait_warp(p_empty, (g & 1) ^ 1, p.status, (KERNEL_ID << 16) | 11)) { ok = false; break; }
        }
        // row `row` of the K-major tile: eight 16-byte chunks, chunk index XORed with (row & 7)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v4 = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          *reinterpret_cast<uint4*>(p_gen + row * 128 + ((c ^ (row & 7)) << 4)) = v4;
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(p_full);
        ++g;
      }
      if (!ok) break;
      // ---- epilogue of the work item: wait for the last P.V, normalise, store
      if (!mbar_wait_warp(p_empty, (g & 1) ^ 1, p.status, (KERNEL_ID << 16) | 12)) { ok = false; break; }
      tc_fence_after();
      const float inv_l = (l > 0.f) ? (1.f / l) : 0.f;
      const float* vsh = p.vs + w.h * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_sel + c, o);
        tmem_wait_ld();
        if (qrow < p.Lq) {
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            uint4 ov;
            T* ot = reinterpret_cast<T*>(&ov);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              ot[i] = HalfOps<T>::from_f(__uint_as_float(o[v8 * 8 + i]) * inv_l * __ldg(vsh + c + v8 * 8 + i));
            *reinterpret_cast<uint4*>(orow + c + v8 * 8) = ov;
          }
        }
      }
      tc_fence_before();
    }
  }

  // ------------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace attn
}  // namespace ksb

using namespace ksb;

extern "C" int ksb_sage_attn(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                             const float* vs, int64_t H, int64_t Lq, int64_t Lk, const int32_t* tile_offsets,
                             const int32_t* tile_entries, void* out, int dtype, int64_t out_token_stride,
                             int64_t out_head_stride, int32_t* counter, ksb_stream_t stream) {
  (void)counter;
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (H <= 0 || Lq <= 0 || Lk <= 0) return fail(KSB_ERR_INVALID, "bad shape H=%lld Lq=%lld Lk=%lld", (long long)H, (long long)Lq, (long long)Lk);
  if (!q8 || !qs || !k8 || !ks || !vt || !vs || !out) return fail(KSB_ERR_INVALID, "null pointer");
  if ((tile_offsets == nullptr) != (tile_entries == nullptr)) return fail(KSB_ERR_INVALID, "tile_offsets and tile_entries must both be given or both be NULL");
  if (!aligned16(out) || out_token_stride % 8 != 0 || out_head_stride % 8 != 0) return fail(KSB_ERR_INVALID, "out must be 16-byte aligned with strides multiple of 8 elements");
  const int64_t nq = (Lq + 127) / 128, nkv = (Lk + 127) / 128;
  if (H * nq > INT32_MAX / 256 || H * nkv > INT32_MAX / 256) return fail(KSB_ERR_INVALID, "problem too large");
  CUtensorMap tq, tk, tv;
  if (int rc = encode_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q8, 128, (uint64_t)(H * nq * 128), 128, 128, 128)) return rc;
  if (int rc = encode_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, 128, (uint64_t)(H * nkv * 128), 128, 128, 128)) return rc;
  if (int rc = encode_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, vt, (uint64_t)(nkv * 128), (uint64_t)(H * 128), (uint64_t)(nkv * 128), 128, 128)) return rc;
  attn::Params p{};
  p.qs = qs; p.ks = ks; p.vs = vs;
  p.H = (int)H; p.Lq = (int)Lq; p.Lk = (int)Lk; p.nq = (int)nq; p.nkv = (int)nkv;
  p.offsets = tile_offsets; p.entries = tile_entries;
  p.out = out; p.out_ts = out_token_stride; p.out_hs = out_head_stride;
  p.status = status_words();
  if (!p.status) return fail(KSB_ERR_CUDA, "status words unavailable");
  const int64_t total = H * nq;
  const int64_t cap = 2 * (int64_t)sm_count();
  const int grid = (int)(total < cap ? total : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == KSB_BF16) {
    if (cudaFuncSetAttribute(attn::sage_attn_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES) != cudaSuccess)
      return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");
    attn::sage_attn_kernel<__nv_bfloat16><<<grid, attn::THREADS, attn::SMEM_BYTES, st>>>(tq, tk, tv, p);
  } else {
    if (cudaFuncSetAttribute(attn::sage_attn_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_BYTES) != cudaSuccess)
      return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");
    attn::sage_attn_kernel<__half><<<grid, attn::THREADS, attn::SMEM_BYTES, st>>>(tq, tk, tv, p);
  }
  return check_launch("sage attention");
}
