// Dense Sage-style attention with TWO 128-row Q blocks of a head per CTA, one CTA per SM.
//
// Same arithmetic, tile shapes and per-block pipeline as sage_attn_kernel (see sage_attn.cu), but the two Q blocks
// that used to run as two independent CTAs on an SM now live in one CTA and share every K and V^T tile: the tile is
// fetched from L2 and written to shared memory once for 256 query rows instead of once per 128.  Under the 1 kW cap
// that traffic decides the clock: with it halved the kernel holds the maximum SM clock where the one-block kernel
// settles ~6 % lower.
//
// Warp roles (384 threads):
//   warp 0        TMA producer: both Q blocks once per work item, then K and V^T tiles through 4-deep rings
//   warps 1, 2    MMA issuer of half 0 / half 1 (one thread each): S = Q.K^T of tile j+1 queued before P.V of tile j;
//                 a ring stage is free when both issuers' MMAs on it have completed (barrier count 2)
//   warp 3        idle (donates registers)
//   warps 4..7    softmax of half 0, warps 8..11 of half 1: one row per thread, as in the one-block kernel
// Tensor memory (512 columns): half h has S at 256 h, O at 256 h + 128.  The halves are independent pipelines; only
// the producer and the ring barriers are shared, so one half's softmax still overlaps the other half's MMAs.
// An odd last block pair has one live half; the other half's issuer keeps the rings moving by arriving in place of
// its MMAs.
// Tile lists (block-sparse masks) are given per PAIR of Q blocks: the union of the two blocks' lists, each entry =
// KV tile * 16 + keep bits of block 2i (bits 0-1: tokens 0-63 / 64-127 of the tile) + keep bits of block 2i+1 (bits
// 2-3).  Both halves walk the whole union; a half masks the 64-token halves it does not keep (a tile it does not keep
// at all costs it a fully masked pass: P = 0), so pairing pays only where the two lists nearly coincide; the host
// side decides (ops.py) and otherwise sends tile lists to the one-block kernel.
#include "sage_attn_common.cuh"
#include "host_utils.h"

namespace ksb {
namespace attn {
namespace dual {

#ifndef KSB_ATTN_DUAL_RING
#define KSB_ATTN_DUAL_RING 4
#endif
constexpr int RST = KSB_ATTN_DUAL_RING;  // K and V ring depth
constexpr int THREADS2 = 384;
constexpr int TMEM_COLS2 = 512;
constexpr int KERNEL_ID2 = 3;
constexpr int NUM_BARS2 = 32;
// Q x 2 | P x 2 halves x 2 buffers | K x RST | V x RST | constants | barriers
constexpr int NUM_TILES2 = 2 + 4 + 2 * RST;
constexpr int SMEM_BYTES2 = 1024 + NUM_TILES2 * TILE_BYTES + CONST_BYTES + 8 * NUM_BARS2 + 64;
constexpr int PRODUCER_REGS = 56, SOFTMAX_REGS = 200;

struct PairWork {
  int h, pr, n;
  const int32_t* ents;
};
// LISTS = false is the dense kernel: every pair walks all KV tiles and the list code compiles away.
template <bool LISTS>
__device__ __forceinline__ PairWork get_pair(const Params& p, int idx, int npairs) {
  PairWork w;
  w.h = idx / npairs;
  w.pr = idx - w.h * npairs;
  if (LISTS && p.order) w.pr = p.order[w.pr];
  if (LISTS && p.offsets) {
    const int a = p.offsets[w.pr];
    w.n = p.offsets[w.pr + 1] - a;
    w.ents = p.entries + a;
  } else {
    w.n = p.nkv;
    w.ents = nullptr;
  }
  return w;
}
template <bool LISTS>
__device__ __forceinline__ int pair_entry(const PairWork& w, int j) { return (LISTS && w.ents) ? w.ents[j] : (j * 16 + 15); }

template <typename T, bool LISTS>
__global__ void __launch_bounds__(THREADS2, 1)
sage_attn_dual_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base, p_smem = base + 2 * TILE_BYTES;
  const uint32_t k_smem = base + 6 * TILE_BYTES, v_smem = k_smem + RST * TILE_BYTES;
  const uint32_t const_smem = v_smem + RST * TILE_BYTES;
  const uint32_t bars = const_smem + CONST_BYTES;
  const uint32_t q_full = bars, q_empty = bars + 8, k_full = bars + 16, k_empty = k_full + 8 * RST, v_full = k_empty + 8 * RST,
                 v_empty = v_full + 8 * RST;
  const uint32_t half_bars = v_empty + 8 * RST;  // per half: s_full, s_empty, p_full x 2, p_empty x 2 (48 bytes)
  const uint32_t tmem_slot = bars + 8 * NUM_BARS2 + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + NUM_TILES2 * TILE_BYTES + CONST_BYTES + 8 * NUM_BARS2 + 16);
  static_assert(2 + 4 * RST + 12 <= NUM_BARS2, "barrier block too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int npairs = (p.nq + 1) >> 1;
  const int total = p.H * npairs;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);  // both issuers are done with their Q block
    for (int s = 0; s < RST; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 2);  // both halves' MMAs on the stage have completed
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 2);
    }
    for (int h = 0; h < 2; ++h) {
      const uint32_t hb = half_bars + 48 * h;
      mbar_init(hb, 1);      // s_full
      mbar_init(hb + 8, 4);  // s_empty: one arrival per softmax warp
      for (int b = 0; b < 2; ++b) {
        mbar_init(hb + 16 + 8 * b, 4);  // p_full
        mbar_init(hb + 32 + 8 * b, 1);  // p_empty
      }
    }
    fence_barrier_init();
  }
  if (threadIdx.x < CONST_BYTES / 4) {
    // operands of the accumulator pre-load MMA (see sage_attn.cu)
    const uint32_t word = (threadIdx.x & 3) ? 0u : (threadIdx.x < CONST_BYTES / 8 ? 0x3F80u : 0x4AC0u);
    reinterpret_cast<uint32_t*>(gen + NUM_TILES2 * TILE_BYTES)[threadIdx.x] = word;
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS2);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      uint32_t wi = 0, it = 0;
      bool ok = true;
      for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
        const PairWork w = get_pair<LISTS>(p, idx, npairs);
        if (w.n == 0) continue;
        const int h = w.h, qt0 = w.pr * 2;
        const bool two = qt0 + 1 < p.nq;
        if (!mbar_wait(q_empty, (wi & 1) ^ 1, p.status, (KERNEL_ID2 << 16) | 1)) { ok = false; break; }
        mbar_arrive_expect_tx(q_full, (two ? 2 : 1) * TILE_BYTES);
        tma_load_2d(q_smem, &tmap_q, q_full, 0, (h * p.nq + qt0) * BQ);
        if (two) tma_load_2d(q_smem + TILE_BYTES, &tmap_q, q_full, 0, (h * p.nq + qt0 + 1) * BQ);
        for (int j = 0; j < w.n; ++j, ++it) {
          const int t = pair_entry<LISTS>(w, j) >> 4;
          const uint32_t s = it % RST, ph = (it / RST) & 1;
          if (!mbar_wait(k_empty + 8 * s, ph ^ 1, p.status, (KERNEL_ID2 << 16) | 2)) { ok = false; break; }
          mbar_arrive_expect_tx(k_full + 8 * s, TILE_BYTES);
          tma_load_2d(k_smem + s * TILE_BYTES, &tmap_k, k_full + 8 * s, 0, (h * p.nkv + t) * BKV);
          if (!mbar_wait(v_empty + 8 * s, ph ^ 1, p.status, (KERNEL_ID2 << 16) | 3)) { ok = false; break; }
          mbar_arrive_expect_tx(v_full + 8 * s, TILE_BYTES);
          tma_load_2d(v_smem + s * TILE_BYTES, &tmap_v, v_full + 8 * s, t * BKV, h * D);
        }
        ++wi;
      }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer of one half
      const int hf = warp - 1;
      const uint32_t hb = half_bars + 48 * hf;
      const uint32_t s_full = hb, s_empty = hb + 8, p_full = hb + 16, p_empty = hb + 32;
      const uint32_t tmem_s = tmem_base + 256 * hf, tmem_o = tmem_s + 128;
      constexpr uint32_t idesc_qk = IDESC_S8_S32(BQ, BKV);
      constexpr uint32_t idesc_pv = IDESC_F8_E4M3_F32(BQ, D);
      constexpr uint32_t idesc_pre = IDESC_BF16_F32(BQ, BKV);
      const uint64_t dq = make_kmajor_sw128_desc(q_smem + hf * TILE_BYTES);
      const uint64_t dca = make_noswizzle_desc(const_smem, 16, 16);
      const uint64_t dcb = make_noswizzle_desc(const_smem + CONST_BYTES / 2, 16, 16);
      uint32_t wi = 0, itk = 0, itv = 0, g = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t gg) -> bool {
        const uint32_t s = itk % RST, ph = (itk / RST) & 1;
        if (!mbar_wait(k_full + 8 * s, ph, p.status, (KERNEL_ID2 << 16) | 4)) return false;
        if (!mbar_wait(s_empty, gg & 1, p.status, (KERNEL_ID2 << 16) | 5)) return false;  // S read by the softmax warps (completion #gg)
        tc_fence_after();
        const uint64_t dk = make_kmajor_sw128_desc(k_smem + s * TILE_BYTES);
        mma_bf16_ss(tmem_s, dca, dcb, idesc_pre, 0);  // every accumulator = 12582912.0f
#pragma unroll
        for (int kk = 0; kk < D / UMMA_K; ++kk) mma_i8_ss(tmem_s, dq + 2 * kk, dk + 2 * kk, idesc_qk, 1);
        mma_commit(s_full);
        mma_commit(k_empty + 8 * s);
        ++itk;
        return true;
      };
      for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
        const PairWork w = get_pair<LISTS>(p, idx, npairs);
        if (w.n == 0) continue;
        const int nt = w.n, qt = w.pr * 2 + hf;
        if (!mbar_wait(q_full, wi & 1, p.status, (KERNEL_ID2 << 16) | 6)) { ok = false; break; }
        if (qt >= p.nq) {
          // no block for this half: hand every stage back as soon as it has been filled
          mbar_arrive(q_empty);
          for (int j = 0; j < nt && ok; ++j, ++itk, ++itv) {
            const uint32_t s = itk % RST, ph = (itk / RST) & 1;
            if (!mbar_wait(k_full + 8 * s, ph, p.status, (KERNEL_ID2 << 16) | 4)) { ok = false; break; }
            mbar_arrive(k_empty + 8 * s);
            if (!mbar_wait(v_full + 8 * s, ph, p.status, (KERNEL_ID2 << 16) | 7)) { ok = false; break; }
            mbar_arrive(v_empty + 8 * s);
          }
          ++wi;
          continue;
        }
        if (!issue_qk(g)) { ok = false; break; }
        for (int j = 0; j < nt; ++j) {
          if (j + 1 < nt) {
            if (!issue_qk(g + 1)) { ok = false; break; }
          } else {
            mma_commit(q_empty);  // every S = Q.K^T of this block has been issued
          }
          const uint32_t s = itv % RST, ph = (itv / RST) & 1;
          if (!mbar_wait(v_full + 8 * s, ph, p.status, (KERNEL_ID2 << 16) | 7)) { ok = false; break; }
          const uint32_t pb = g & 1, pph = (g >> 1) & 1;
          if (!mbar_wait(p_full + 8 * pb, pph, p.status, (KERNEL_ID2 << 16) | 8)) { ok = false; break; }
          const uint64_t dp = make_kmajor_sw128_desc(p_smem + (2 * hf + pb) * TILE_BYTES);
          tc_fence_after();
          const uint64_t dv = make_kmajor_sw128_desc(v_smem + s * TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < BKV / UMMA_K; ++kk) mma_f8_ss(tmem_o, dp + 2 * kk, dv + 2 * kk, idesc_pv, (j | kk) != 0);
          mma_commit(p_empty + 8 * pb);
          mma_commit(v_empty + 8 * s);
          ++itv;
          ++g;
        }
        ++wi;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
    // ------------------------------------------------------------------ softmax warps (one row per thread)
    const int hf = (warp - 4) >> 2;
    const int qrt = warp & 3;
    const int row = qrt * 32 + lane;
    const uint32_t hb = half_bars + 48 * hf;
    const uint32_t s_full = hb, s_empty = hb + 8, p_full = hb + 16, p_empty = hb + 32;
    const uint32_t tmem_s = tmem_base + 256 * hf, tmem_o = tmem_s + 128;
    uint8_t* p_gen = gen + (2 + 2 * hf) * TILE_BYTES;
    const uint32_t lane_sel = static_cast<uint32_t>(qrt * 32) << 16;
    const int nk64 = p.nkv * 2;
    T* out = static_cast<T*>(p.out);
    uint32_t g = 0;
    bool ok = true;
    // the score accumulator is free for the first S = Q.K^T (completion #0 of s_empty)
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(s_empty);
    for (int idx = blockIdx.x; idx < total && ok; idx += gridDim.x) {
      const PairWork w = get_pair<LISTS>(p, idx, npairs);
      const int h = w.h, qt = w.pr * 2 + hf;
      if (qt >= p.nq) continue;
      const int qrow = qt * BQ + row;
      T* orow;
      if (p.n_peers > 0) {
        const int dest = min(qrow / p.rows_per_peer, p.n_peers - 1);  // rows past Lq are never stored
        orow = static_cast<T*>(p.peers[dest]) + static_cast<int64_t>(qrow - dest * p.rows_per_peer) * p.out_ts + static_cast<int64_t>(h) * p.out_hs;
      } else {
        orow = out + static_cast<int64_t>(qrow) * p.out_ts + static_cast<int64_t>(h) * p.out_hs;
      }
      if (w.n == 0) {  // both blocks of the pair have empty lists: zeros
        if (qrow < p.Lq) {
#pragma unroll
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const float qsc = p.qs[h * p.nq + qt];
      float m_ref = -INFINITY, l = 0.f;
      // per-tile metadata (list entry and the two K-block scales) is fetched one tile ahead
      int e_next = pair_entry<LISTS>(w, 0);
      float ks0_next = p.ks[h * nk64 + 2 * (e_next >> 4)], ks1_next = p.ks[h * nk64 + 2 * (e_next >> 4) + 1];
      for (int j = 0; j < w.n; ++j) {
        const int e = e_next;
        const float sc0 = qsc * ks0_next, sc1 = qsc * ks1_next;
        if (j + 1 < w.n) {
          e_next = pair_entry<LISTS>(w, j + 1);
          ks0_next = p.ks[h * nk64 + 2 * (e_next >> 4)];
          ks1_next = p.ks[h * nk64 + 2 * (e_next >> 4) + 1];
        }
        const int t = LISTS ? (e >> 4) : j, halves = LISTS ? ((e >> (2 * hf)) & 3) : 3;
        const int valid = min(BKV, p.Lk - t * BKV);
        const bool full = (halves == 3) && (valid == BKV);
        if (!mbar_wait_warp(s_full, g & 1, p.status, (KERNEL_ID2 << 16) | 9)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[4][32];
        tmem_ld32(tmem_s + lane_sel + 0, s[0]);
        tmem_ld32(tmem_s + lane_sel + 32, s[1]);
        tmem_ld32(tmem_s + lane_sel + 64, s[2]);
        tmem_ld32(tmem_s + lane_sel + 96, s[3]);
        tmem_wait_ld();
        // the scores are in registers: hand the accumulator back to the MMA issuer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty);
        if (!full) {
          // masked columns (ragged tail or a 64-token half this block does not keep) become -inf: never the maximum, P = 0
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int col = c * 32 + i;
              const bool keep = (col < valid) && ((halves >> (col >> 6)) & 1);
              if (!keep) s[c][i] = 0xff800000u;
            }
        }
        // exact: both operands of the subtraction are integers below 2^24
        const float m_tile = fmaxf((tree_max64(s[0], s[1]) - S_MAGIC) * sc0, (tree_max64(s[2], s[3]) - S_MAGIC) * sc1);
        const bool grow = m_tile > m_ref + REF_SLACK;  // also true for the first tile with a valid score (m_ref = -inf)
        const bool rescale = __any_sync(0xffffffffu, grow);
        float alpha = 1.f;
        if (rescale) {
          const float m_new = grow ? m_tile : m_ref;
          alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
          l *= alpha;
          m_ref = m_new;
        }
        const float neg_m = (m_ref == -INFINITY) ? 0.f : (P_SHIFT - m_ref);
        uint32_t pk[32];
        float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float c0 = fmaf(-S_MAGIC, sc0, neg_m), c1 = fmaf(-S_MAGIC, sc1, neg_m);
        // no wait for the P buffer: S_j was issued behind the P.V of tile j - 2, its last reader (see sage_attn.cu)
        const uint32_t pb = g & 1;
        uint8_t* prow = p_gen + pb * TILE_BYTES + row * 128;
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          exp_chunk(s[hh], hh < 2 ? sc0 : sc1, hh < 2 ? c0 : c1, pk + 8 * hh, acc);
#pragma unroll
          for (int c = 2 * hh; c < 2 * hh + 2; ++c)
            *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        }
        l += ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
        fence_proxy_async_smem();
        if (rescale && j > 0) {
          // O *= alpha; the previous tile's P.V (the other P buffer) must have finished writing O
          if (!mbar_wait_warp(p_empty + 8 * (pb ^ 1), ((g - 1) >> 1) & 1, p.status, (KERNEL_ID2 << 16) | 10)) { ok = false; break; }
          tc_fence_after();
          uint32_t o[4][32];
          tmem_ld32(tmem_o + lane_sel + 0, o[0]);
          tmem_ld32(tmem_o + lane_sel + 32, o[1]);
          tmem_ld32(tmem_o + lane_sel + 64, o[2]);
          tmem_ld32(tmem_o + lane_sel + 96, o[3]);
          tmem_wait_ld();
          const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 r = __fmul2_rn(make_float2(__uint_as_float(o[c][i]), __uint_as_float(o[c][i + 1])), a2);
              o[c][i] = __float_as_uint(r.x);
              o[c][i + 1] = __float_as_uint(r.y);
            }
            tmem_st32(tmem_o + lane_sel + 32 * c, o[c]);
          }
          tmem_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full + 8 * pb);
        ++g;
      }
      if (!ok) break;
      // ---- epilogue of the block: wait for the last P.V, normalise, store
      if (!mbar_wait_warp(p_empty + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, p.status, (KERNEL_ID2 << 16) | 12)) { ok = false; break; }
      tc_fence_after();
      const float inv_l = (l > 0.f) ? (1.f / l) : 0.f;
      const float* vsh = p.vs + h * D;
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
    tmem_dealloc(tmem_base, TMEM_COLS2);
  }
}

}  // namespace dual
}  // namespace attn
}  // namespace ksb

using namespace ksb;

// Launches the two-block kernel on a dense problem.  Returns KSB_ERR_UNSUPPORTED (without an error text) when the
// build cannot run it, so that the caller falls back to the one-block kernel.
int ksb_attn_launch_dual(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const attn::Params& p, int dtype,
                         cudaStream_t st) {
  namespace d = attn::dual;
  const bool lists = p.offsets != nullptr;
  const void* fn = dtype == KSB_BF16 ? (lists ? reinterpret_cast<const void*>(d::sage_attn_dual_kernel<__nv_bfloat16, true>)
                                             : reinterpret_cast<const void*>(d::sage_attn_dual_kernel<__nv_bfloat16, false>))
                                     : (lists ? reinterpret_cast<const void*>(d::sage_attn_dual_kernel<__half, true>)
                                             : reinterpret_cast<const void*>(d::sage_attn_dual_kernel<__half, false>));
  // setmaxnreg.inc blocks until the CTA's register pool (registers at launch x threads) holds what it asks for:
  // refuse a build whose launch-time register count cannot cover the targets
  static int checked[4] = {0, 0, 0, 0};
  int& ck = checked[(dtype == KSB_BF16 ? 0 : 1) + (lists ? 2 : 0)];
  if (ck == 0) {
    cudaFuncAttributes fa{};
    if (cudaFuncGetAttributes(&fa, fn) != cudaSuccess) return fail(KSB_ERR_CUDA, "cannot read the attention kernel's attributes");
    ck = (fa.numRegs * d::THREADS2 >= 128 * d::PRODUCER_REGS + 256 * d::SOFTMAX_REGS) ? 1 : -1;
  }
  if (ck < 0) return KSB_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, d::SMEM_BYTES2) != cudaSuccess)
    return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");
  const int64_t total = (int64_t)p.H * ((p.nq + 1) / 2);
  const int grid = (int)(total < sm_count() ? total : sm_count());
  if (dtype == KSB_BF16) {
    if (lists) d::sage_attn_dual_kernel<__nv_bfloat16, true><<<grid, d::THREADS2, d::SMEM_BYTES2, st>>>(tq, tk, tv, p);
    else d::sage_attn_dual_kernel<__nv_bfloat16, false><<<grid, d::THREADS2, d::SMEM_BYTES2, st>>>(tq, tk, tv, p);
  } else {
    if (lists) d::sage_attn_dual_kernel<__half, true><<<grid, d::THREADS2, d::SMEM_BYTES2, st>>>(tq, tk, tv, p);
    else d::sage_attn_dual_kernel<__half, false><<<grid, d::THREADS2, d::SMEM_BYTES2, st>>>(tq, tk, tv, p);
  }
  return check_launch("sage attention (two Q blocks per CTA)");
}
