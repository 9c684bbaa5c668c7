// Sage-style quantised attention core on the Blackwell tensor cores, dense or block-sparse.
//
//   S = Q8 . K8^T            tcgen05.mma kind::i8   (s32 accumulator in tensor memory, see below)
//   X = float(S) * qs * ks   fp32, exp2 domain (softmax scale and log2 e are folded into Q8's scale)
//   P = exp2(X - r + 5)      fp32 online softmax against a per-row reference point r, rounded to e4m3
//   O += P . V8              tcgen05.mma kind::f8f6f4 (f32 accumulator in tensor memory)
//   out = O / l * vs
//
// Reference point: r follows the running row maximum lazily.  It moves (r = tile maximum, O and l scaled by
// 2^(r_old - r)) only in a tile whose row maximum exceeds it by more than 3.5; otherwise the tile is processed
// against the r it found.  P therefore never exceeds 2^(5 + 3.5) = 362 < 448, the e4m3 maximum, and after the
// first tile of a row almost no tile pays for a rescale of O.
//
// One CTA works on one (head, 128-row Q block) at a time and walks that block's list of 128-token KV
// tiles; two CTAs share an SM (256 tensor-memory columns and ~113 KB of shared memory each), so one
// CTA's softmax overlaps the other's MMAs.  Warp roles inside a CTA:
//   warp 0      TMA producer (Q block once per work item; K and V^T tiles through 2-deep rings)
//   warp 1      MMA issuer (single thread): S = Q.K^T for tile j+1 is queued before P.V of tile j; P alternates between two shared-memory buffers
//   warps 2,3   idle (they only donate registers)
//   warps 4..7  softmax: one row per thread; tcgen05.ld S, max, exp2, e4m3 P written to shared memory
//               in the 128-byte-swizzled K-major layout the MMA reads, O rescaled in tensor memory in the rare
//               tiles where a reference point of the warp moved; final normalisation and store
// The s32 score accumulator must read back as an fp32 number: every S = Q.K^T starts with one bf16 MMA
// (A = 1 at k = 0 and 8, B = 1.5 * 2^22 at k = 0 and 8, both from constant shared-memory blocks) that writes
// 12582912.0f = 0x4B400000 to all 128 x 128 accumulators, and the INT8 MMAs accumulate on top of those bits: taken as
// fp32 they are exactly 12582912 + S (|S| < 2^22), so the scores need no integer-to-float conversion and
// X - r + 5 = fma(bits_as_float, scale, -12582912 * scale - r + 5).
// Every mbarrier wait is bounded (see common.cuh).
//
// What bounds it: the 16 384 exp2 of a tile are 1024 cycles of the special-function unit against 512 tensor-pipe
// cycles, and special-function instructions share their issue queue with the shared-memory, barrier and
// tensor-memory instructions of the other CTA's softmax warp on the same scheduler, so every hand-off of a warp that
// is between two exponential phases waits behind its neighbour's exponentials.  Fewer hand-offs per tile is what
// pays: the P buffer needs no "free" barrier (the barrier that announces S_j is committed behind the P.V of tile
// j - 2, the buffer's last reader), and the lazy reference point removes most O rescales and their waits.
//
// Tensor-bound: 4 * 128 * 128 * 128 flop per visited (Q block, KV tile) pair.
#include "sage_attn_common.cuh"
#include "host_utils.h"

namespace ksb {
namespace attn {

template <typename T>
__global__ void __launch_bounds__(THREADS, 2)
sage_attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  uint8_t* gen = smem_raw;
  const uint32_t q_smem = base, p_smem = base + TILE_BYTES;
  const uint32_t k_smem = base + (1 + PST) * TILE_BYTES, v_smem = k_smem + KST * TILE_BYTES;
  const uint32_t const_smem = v_smem + VST * TILE_BYTES;
  const uint32_t bars = const_smem + CONST_BYTES;
  const uint32_t q_full = bars, q_empty = bars + 8, k_full = bars + 16, k_empty = bars + 32, v_full = bars + 48,
                 v_empty = bars + 64, s_full = bars + 80, s_empty = bars + 88, p_full = bars + 96, p_empty = bars + 112;  // p_*: PST each
  const uint32_t tmem_slot = bars + 8 * NUM_BARS + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + NUM_TILES * TILE_BYTES + CONST_BYTES + 8 * NUM_BARS + 16);
  uint8_t* p_gen = gen + TILE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.H * p.nq;
  if ((base & 1023u) != 0) {  // uniform over the CTA: the swizzled tiles need a 1024-byte aligned window
    if (threadIdx.x == 0) report_error(p.status, KSB_ERR_BAD_SMEM_ALIGNMENT, (KERNEL_ID << 16) | 99);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KST; ++s) { mbar_init(k_full + 8 * s, 1); mbar_init(k_empty + 8 * s, 1); }
    for (int s = 0; s < VST; ++s) { mbar_init(v_full + 8 * s, 1); mbar_init(v_empty + 8 * s, 1); }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 4);  // one arrival per softmax warp (an elected lane, after the warp has synchronised)
    for (int b = 0; b < PST; ++b) { mbar_init(p_full + 8 * b, 4); mbar_init(p_empty + 8 * b, 1); }
    fence_barrier_init();
  }
  if (threadIdx.x < CONST_BYTES / 4) {
    // bf16 operands of the pre-load MMA, every 16-byte chunk (8 values along k) the same within a block:
    // A chunk = {1, 0, ...}, B chunk = {1.5 * 2^22, 0, ...}; a row's k = 0..15 are two such chunks
    const uint32_t word = (threadIdx.x & 3) ? 0u : (threadIdx.x < CONST_BYTES / 8 ? 0x3F80u : 0x4AC0u);
    reinterpret_cast<uint32_t*>(gen + NUM_TILES * TILE_BYTES)[threadIdx.x] = word;
    fence_proxy_async_smem();  // read by the tensor core
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
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
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
      const uint64_t dq = make_kmajor_sw128_desc(q_smem);
      constexpr uint32_t idesc_pre = IDESC_BF16_F32(BQ, BKV);
      // constant blocks: every 16-byte chunk of a block is the same, so only the footprint of the descriptors
      // matters -- core matrices 16 B apart in both directions stay inside the 384-byte block
      const uint64_t dca = make_noswizzle_desc(const_smem, 16, 16);
      const uint64_t dcb = make_noswizzle_desc(const_smem + CONST_BYTES / 2, 16, 16);
      uint32_t wi = 0, itk = 0, itv = 0, g = 0;
      bool ok = true;
      auto issue_qk = [&](uint32_t gg) -> bool {
        const uint32_t s = itk % KST, ph = (itk / KST) & 1;
        if (!mbar_wait(k_full + 8 * s, ph, p.status, (KERNEL_ID << 16) | 4)) return false;
        if (!mbar_wait(s_empty, gg & 1, p.status, (KERNEL_ID << 16) | 5)) return false;  // S read by the softmax warps (completion #gg)
        tc_fence_after();
        const uint64_t dk = make_kmajor_sw128_desc(k_smem + s * TILE_BYTES);
        mma_bf16_ss(tmem_s, dca, dcb, idesc_pre, 0);  // every accumulator = 12582912.0f
#pragma unroll
        for (int kk = 0; kk < D / UMMA_K; ++kk) mma_i8_ss(tmem_s, dq + 2 * kk, dk + 2 * kk, idesc_qk, 1);  // on top of the pre-load
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
          const uint32_t pb = g & 1, pph = (g >> 1) & 1;
          if (!mbar_wait(p_full + 8 * pb, pph, p.status, (KERNEL_ID << 16) | 8)) { ok = false; break; }
          const uint64_t dp = make_kmajor_sw128_desc(p_smem + pb * TILE_BYTES);
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
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    // ------------------------------------------------------------------ softmax warps (one row per thread)
    const int qrt = warp & 3;
    const int row = qrt * 32 + lane;
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
      const Work w = get_work(p, idx);
      const int qrow = w.qt * BQ + row;
      T* orow;
      if (p.n_peers > 0) {
        const int dest = min(qrow / p.rows_per_peer, p.n_peers - 1);  // rows past Lq are never stored
        orow = static_cast<T*>(p.peers[dest]) + static_cast<int64_t>(qrow - dest * p.rows_per_peer) * p.out_ts + static_cast<int64_t>(w.h) * p.out_hs;
      } else {
        orow = out + static_cast<int64_t>(qrow) * p.out_ts + static_cast<int64_t>(w.h) * p.out_hs;
      }
      if (w.n == 0) {
        if (qrow < p.Lq) {
#pragma unroll
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const float qsc = p.qs[w.h * p.nq + w.qt];
      float m_ref = -INFINITY, l = 0.f;
      // per-tile metadata (list entry and the two K-block scales) is fetched one tile ahead
      int e_next = entry_at(w, 0);
      float ks0_next = p.ks[w.h * nk64 + 2 * (e_next >> 2)], ks1_next = p.ks[w.h * nk64 + 2 * (e_next >> 2) + 1];
      for (int j = 0; j < w.n; ++j) {
        const int e = e_next;
        const float sc0 = qsc * ks0_next, sc1 = qsc * ks1_next;
        if (j + 1 < w.n) {
          e_next = entry_at(w, j + 1);
          ks0_next = p.ks[w.h * nk64 + 2 * (e_next >> 2)];
          ks1_next = p.ks[w.h * nk64 + 2 * (e_next >> 2) + 1];
        }
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
        // the scores are in registers: hand the accumulator back to the MMA issuer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty);
        if (!full) {
          // masked columns (ragged tail or dropped 64-token half) become -inf: never the maximum, P = 0
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
        // The reference point moves only for a row whose tile maximum outgrew it by more than the slack; O and l are
        // rescaled in the tiles in which that happened to some row of the warp (the other rows get the factor 1).
        const bool grow = m_tile > m_ref + REF_SLACK;  // also true for the first tile with a valid score (m_ref = -inf)
        const bool rescale = __any_sync(0xffffffffu, grow);
        float alpha = 1.f;
        if (rescale) {
          const float m_new = grow ? m_tile : m_ref;
          alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
          l *= alpha;
          m_ref = m_new;
        }
        // P = exp2(X - m_ref + 5) -> e4m3, packed 4 per word; masked columns give exactly 0
        const float neg_m = (m_ref == -INFINITY) ? 0.f : (P_SHIFT - m_ref);
        uint32_t pk[32];
        float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float c0 = fmaf(-S_MAGIC, sc0, neg_m), c1 = fmaf(-S_MAGIC, sc1, neg_m);
        // This tile's P buffer was last read by the P.V of two tiles ago, and that P.V has completed: S_j was issued
        // behind it and the barrier awaited above covers everything issued before S_j.  Each 32-score chunk is stored
        // as soon as it is packed (row `row` of the K-major tile: 16-byte chunks, chunk index XORed with (row & 7)).
        const uint32_t pb = g & 1;
        uint8_t* prow = p_gen + pb * TILE_BYTES + row * 128;
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          exp_chunk(s[h], h < 2 ? sc0 : sc1, h < 2 ? c0 : c1, pk + 8 * h, acc);
#pragma unroll
          for (int c = 2 * h; c < 2 * h + 2; ++c)
            *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        }
        l += ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
        fence_proxy_async_smem();
        if (rescale && j > 0) {
          // O *= alpha with all four 32-column chunks in flight (the score registers are dead by now); the
          // previous tile's P.V (the other P buffer) must have finished writing O
          if (!mbar_wait_warp(p_empty + 8 * (pb ^ 1), ((g - 1) >> 1) & 1, p.status, (KERNEL_ID << 16) | 10)) { ok = false; break; }
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
      // ---- epilogue of the work item: wait for the last P.V, normalise, store
      if (!mbar_wait_warp(p_empty + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, p.status, (KERNEL_ID << 16) | 12)) { ok = false; break; }
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

int ksb_attn_launch_dual(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const attn::Params& p, int dtype, cudaStream_t st);

// 1: dense problems run on the kernel with two Q blocks per CTA (sage_attn_dual.cu); 0: always one block per CTA
static int g_dual_mode = 1;

extern "C" int ksb_attn_dual_mode(int mode) {
  const int previous = g_dual_mode;
  if (mode == 0 || mode == 1) g_dual_mode = mode;
  return previous;
}

static int attn_entry(bool pair_lists, const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                      const float* vs, int64_t H, int64_t Lq, int64_t Lk, const int32_t* tile_offsets,
                      const int32_t* tile_entries, const int32_t* q_order, void* out, int dtype,
                      int64_t out_token_stride, int64_t out_head_stride, void* const* peer_out, int n_peers,
                      int64_t rows_per_peer, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (H <= 0 || Lq <= 0 || Lk <= 0) return fail(KSB_ERR_INVALID, "bad shape H=%lld Lq=%lld Lk=%lld", (long long)H, (long long)Lq, (long long)Lk);
  if (!q8 || !qs || !k8 || !ks || !vt || !vs || (!out && !peer_out)) return fail(KSB_ERR_INVALID, "null pointer");
  if (peer_out) {
    if (n_peers < 1 || n_peers > KSB_MAX_PEERS || rows_per_peer <= 0 || rows_per_peer * n_peers < Lq || rows_per_peer > INT32_MAX)
      return fail(KSB_ERR_INVALID, "peer_out needs 1..%d peers and rows_per_peer * n_peers >= Lq", KSB_MAX_PEERS);
    for (int i = 0; i < n_peers; ++i)
      if (!peer_out[i] || !aligned16(peer_out[i])) return fail(KSB_ERR_INVALID, "peer buffer %d null or unaligned", i);
  } else {
    n_peers = 0;
  }
  if ((tile_offsets == nullptr) != (tile_entries == nullptr)) return fail(KSB_ERR_INVALID, "tile_offsets and tile_entries must both be given or both be NULL");
  if ((out && !aligned16(out)) || out_token_stride % 8 != 0 || out_head_stride % 8 != 0) return fail(KSB_ERR_INVALID, "out must be 16-byte aligned with strides multiple of 8 elements");
  const int64_t nq = (Lq + 127) / 128, nkv = (Lk + 127) / 128;
  if (H * nq > INT32_MAX / 256 || H * nkv > INT32_MAX / 256) return fail(KSB_ERR_INVALID, "problem too large");
  CUtensorMap tq, tk, tv;
  if (int rc = encode_tmap_2d(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q8, 128, (uint64_t)(H * nq * 128), 128, 128, 128)) return rc;
  if (int rc = encode_tmap_2d(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, 128, (uint64_t)(H * nkv * 128), 128, 128, 128)) return rc;
  if (int rc = encode_tmap_2d(&tv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, vt, (uint64_t)(nkv * 128), (uint64_t)(H * 128), (uint64_t)(nkv * 128), 128, 128)) return rc;
  attn::Params p{};
  p.qs = qs; p.ks = ks; p.vs = vs;
  p.H = (int)H; p.Lq = (int)Lq; p.Lk = (int)Lk; p.nq = (int)nq; p.nkv = (int)nkv;
  p.offsets = tile_offsets; p.entries = tile_entries; p.order = q_order;
  p.out = out; p.out_ts = out_token_stride; p.out_hs = out_head_stride;
  p.n_peers = n_peers; p.rows_per_peer = (int)rows_per_peer;
  for (int i = 0; i < n_peers; ++i) p.peers[i] = peer_out[i];
  p.status = status_words();
  if (!p.status) return fail(KSB_ERR_CUDA, "status words unavailable");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pair_lists) {
    if (!tile_offsets) return fail(KSB_ERR_INVALID, "ksb_sage_attn_pairs needs the per-pair tile lists");
    const int rc = ksb_attn_launch_dual(tq, tk, tv, p, dtype, st);
    return rc == KSB_ERR_UNSUPPORTED ? fail(KSB_ERR_UNSUPPORTED, "the two-block attention kernel cannot run in this build") : rc;
  }
  if (g_dual_mode == 1 && !tile_offsets && !q_order) {
    const int rc = ksb_attn_launch_dual(tq, tk, tv, p, dtype, st);
    if (rc != KSB_ERR_UNSUPPORTED) return rc;
  }
  const int64_t total = H * nq;
  const int64_t cap = 2 * (int64_t)sm_count();
  const int grid = (int)(total < cap ? total : cap);
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

extern "C" int ksb_sage_attn(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                             const float* vs, int64_t H, int64_t Lq, int64_t Lk, const int32_t* tile_offsets,
                             const int32_t* tile_entries, const int32_t* q_order, void* out, int dtype,
                             int64_t out_token_stride, int64_t out_head_stride, void* const* peer_out, int n_peers,
                             int64_t rows_per_peer, ksb_stream_t stream) {
  return attn_entry(false, q8, qs, k8, ks, vt, vs, H, Lq, Lk, tile_offsets, tile_entries, q_order, out, dtype, out_token_stride,
                    out_head_stride, peer_out, n_peers, rows_per_peer, stream);
}

extern "C" int ksb_sage_attn_pairs(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt,
                                   const float* vs, int64_t H, int64_t Lq, int64_t Lk, const int32_t* pair_offsets,
                                   const int32_t* pair_entries, const int32_t* pair_order, void* out, int dtype,
                                   int64_t out_token_stride, int64_t out_head_stride, void* const* peer_out, int n_peers,
                                   int64_t rows_per_peer, ksb_stream_t stream) {
  return attn_entry(true, q8, qs, k8, ks, vt, vs, H, Lq, Lk, pair_offsets, pair_entries, pair_order, out, dtype, out_token_stride,
                    out_head_stride, peer_out, n_peers, rows_per_peer, stream);
}
