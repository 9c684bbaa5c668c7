// FP8 (e4m3) GEMM with per-token x per-output-channel scales on the Blackwell tensor cores.
//
//   out[m,n] = epi( (sum_k A[m,k] * W[n,k])_f32 * sa[m] * sw[n] + bias[n] )
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128 x 128 B tile of A and 256 x 128 B tile of W per stage, 128-byte swizzle,
//               STAGES-deep ring in shared memory, completion on mbarriers
//   warp 1      MMA issuer: one thread issues tcgen05.mma (kind::f8f6f4, M128 N256 K32) from shared-memory
//               descriptors into a tensor-memory accumulator; two accumulators (2 x 256 columns) alternate
//               so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread), apply scales / bias / fused
//               GELU-tanh or gated residual, convert to half, store.  The scatter epilogue (fused Ulysses
//               exchange) stages 128-byte row pieces in shared memory and sends each with one bulk copy to the
//               memory of the GPU that owns the head: NVLink carries 128-byte writes, not 16-byte ones
// Tiles are visited in groups of `group_m` row-tiles (all column tiles of a group, row-tile fastest) so that
// CTAs running at the same time share operand tiles in L2.  The weight is streamed from HBM once per group,
// the group's activation rows stay in L2 while the group sweeps the columns: the host picks the group height so
// that those rows take about 32 MB (32 row-tiles at K = 5120, 16 at K = 13824).  Ragged M, N, K edges rely on TMA zero fill for loads and on predicated stores.
//
// Tensor-bound: 2*M*N*K flop per launch; minimal traffic M*K + N*K + 2*M*N bytes.
#include "../../include/ksana_b200.h"
#include "common.cuh"
#include "host_utils.h"

namespace ksb {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 128;  // BK in bytes == e4m3 elements
constexpr int UMMA_K = 32;
constexpr int A_BYTES = BM * BK;
constexpr int threads_for(int epilogue_warps) { return 64 + 32 * epilogue_warps; }
constexpr int TMEM_COLS = 512;
constexpr int KERNEL_ID = 1;
// Output staging of the scatter epilogue: one 128-byte row piece per epilogue thread, rows 144 bytes apart (the
// 16-byte skew keeps the 16-byte shared-memory stores of a quarter warp on distinct banks).
constexpr int SCATTER_COLS = 64, SCATTER_ROW_BYTES = SCATTER_COLS * 2 + 16, SCATTER_BYTES = 128 * SCATTER_ROW_BYTES;
// CTAS = 1: every CTA computes 128 x 256 tiles on its own.  CTAS = 2: two CTAs of a cluster compute one 256 x 256
// tile with tcgen05.mma.cta_group::2 -- each holds its 128 rows of A and 128 of the 256 rows of the W tile, so a
// stage is 32 KB instead of 48 KB per CTA (a third less operand traffic from L2 and into shared memory per flop)
// and six stages fit where four did.
//
// EW epilogue warps: 4 (one thread per accumulator row and all 256 columns; the scatter epilogue) or 8 (two threads per
// row, 128 columns each: GELU and the gated residual cost 15 - 20 instructions per element, and with four warps the
// epilogue of a tile took longer than the main loop of the next one at K = 5120).
template <int CTAS, int EW> struct Cfg {
  static constexpr int B_ROWS = BN / CTAS;
  static constexpr int B_BYTES = B_ROWS * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = CTAS == 1 ? 4 : 6;
  static constexpr int THREADS = threads_for(EW);
  static constexpr int COLP_BYTES = 3 * BN * 4 + 128 * 4;  // [sw | bias | gate] x BN, then one float per row (sums of squares of the upper column half)
  // dynamic shared memory: [1024 align slack][STAGES x (A | B)][col params][barriers][scatter staging (4 warps only)]
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + COLP_BYTES + 256 + (EW == 4 ? SCATTER_BYTES : 0);
};

struct Params {
  int M, N, K;
  int group_m;  // row-tiles per rasterisation group
  const float* sa;
  const float* sw;
  const void* bias;
  void* out;
  int64_t ldo;
  int epilogue;
  const void* resid;
  int64_t ldr;
  const void* gate;
  int64_t gate_rows;
  int rows_per_gate;  // M / gate_rows: row m reads gate row m / rows_per_gate
  int* status;
  // KSB_EPI_SCATTER_HEADS (fused QKV projection + Ulysses exchange): the output row of local token m and
  // column n = which * C + head * 128 + d goes to peer head / heads_per_peer, into its [tokens_all, 3, heads_per_peer,
  // 128] buffer at token (rank * M + m); the sum of squares of every row of each 256-column tile is written to
  // tile_sumsq[tile_n][m] for the tiles of the Q and K thirds.
  void* peers[KSB_MAX_PEERS];
  int n_peers, rank, heads_per_peer, C;
  float* tile_sumsq;
  int sumsq_cols;   // tiles that start below this column write their row sums of squares (any epilogue that stores rows)
  int fetch_ahead;  // gated-residual epilogue: fetch residual / gate one chunk ahead (short main loops)
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

__device__ __forceinline__ void bulk_store_128(void* dst, uint32_t src_smem) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 128;" ::"l"(dst), "r"(src_smem) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_source_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float gelu_tanh(float x) {
  // 0.5 x (1 + tanh(u)) = x * sigmoid(2u),  u = sqrt(2/pi) (x + 0.044715 x^3)
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  // fast reciprocal: two instructions and no slow path when exp overflows to inf (the quotient is then 0, as it
  // should be); the IEEE division costs ~10 instructions per element and made this epilogue the bottleneck
  return __fdividef(x, 1.f + __expf(-2.f * u));
}

template <typename T, int CTAS, int EW>
__global__ void __launch_bounds__(threads_for(EW), 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, const Params p) {
  using C = Cfg<CTAS, EW>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, COLP_BYTES = C::COLP_BYTES;
  static_assert(EW == 4 || EW == 8, "four or eight epilogue warps");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  float* colp = reinterpret_cast<float*>(gen + STAGES * STAGE_BYTES);  // [sw | bias | gate] x BN
  float* ssq_upper = colp + 3 * BN;                                   // [128] (eight epilogue warps only)
  const uint32_t bars = base + STAGES * STAGE_BYTES + COLP_BYTES;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES, tfull0 = bars + 16 * STAGES, tempty0 = tfull0 + 16;
  const uint32_t tmem_slot = tempty0 + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + STAGES * STAGE_BYTES + COLP_BYTES + 16 * STAGES + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A pair walks the 256-row tiles together; CTA `crank` of the pair owns rows crank * 128 .. + 127 of each.
  const uint32_t crank = CTAS == 2 ? cluster_ctarank() : 0u;
  const int worker = CTAS == 2 ? blockIdx.x >> 1 : blockIdx.x, workers = CTAS == 2 ? gridDim.x >> 1 : gridDim.x;
  const int tiles_m = (p.M + CTAS * BM - 1) / (CTAS * BM), tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // the producer's expect_tx arrival (of the even CTA in a pair) + the bytes of every load
      mbar_init(empty0 + 8 * s, 1);  // one commit (delivered to both CTAs of a pair)
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, EW * CTAS);  // one arrival per epilogue warp (of both CTAs, at the even CTA)
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    if (CTAS == 2) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // the partner's barriers exist before anything is signalled to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_w);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = worker; tile < num_tiles && ok; tile += workers) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
        for (int k = 0; k < num_k; ++k, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1, p.status, (KERNEL_ID << 16) | 1)) { ok = false; break; }
          const uint32_t sa = base + s * STAGE_BYTES;
          if (CTAS == 2) {
            // both CTAs' loads of this stage are counted by the even CTA's barrier, whose MMA thread consumes them
            const uint32_t full_even = mapa_shared(full0 + 8 * s, 0);
            if (crank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
            tma_load_2d_pair(sa, &tmap_a, full_even, k * BK, (tm * 2 + (int)crank) * BM);
            tma_load_2d_pair(sa + A_BYTES, &tmap_w, full_even, k * BK, tn * BN + (int)crank * C::B_ROWS);
          } else {
            mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
            tma_load_2d(sa, &tmap_a, full0 + 8 * s, k * BK, tm * BM);
            tma_load_2d(sa + A_BYTES, &tmap_w, full0 + 8 * s, k * BK, tn * BN);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (in a pair: the even CTA's)
    if (lane == 0 && crank == 0) {
      constexpr uint32_t idesc = IDESC_F8_E4M3_F32(CTAS * BM, BN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = worker; tile < num_tiles && ok; tile += workers, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!mbar_wait(tempty0 + 8 * acc, aph ^ 1, p.status, (KERNEL_ID << 16) | 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int k = 0; k < num_k; ++k, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(full0 + 8 * s, ph, p.status, (KERNEL_ID << 16) | 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * STAGE_BYTES;
          const uint64_t da = make_kmajor_sw128_desc(sa), db = make_kmajor_sw128_desc(sa + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            if (CTAS == 2) mma_f8_ss_pair(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (k | kk) != 0);
            else mma_f8_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (k | kk) != 0);
          }
          // frees the stage (in both CTAs) once these MMAs have read it
          if (CTAS == 2) mma_commit_pair(empty0 + 8 * s); else mma_commit(empty0 + 8 * s);
        }
        if (ok) {
          if (CTAS == 2) mma_commit_pair(tfull0 + 8 * acc); else mma_commit(tfull0 + 8 * acc);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2 .. 2 + EW - 1)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const int et = threadIdx.x - 64;
    constexpr int ET = EW * 32;           // epilogue threads
    constexpr int CW = BN / (EW / 4);     // columns per thread: all 256, or the lower / upper 128
    const int cbeg = ((warp - 2) >> 2) * CW, cend = cbeg + CW;
    uint8_t* stage_row = gen + STAGES * STAGE_BYTES + COLP_BYTES + 256 + (EW == 4 ? et : 0) * SCATTER_ROW_BYTES;
    uint32_t tcount = 0;
    bool failed = false;
    T* out = static_cast<T*>(p.out);
    const uint32_t tempty_even = CTAS == 2 ? mapa_shared(tempty0, 0) : 0u;
    for (int tile = worker; tile < num_tiles; tile += workers, ++tcount) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
      if (CTAS == 2) tm = tm * 2 + (int)crank;  // this CTA's 128 rows of the 256-row tile
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      // All four epilogue warps leave together if any of their waits ran out (a warp must never be
      // left alone at the named barrier below); the same barrier protects the reuse of colp.
      if (named_bar_or(1, ET, failed)) break;
      // stage the per-column parameters of this tile
      for (int c = et; c < BN; c += ET) {
        const int n = tn * BN + c;
        const bool in = n < p.N;
        colp[c] = in ? p.sw[n] : 0.f;
        colp[BN + c] = (in && p.bias) ? HalfOps<T>::to_f(static_cast<const T*>(p.bias)[n]) : 0.f;
        colp[2 * BN + c] = (in && p.gate && p.gate_rows == 1) ? HalfOps<T>::to_f(static_cast<const T*>(p.gate)[n]) : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
      if (!mbar_wait_warp(tfull0 + 8 * acc, aph, p.status, (KERNEL_ID << 16) | 4)) { failed = true; continue; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float sa = row_ok ? p.sa[row] : 0.f;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      T* orow = out + static_cast<int64_t>(row) * p.ldo + tn * BN;
      const T* rrow = p.resid ? static_cast<const T*>(p.resid) + static_cast<int64_t>(row) * p.ldr + tn * BN : nullptr;
      const T* grow = (p.gate && p.gate_rows != 1) ? static_cast<const T*>(p.gate) + static_cast<int64_t>(row / p.rows_per_gate) * p.N + tn * BN : nullptr;
      const bool scatter = EW == 4 && p.epilogue == KSB_EPI_SCATTER_HEADS;
      const bool want_ssq = p.tile_sumsq != nullptr && tn * BN < p.sumsq_cols;
      float ssq = 0.f;
      // The residual (and a per-row gate) are fetched one 32-column chunk ahead when the main loop is short
      // (K <= 8192): a thread reads its own row, so these are latency-bound scattered loads, and with 40 k-steps
      // per tile the epilogue must not wait for them (o-projection 1.94 -> 1.62 ms).  With a long main loop the
      // epilogue is hidden anyway and fetching ahead measured slower (down-projection 3.96 -> 4.37 ms).
      const bool gated = p.epilogue == KSB_EPI_GATE_RESIDUAL && row_ok;
      uint4 rv_next[4], gv_next[4];
      auto fetch = [&](int c0) {
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          const int cb = c0 + v8 * 8;
          const bool in = gated && c0 < cend && tn * BN + cb < p.N;
          rv_next[v8] = in ? *reinterpret_cast<const uint4*>(rrow + cb) : make_uint4(0, 0, 0, 0);
          gv_next[v8] = (in && grow) ? *reinterpret_cast<const uint4*>(grow + cb) : make_uint4(0, 0, 0, 0);
        }
      };
      if (p.fetch_ahead) fetch(cbeg);
#pragma unroll 1
      for (int c0 = cbeg; c0 < cend; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(t_row + c0, r);
        uint4 rv_cur[4], gv_cur[4];
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          rv_cur[v8] = rv_next[v8];
          gv_cur[v8] = gv_next[v8];
        }
        if (p.fetch_ahead) {
          fetch(c0 + 32);
        } else {
          fetch(c0);
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            rv_cur[v8] = rv_next[v8];
            gv_cur[v8] = gv_next[v8];
          }
        }
        tmem_wait_ld();
        if (row_ok) {
          // the staged row piece is rewritten every 64 columns: wait until the previous bulk copy has read it
          if (scatter && (c0 & 32) == 0) bulk_wait_source_read();
#pragma unroll
          for (int v8 = 0; v8 < 4; ++v8) {
            const int cb = c0 + v8 * 8;
            if (tn * BN + cb < p.N) {
              float y[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float a = __uint_as_float(r[v8 * 8 + i]);
                y[i] = a * sa * colp[cb + i] + colp[BN + cb + i];
              }
              if (p.epilogue == KSB_EPI_GELU_TANH) {
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = gelu_tanh(HalfOps<T>::to_f(HalfOps<T>::from_f(y[i])));
              } else if (p.epilogue == KSB_EPI_GATE_RESIDUAL) {
                const T* rt = reinterpret_cast<const T*>(&rv_cur[v8]);
                const T* gt = reinterpret_cast<const T*>(&gv_cur[v8]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float g = grow ? HalfOps<T>::to_f(gt[i]) : colp[2 * BN + cb + i];
                  y[i] = fmaf(HalfOps<T>::to_f(HalfOps<T>::from_f(y[i])), g, HalfOps<T>::to_f(rt[i]));
                }
              }
              uint4 o;
              T* ot = reinterpret_cast<T*>(&o);
#pragma unroll
              for (int i = 0; i < 8; ++i) ot[i] = HalfOps<T>::from_f(y[i]);
              if (scatter) {
                *reinterpret_cast<uint4*>(stage_row + (cb & 63) * 2) = o;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float v = HalfOps<T>::to_f(ot[i]);
                  ssq = fmaf(v, v, ssq);
                }
              } else {
                *reinterpret_cast<uint4*>(orow + cb) = o;
                if (want_ssq) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    const float v = HalfOps<T>::to_f(ot[i]);
                    ssq = fmaf(v, v, ssq);
                  }
                }
              }
            }
          }
          if (scatter && (c0 & 32) != 0) {
            // 64 columns staged: they never straddle a head (128 columns) or a Q / K / V third (C % 256 == 0)
            const int n = tn * BN + c0 - 32;
            const int which = n / p.C, c = n - which * p.C;
            const int head = c >> 7, dest = head / p.heads_per_peer, hl = head - dest * p.heads_per_peer;
            T* dst = static_cast<T*>(p.peers[dest]) +
                     ((static_cast<int64_t>(p.rank) * p.M + row) * 3 + which) * (static_cast<int64_t>(p.heads_per_peer) * 128) + hl * 128 + (c & 127);
            fence_async_proxy_smem();
            bulk_store_128(dst, smem_u32(stage_row));
          }
        }
      }
      if (EW == 8) {
        if (want_ssq) {  // uniform over the tile: the two threads of a row add their halves (lower + upper)
          if (cbeg != 0) ssq_upper[q * 32 + lane] = ssq;
          asm volatile("bar.sync 1, %0;" ::"n"(ET) : "memory");
          if (cbeg == 0 && row_ok) p.tile_sumsq[static_cast<int64_t>(tn) * p.M + row] = ssq + ssq_upper[q * 32 + lane];
        }
      } else {
        if (want_ssq && row_ok) p.tile_sumsq[static_cast<int64_t>(tn) * p.M + row] = ssq;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) mbar_arrive_cluster(tempty_even + 8 * acc); else mbar_arrive(tempty0 + 8 * acc);
      }
    }
    bulk_wait_all();  // no bulk copy of this thread may outlive the kernel's shared memory
  }

  // ------------------------------------------------------------------ common exit
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (CTAS == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace ksb

using namespace ksb;

static int launch_gemm(gemm::Params& p, const void* a, const void* w, int dtype, cudaStream_t st);

extern "C" int ksb_fp8_gemm_qkv_scatter(const void* a, const float* a_scale, const void* w, const float* w_scale,
                                        const void* bias, int64_t M, int64_t C, int64_t K, int dtype, void* const* peer_out,
                                        int n_peers, int rank, int64_t heads, float* tile_sumsq, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (M <= 0 || C <= 0 || K <= 0 || M > INT32_MAX / 4 || C > INT32_MAX / 4 || K > INT32_MAX) return fail(KSB_ERR_INVALID, "bad shape");
  if (K % 16 != 0 || C % 256 != 0 || heads * 128 != C) return fail(KSB_ERR_INVALID, "need K %% 16 == 0, C %% 256 == 0 and C == heads * 128");
  if (n_peers < 1 || n_peers > KSB_MAX_PEERS || rank < 0 || rank >= n_peers || heads % n_peers != 0)
    return fail(KSB_ERR_INVALID, "n_peers must be 1..%d, rank inside it, heads divisible by it", KSB_MAX_PEERS);
  if (!a || !a_scale || !w || !w_scale || !peer_out || !tile_sumsq) return fail(KSB_ERR_INVALID, "null pointer");
  gemm::Params p{};
  p.rows_per_gate = 1;
  p.M = (int)M; p.N = (int)(3 * C); p.K = (int)K;
  p.sa = a_scale; p.sw = w_scale; p.bias = bias; p.out = peer_out[rank]; p.ldo = 3 * C; p.epilogue = KSB_EPI_SCATTER_HEADS;
  for (int i = 0; i < n_peers; ++i) {
    if (!peer_out[i] || !aligned16(peer_out[i])) return fail(KSB_ERR_INVALID, "peer buffer %d null or unaligned", i);
    p.peers[i] = peer_out[i];
  }
  p.n_peers = n_peers; p.rank = rank; p.heads_per_peer = (int)(heads / n_peers); p.C = (int)C; p.tile_sumsq = tile_sumsq; p.sumsq_cols = (int)(2 * C);
  return launch_gemm(p, a, w, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int ksb_fp8_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale,
                            const void* bias, int64_t M, int64_t N, int64_t K, void* out, int dtype, int64_t ldo,
                            int epilogue, const void* resid, int64_t ldr, const void* gate, int64_t gate_rows,
                            ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (M < 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(KSB_ERR_INVALID, "bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (K % 16 != 0 || N % 8 != 0) return fail(KSB_ERR_INVALID, "K must be a multiple of 16 and N of 8 (K=%lld N=%lld)", (long long)K, (long long)N);
  if (M == 0) return 0;
  if (!a || !a_scale || !w || !w_scale || !out) return fail(KSB_ERR_INVALID, "null pointer");
  if (ldo < N || ldo % 8 != 0 || !aligned16(out)) return fail(KSB_ERR_INVALID, "out must be 16-byte aligned with ldo >= N, ldo %% 8 == 0");
  if (epilogue < KSB_EPI_NONE || epilogue > KSB_EPI_GATE_RESIDUAL) return fail(KSB_ERR_INVALID, "unknown epilogue %d", epilogue);
  if (epilogue == KSB_EPI_GATE_RESIDUAL) {
    if (!resid || !gate) return fail(KSB_ERR_INVALID, "gate-residual epilogue needs resid and gate");
    if (ldr < N || ldr % 8 != 0 || !aligned16(resid) || !aligned16(gate)) return fail(KSB_ERR_INVALID, "resid/gate alignment");
    if (gate_rows < 1 || gate_rows > M || M % gate_rows != 0) return fail(KSB_ERR_INVALID, "gate_rows must divide M");
  } else {
    resid = nullptr;
    gate = nullptr;
  }
  gemm::Params p{};
  p.rows_per_gate = 1;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.sa = a_scale; p.sw = w_scale; p.bias = bias; p.out = out; p.ldo = ldo; p.epilogue = epilogue;
  p.resid = resid; p.ldr = ldr; p.gate = gate; p.gate_rows = gate_rows;
  p.rows_per_gate = (gate && gate_rows > 0) ? static_cast<int>(M / gate_rows) : 1;
  return launch_gemm(p, a, w, dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int ksb_fp8_gemm_rowstats(const void* a, const float* a_scale, const void* w, const float* w_scale,
                                     const void* bias, int64_t M, int64_t N, int64_t K, void* out, int dtype, int64_t ldo,
                                     float* tile_sumsq, int64_t sumsq_cols, ksb_stream_t stream) {
  if (dtype != KSB_BF16 && dtype != KSB_FP16) return fail(KSB_ERR_INVALID, "dtype must be KSB_BF16 or KSB_FP16");
  if (M <= 0 || N <= 0 || K <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(KSB_ERR_INVALID, "bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
  if (K % 16 != 0 || N % 8 != 0) return fail(KSB_ERR_INVALID, "K must be a multiple of 16 and N of 8 (K=%lld N=%lld)", (long long)K, (long long)N);
  if (!a || !a_scale || !w || !w_scale || !out || !tile_sumsq) return fail(KSB_ERR_INVALID, "null pointer");
  if (ldo < N || ldo % 8 != 0 || !aligned16(out)) return fail(KSB_ERR_INVALID, "out must be 16-byte aligned with ldo >= N, ldo %% 8 == 0");
  if (sumsq_cols <= 0 || sumsq_cols > N || sumsq_cols % gemm::BN != 0)
    return fail(KSB_ERR_INVALID, "sumsq_cols must be a positive multiple of %d and <= N", gemm::BN);
  gemm::Params p{};
  p.rows_per_gate = 1;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.sa = a_scale; p.sw = w_scale; p.bias = bias; p.out = out; p.ldo = ldo; p.epilogue = KSB_EPI_NONE;
  p.tile_sumsq = tile_sumsq; p.sumsq_cols = (int)sumsq_cols;
  return launch_gemm(p, a, w, dtype, static_cast<cudaStream_t>(stream));
}

// epilogue warps of every launch that writes local rows (the scatter epilogue always has four)
#ifndef KSB_GEMM_EPILOGUE_WARPS
#define KSB_GEMM_EPILOGUE_WARPS 8
#endif

// 0: every CTA on its own (cta_group::1); 1: CTA pairs (cta_group::2).
// The pair form is the default: same bits, 2 - 20 % less time at the 75 600-token shapes under the power cap.
static int g_pair_mode = 1;

extern "C" int ksb_gemm_pair_mode(int mode) {
  const int previous = g_pair_mode;
  if (mode == 0 || mode == 1) g_pair_mode = mode;
  return previous;
}

template <typename T, int CTAS, int EW>
static int launch_gemm_as(const gemm::Params& p, const CUtensorMap& ta, const CUtensorMap& tw, int grid, cudaStream_t st) {
  auto kernel = gemm::fp8_gemm_kernel<T, CTAS, EW>;
  constexpr int smem = gemm::Cfg<CTAS, EW>::SMEM_BYTES;
  constexpr int threads = gemm::Cfg<CTAS, EW>::THREADS;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return fail(KSB_ERR_CUDA, "cannot raise dynamic shared memory limit");
  if (CTAS == 1) {
    kernel<<<grid, threads, smem, st>>>(ta, tw, p);
    return check_launch("fp8 gemm");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, ta, tw, p) != cudaSuccess) return fail(KSB_ERR_CUDA, "cluster launch failed: %s", cudaGetErrorString(cudaGetLastError()));
  return check_launch("fp8 gemm (CTA pairs)");
}

static int launch_gemm(gemm::Params& p, const void* a, const void* w, int dtype, cudaStream_t st) {
  const int64_t M = p.M, N = p.N, K = p.K;
  p.fetch_ahead = K <= 8192 ? 1 : 0;
  const bool pair = g_pair_mode == 1 && sm_count() >= 2;
  CUtensorMap ta, tw;
  if (int rc = encode_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a, (uint64_t)K, (uint64_t)M, (uint64_t)K, gemm::BK, gemm::BM)) return rc;
  if (int rc = encode_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w, (uint64_t)K, (uint64_t)N, (uint64_t)K, gemm::BK, pair ? gemm::BN / 2 : gemm::BN)) return rc;
  p.group_m = 64;
  while (p.group_m > 8 && (int64_t)p.group_m * gemm::BM * K > (32ll << 20)) p.group_m >>= 1;
  p.status = status_words();
  if (!p.status) return fail(KSB_ERR_CUDA, "status words unavailable");
  const int tiles_n = (int)((N + gemm::BN - 1) / gemm::BN);
  if (pair) {
    p.group_m >>= 1;  // counted in 256-row tiles
    const int tiles = (int)((M + 2 * gemm::BM - 1) / (2 * gemm::BM)) * tiles_n;
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    if (p.epilogue == KSB_EPI_SCATTER_HEADS)
      return dtype == KSB_BF16 ? launch_gemm_as<__nv_bfloat16, 2, 4>(p, ta, tw, 2 * pairs, st) : launch_gemm_as<__half, 2, 4>(p, ta, tw, 2 * pairs, st);
    return dtype == KSB_BF16 ? launch_gemm_as<__nv_bfloat16, 2, KSB_GEMM_EPILOGUE_WARPS>(p, ta, tw, 2 * pairs, st) : launch_gemm_as<__half, 2, KSB_GEMM_EPILOGUE_WARPS>(p, ta, tw, 2 * pairs, st);
  }
  const int tiles = (int)((M + gemm::BM - 1) / gemm::BM) * tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (p.epilogue == KSB_EPI_SCATTER_HEADS)
    return dtype == KSB_BF16 ? launch_gemm_as<__nv_bfloat16, 1, 4>(p, ta, tw, grid, st) : launch_gemm_as<__half, 1, 4>(p, ta, tw, grid, st);
  return dtype == KSB_BF16 ? launch_gemm_as<__nv_bfloat16, 1, KSB_GEMM_EPILOGUE_WARPS>(p, ta, tw, grid, st) : launch_gemm_as<__half, 1, KSB_GEMM_EPILOGUE_WARPS>(p, ta, tw, grid, st);
}
