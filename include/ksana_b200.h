/*
 * ksana_b200 -- C ABI of the B200 (sm_100a) DiT-block kernels.
 *
 * KsanaDiT is pure Python: its DiT block reaches its kernels through torch and third-party Python
 * packages, so it has no FFI of its own.  Each entry point below names the Python call site in
 * KsanaDiT (path inside that project, file:line) whose work it takes over; the Python classes in
 * ksanadit_b200/ adapt these to KsanaDiT's operator contracts.
 *
 * Conventions
 *   - every pointer is a device pointer owned by the caller and must stay valid until the work
 *     queued on `stream` has finished; nothing is allocated or freed here
 *   - `stream` is a cudaStream_t (NULL = legacy default stream)
 *   - return value 0 = queued; negative = rejected before any launch
 *     (-1 invalid argument, -2 CUDA error, -3 unsupported); ksb_last_error() gives the text
 *   - half-precision tensors carry a dtype tag: KSB_BF16 or KSB_FP16
 *   - FP8 means e4m3 (finite, max 448); INT8 is signed; scales are fp32
 */
#ifndef KSANA_B200_H
#define KSANA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KSB_BF16 0
#define KSB_FP16 1

/* GEMM epilogues */
#define KSB_EPI_NONE 0          /* out = acc*sa*sw + bias */
#define KSB_EPI_GELU_TANH 1     /* out = gelu_tanh(round(acc*sa*sw + bias)) */
#define KSB_EPI_GATE_RESIDUAL 2 /* out = resid + round(acc*sa*sw + bias) * gate */
#define KSB_EPI_SCATTER_HEADS 3 /* only through ksb_fp8_gemm_qkv_scatter */

/* most GPUs one exchange can span (the ranks of one NVLink / NVSwitch box) */
#define KSB_MAX_PEERS 8

/* token-block sizes of the INT8 scales and padding of the quantised attention operands */
#define KSB_Q_BLOCK 128
#define KSB_K_BLOCK 64
#define KSB_KV_TILE 128

typedef void* ksb_stream_t;

/* Library / error state ------------------------------------------------------------------- */
int ksb_version(void);
const char* ksb_last_error(void);
/* Synchronises the device, returns the status words written by kernels whose bounded waits ran out
 * (code 0 = none; code 1 = a wait timed out, detail = kernel id << 16 | wait site; kernel ids: 1 FP8 GEMM,
 * 2 attention with one Q block per CTA, 3 attention with two, 15 the self-test) and clears them.
 * The words are sticky: from the moment a wait has run out, every later wait of every kernel on that GPU gives
 * up at once and leaves its outputs unwritten, until this call has read the words.  A caller that consumes
 * results should therefore check once per step, at a point where it synchronises anyway. */
int ksb_device_status(int* code, int* detail);
int ksb_sm_count(void);
/* Diagnostic with no counterpart in KsanaDiT: launches one small kernel in which a thread waits, for at most
 * limit_ns (<= 1e9), on a barrier that nothing ever completes.  The kernel must return by itself, store 2 in
 * *returned (device int; 1 would mean the wait succeeded) and leave (1, 15 << 16 | 1) in the status words;
 * the next launch on the GPU must work.  Used by the tests to exercise the time-out path without faulting a GPU. */
int ksb_selftest_bounded_wait(int64_t limit_ns, int* returned, ksb_stream_t stream);

/* Per-token FP8 activation quantiser.
 * Replaces the eager `(input * (1.0 / scale_input).to(dtype)).to(float8_e4m3fn)` pass of
 * ksana/operations/linear/fp8_linear.py:52-58, with one scale per row:
 *   scale[m] = absmax(x[m,:]) / 448 (1.0 for a zero row); q = e4m3(x * half(1/scale[m])).
 * x: [M,K] half, row stride ldx elements; q: [M,K] e4m3 contiguous; scale: [M]. K % 16 == 0. */
int ksb_quant_fp8_rowwise(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, void* q, float* scale,
                          ksb_stream_t stream);

/* The reference's own activation quantisers (fp8_linear.py:48-58): scale_input == NULL ->
 * clamp(+-448) then cast; else q = e4m3(x * half(1/scale_input[0])) saturated.  scale_out[M] receives
 * the row scale the GEMM must apply (1 or scale_input[0]). */
int ksb_quant_fp8_static(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const float* scale_input,
                         void* q, float* scale_out, ksb_stream_t stream);

/* adaLN modulate fused with the per-token FP8 quantiser.
 * Replaces `torch.addcmul(shift, LayerNorm(x), 1 + scale)` (ksana/models/wan/wan_model.py:374,391;
 * ksana/operations/ops.py:41-52) followed by the quantiser above.
 *   h = shift + LN(x) * (1 + scale), LN without affine, eps; computed in fp32, rounded to half at the
 *   points the eager path rounds: after LN, after 1+scale, after the addcmul (round_product == 0, Wan), or
 *   additionally after the product for `LN(x) * (1 + scale) + shift` written as two eager ops
 *   (round_product == 1, Qwen-Image: ksana/models/qwen/transformer.py:171-194).
 * shift/scale: [mod_rows, K] half with mod_rows == 1 (broadcast) or M.  h_out (optional, may be NULL)
 * receives h in half precision.  K % 16 == 0, K <= 16384. */
int ksb_adaln_quant_fp8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const void* shift,
                        const void* scale, int64_t mod_rows, int round_product, float eps, void* h_out, void* q,
                        float* qscale, ksb_stream_t stream);

/* Affine fp32 LayerNorm fused with the per-token FP8 quantiser (Wan norm3 before cross-attention,
 * wan_model.py:296-302,390; ops.py:45-50).  w, b: fp32 [K] (b may be NULL). */
int ksb_layernorm_quant_fp8(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const float* w,
                            const float* b, float eps, void* h_out, void* q, float* qscale, ksb_stream_t stream);

/* FP8 GEMM with per-token x per-output-channel scales on the tcgen05 tensor cores.
 * Replaces `torch._scaled_mm(input, w, out_dtype, bias, scale_a, scale_b)` of fp8_linear.py:60-63 and,
 * through the epilogue switch, the eager passes that follow it in the block:
 * nn.GELU(approximate="tanh") (wan_model.py:317-321) and torch.addcmul(x, y, gate) (wan_model.py:385,392).
 *   out[m,n] = epi( (sum_k a[m,k]*w[n,k])_fp32 * a_scale[m] * w_scale[n] + bias[n] )
 * a: [M,K] e4m3 contiguous; w: [N,K] e4m3 contiguous; bias: half [N] or NULL; out: [M,N] half, row
 * stride ldo.  resid: [M,N] half (row stride ldr) and gate: [gate_rows, N] half, both only for
 * KSB_EPI_GATE_RESIDUAL.  gate_rows divides M and row m uses gate row m / (M / gate_rows): 1 = one gate for all
 * rows, M = one per token, B = one per sample of a batch of B equal-length sequences folded into M
 * (cond / uncond batching, ksana/generators/generator.py:356-375).  K % 16 == 0, N % 8 == 0. */
int ksb_fp8_gemm(const void* a, const float* a_scale, const void* w, const float* w_scale, const void* bias,
                 int64_t M, int64_t N, int64_t K, void* out, int dtype, int64_t ldo, int epilogue,
                 const void* resid, int64_t ldr, const void* gate, int64_t gate_rows, ksb_stream_t stream);

/* Fused QKV projection + Ulysses "scatter heads, gather sequence" exchange (sequence parallelism over P GPUs
 * of one box).  Replaces the fused QKV Linear (ksana/operations/fuse_qkv/fuse_qkv.py:226-233) followed by the three
 * all_to_all(x, scatter_dim=2, gather_dim=1) of ksana/models/wan/wan_model.py:134-141 (ksana/utils/distribute.py:112-122):
 * the GEMM epilogue stores each output element straight into the memory of the GPU that owns its head (plain
 * peer stores over NVLink, no separate exchange kernel, no pack / unpack copies).
 *   a [M, K] e4m3 (this rank's M tokens), w [3C, K] e4m3 (rows: Q | K | V), C = heads * 128, C % 256 == 0.
 *   peer_out[p] (host array of n_peers device pointers, peer_out[rank] is this GPU's own): each a
 *   [n_peers * M, 3, heads / n_peers, 128] half buffer; row (rank * M + m) receives this rank's token m.
 *   tile_sumsq: fp32 scratch [2 * C / 256][M]; receives, per 256-column tile of the Q and K thirds, the sum of
 *   squares of each output row (for the full-width RMSNorm that follows, see ksb_rowsumsq_to_rstd_scatter).
 * The caller must synchronise the peers (all of them done with this call) before any of them reads its buffer. */
int ksb_fp8_gemm_qkv_scatter(const void* a, const float* a_scale, const void* w, const float* w_scale, const void* bias,
                             int64_t M, int64_t C, int64_t K, int dtype, void* const* peer_out, int n_peers, int rank,
                             int64_t heads, float* tile_sumsq, ksb_stream_t stream);

/* Turns the tile sums of squares above into rstd = rsqrt(sum / C + eps) per (Q | K, token) and stores them into
 * every peer's fp32 [2, n_peers * M] table at column rank * M + m (what norm_q / norm_k,
 * ksana/operations/ops.py:64-70, need once the heads of a token live on different GPUs). */
int ksb_rowsumsq_to_rstd_scatter(const float* tile_sumsq, int64_t M, int64_t C, float eps, float* const* peer_rstd,
                                 int n_peers, int rank, ksb_stream_t stream);

/* Gated residual out = x + y * gate (one rounding), for the places where it is not fused into a GEMM
 * epilogue.  Replaces torch.addcmul(x, y, gate) / x + gate * y (wan_model.py:385,392;
 * ksana/models/qwen/transformer.py:225-234).  x, y, out: [M,N] half contiguous; gate: [gate_rows, N]. */
int ksb_gate_residual(const void* x, const void* y, const void* gate, int64_t gate_rows, void* out, int dtype,
                      int64_t M, int64_t N, ksb_stream_t stream);

/* Residual statistics of the block-level step cache (DBCache): the residual of a group of blocks and its L1
 * distance to the residual kept from an earlier step, in one pass over the activations.
 * Replaces `f_n_residual = x - x_ori` (ksana/cache/dbcache.py:301-306) and the three full-tensor reductions of
 * `compute_diff_and_decide` (dbcache.py:228-239: mean |cur - prev|, mean |cur|, mean |prev|).
 *   r = round(x_new - x_old) in the activation dtype; sums[0] = sum round(|r - prev|), sums[1] = sum |r|,
 *   sums[2] = sum |prev| (fp32; the caller divides by n and forms the relative difference).
 * x_new, x_old: n half elements, n % 8 == 0; prev_residual: n elements or NULL (then sums[0] = sums[2] = 0);
 * residual_out: receives r, or NULL; sums: 3 floats, cleared by this call on `stream`. */
int ksb_residual_diff(const void* x_new, const void* x_old, const void* prev_residual, void* residual_out, float* sums,
                      int dtype, int64_t n, ksb_stream_t stream);

/* Sage pre-passes.  The reference reaches them through the un-vendored `sageattention` /
 * `spas_sage_attn` packages (call sites ksana/operations/attention/backends/sage_attn.py:75-81 and
 * sage_sla.py:198-228, which shows the pre-pass API: k.mean(-2), per-block INT8 Q/K with fp32 scales,
 * transposed + padded per-(head, channel) FP8 V).
 * Input tensors are [L, H, D] views given by element strides (token_stride, head_stride), D == 128
 * contiguous. */

/* km[h,d] = mean over tokens of k (fp32).  partial: fp32 scratch of ksb_sage_kmean_scratch_floats(L,H,D). */
int64_t ksb_sage_kmean_scratch_floats(int64_t L, int64_t H, int64_t D);
int ksb_sage_kmean(const void* k, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                   int64_t head_stride, float* partial, float* km, ksb_stream_t stream);

/* RMSNorm with an fp32 weight, optionally followed by the 3-axis rotary embedding, in place on a [L, C]
 * half view (row stride ld; e.g. the Q or K third of a fused QKV output), C = heads * 128.
 * per_head == 0: normalise over all C channels, w is [C]  (Wan: norm_q / norm_k,
 *   `x.float() * rsqrt(mean(x^2) + eps) * w`, ksana/operations/ops.py:64-70 via
 *   ksana/models/wan/wan_model.py:81-90,164-165);
 * per_head == 1: normalise each head's 128 channels, w is [128]  (Qwen-Image: norm_q / norm_k /
 *   norm_added_q / norm_added_k, ksana/models/qwen/attention.py:267-272,340-343).
 * Rotation (apply_default_rope, ksana/utils/rope.py:62-128; apply_rotary_emb_qwen, qwen/attention.py:31-59):
 * rope_table is fp32 [table_len][64][2] = (cos, sin); rotation pair p of a head reads table row `coord` with
 * coord = the token's frame index for p < nf, its row index for p < nf + nh, else its column index; row l sits
 * at position pos0 + l of an F x Hh x Ww grid (rows past the grid are not rotated).  The caller puts whatever
 * angle belongs to coordinate index r of each axis into row r (Wan: r * inv_freq; Qwen: centred positions).
 * diag == 1 (grid (F,1,1)): the running position drives all three axes (Qwen text tokens).
 * row_rstd (optional, fp32 [L]): use these per-row factors instead of computing rsqrt(mean(x^2) + eps) over the C
 * channels present (for rows whose other heads live on other GPUs; per_head must be 0).
 * rope_table NULL = no rotation.  colsum_partial (fp32 scratch, ksb_rmsnorm_rope_scratch_floats) with
 * colmean [C]: also returns the per-channel mean over the L rows of the values written (the K smoothing
 * vector, sage_sla.py:198); both NULL to skip. */
int64_t ksb_rmsnorm_rope_scratch_floats(int64_t L, int64_t C);
int ksb_rmsnorm_rope_inplace(void* x, int dtype, int64_t L, int64_t C, int64_t ld, const float* w, int per_head,
                             const float* row_rstd, float eps, const float* rope_table, int table_len, int nf, int nh, int F, int Hh,
                             int Ww, int64_t pos0, int diag, float* colsum_partial, float* colmean,
                             ksb_stream_t stream);

/* INT8 block quantiser: xf = float(x) - mean[h,d] (if mean) then * premul (if premul != 0);
 * scale[h,b] = absmax(block)/127 (1 if zero); q = clamp(rint(xf * (127/absmax)), +-127).
 * out: [H, Lpad, D] int8 with Lpad = roundup(L,128), padding zero-filled; scale: [H, Lpad/block].
 * block is 128 (Q) or 64 (K). */
int ksb_sage_quant_int8(const void* x, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                        int64_t head_stride, int block, float premul, const float* mean, void* out,
                        float* scale, ksb_stream_t stream);

/* How ksb_fp8_gemm (and _rowstats) drive the tensor cores: 0 = every CTA computes 128 x 256 tiles on its own
 * (tcgen05.mma.cta_group::1); 1 = two CTAs of a cluster share 256 x 256 tiles (cta_group::2), each fetching its own half
 * of the operands (the default; both forms give the same bits).  Sets the mode when `mode` is 0 or 1, leaves it
 * otherwise (pass -1 to query); returns the mode that was in force before the call.  Process-wide, for every GEMM
 * entry point. */
int ksb_gemm_pair_mode(int mode);

/* The QKV projection with row statistics: ksb_fp8_gemm with KSB_EPI_NONE that also writes, for every 256-column
 * tile that starts below column sumsq_cols (a multiple of 256) and every row m, the sum of squares of the rounded
 * outputs of that tile to tile_sumsq[tile_n][m] (fp32 [sumsq_cols / 256, M]).  RMSNorm over the C leading channels
 * of a row (ksana/models/wan/wan_model.py:163-165, norm_q / norm_k on the projection output) then needs no pass
 * over the output. */
int ksb_fp8_gemm_rowstats(const void* a, const float* a_scale, const void* w, const float* w_scale, const void* bias,
                          int64_t M, int64_t N, int64_t K, void* out, int dtype, int64_t ldo, float* tile_sumsq,
                          int64_t sumsq_cols, ksb_stream_t stream);
/* rstd[g][m] = rsqrt(sum of the C / 256 tiles of column group g / C + eps), g < groups: fp32 [groups, M]. */
int ksb_rowsumsq_to_rstd(const float* tile_sumsq, int64_t M, int64_t C, int groups, float eps, float* rstd,
                         ksb_stream_t stream);

/* RMSNorm (+ rotary embedding) folded into the K mean and the INT8 quantisers: what ksb_rmsnorm_rope_inplace followed
 * by ksb_sage_kmean / ksb_sage_quant_int8 compute, byte for byte, without writing the normalised tensor (Q is read
 * once, K twice).  norm_w: fp32 [H * 128], with row_rstd fp32 [L] = 1 / rms of each token over all heads (from
 * ksb_rowsumsq_to_rstd, or any table); or per_head = 1: norm_w fp32 [128], 1 / rms over each head's own channels
 * (row_rstd ignored).  The rope arguments are those of ksb_rmsnorm_rope_inplace (rope_table NULL: no rotation).
 * Replaces norm_q / norm_k, apply_default_rope (ksana/models/wan/wan_model.py:163-174) and the quantisers inside
 * sageattn. */
int ksb_sage_kmean_normed(const void* k, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                          int64_t head_stride, const float* norm_w, int per_head, const float* row_rstd, float eps,
                          const float* rope_table, int table_len, int nf, int nh, int F, int Hh, int Ww, int64_t pos0,
                          int diag, float* partial, float* km, ksb_stream_t stream);
int ksb_sage_quant_int8_normed(const void* x, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                               int64_t head_stride, int block, float premul, const float* mean, const float* norm_w,
                               int per_head, const float* row_rstd, float eps, const float* rope_table, int table_len,
                               int nf, int nh, int F, int Hh, int Ww, int64_t pos0, int diag, void* out, float* scale,
                               ksb_stream_t stream);

/* V quantiser: vs[h,d] = absmax over tokens / 448 (1 if zero); vt[h,d,l] = e4m3(float(v) * (448/absmax)), token
 * axis contiguous and zero-padded to Lpad.  amax: fp32 scratch [H*D] (overwritten). */
int ksb_sage_quant_v_fp8(const void* v, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                         int64_t head_stride, float* amax, void* vt, float* vs, ksb_stream_t stream);

/* Allocation-free form of the V quantiser above: same inputs, same outputs (bit for bit), but the absmax
 * scratch is a fixed array inside the library instead of a buffer from the caller.  It has no counterpart
 * in KsanaDiT; it exists for callers that may not allocate device memory at the point of the call -- a host
 * runtime that handed the library raw pointers out of an arena it sized in advance and keeps no allocator
 * the library could use, or a latency-critical loop that must not reach cudaMalloc (which can stall on a
 * device-wide synchronisation or fail when the arena owner has left no free memory).  Nothing is allocated
 * or freed here, by the CUDA runtime or by any library.
 *   - limit: H * D <= 65536 (at most 512 heads of 128); larger shapes are rejected with an error text
 *   - the array costs 256 KB of device memory on every GPU that loads the library, until the process exits
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call before starting any stream capture
 *   - every call uses the same array: it is cleared at the start of each call, and two calls that overlap
 *     on the GPU (different streams, or different host threads) race on it -- serialise them */
int ksb_sage_quant_v_fp8_noalloc(const void* v, int dtype, int64_t L, int64_t H, int64_t D, int64_t token_stride,
                                 int64_t head_stride, void* vt, float* vs, ksb_stream_t stream);

/* Sage-style attention core: INT8 Q.K^T (s32 accumulate) -> fp32 online softmax in the exp2 domain ->
 * e4m3 P -> FP8 P.V (f32 accumulate) on tcgen05, dense or block-sparse.
 * Replaces `sageattn(q, k, v, tensor_layout="NHD")` (sage_attn.py:75-81) and
 * `block_sparse_sage2_attn_cuda(q, k, v, mask_id=...)` (radial_sage_attn/radial_sage_attn.py:170-176).
 *   q8 [H,Lq_pad,128], qs [H,Lq_pad/128], k8 [H,Lk_pad,128], ks [H,Lk_pad/64], vt [H,128,Lk_pad], vs [H,128]
 *   out[l,h,:] (half, element strides out_token_stride / out_head_stride) for l < Lq.
 * Block-sparse: tile_offsets int32 [Lq_pad/128 + 1] and tile_entries int32 [nnz] (shared by all heads);
 * entry = kv_tile*4 + keep bits (bit0: tokens 0-63 of the 128-token tile, bit1: tokens 64-127), ascending
 * kv_tile within a row.  NULL/NULL = dense.  A Q block with an empty list produces zeros.
 * q_order (optional, int32 [Lq_pad/128]): a permutation of the Q blocks; the CTAs walk the blocks of a head in
 * this order (pass the blocks sorted by decreasing list length to balance a ragged block-sparse mask over the
 * persistent CTAs).  NULL = ascending.
 * peer_out / n_peers / rows_per_peer (optional; NULL / 0 / 0 = write to `out`): the Ulysses "scatter sequence,
 * gather heads" exchange (ksana/models/wan/wan_model.py:143-146) fused into the output stage: output row l goes
 * to peer_out[l / rows_per_peer] at row l % rows_per_peer, with the same strides as `out` (the caller offsets each
 * peer pointer to this rank's head slot).  The peers must be synchronised before they read. */
/* Which kernel dense calls of ksb_sage_attn (no tile lists, no q_order) use: 1 = two Q blocks of a head per CTA sharing
 * every K / V tile (the default), 0 = one block per CTA (the kernel that also serves tile lists).  Same arithmetic.
 * Sets the mode when `mode` is 0 or 1, leaves it otherwise (pass -1 to query); returns the previous mode. */
int ksb_attn_dual_mode(int mode);
int ksb_sage_attn(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt, const float* vs,
                  int64_t H, int64_t Lq, int64_t Lk, const int32_t* tile_offsets, const int32_t* tile_entries,
                  const int32_t* q_order, void* out, int dtype, int64_t out_token_stride, int64_t out_head_stride,
                  void* const* peer_out, int n_peers, int64_t rows_per_peer, ksb_stream_t stream);

/* ksb_sage_attn with the tile lists given per PAIR of Q blocks (2i, 2i+1), for the kernel that keeps both blocks in one
 * CTA and fetches every K / V tile once for the two: pair_offsets int32 [ceil(Lq_pad/256) + 1], pair_entries int32
 * [nnz], entry = kv_tile*16 + keep bits of block 2i (bit0: tokens 0-63 of the tile, bit1: tokens 64-127) + keep bits of
 * block 2i+1 (bits 2-3), the union of the two blocks' lists in ascending kv_tile order; pair_order (optional, int32
 * [ceil(Lq_pad/256)]) a permutation of the pairs.  Same results as ksb_sage_attn with the per-block lists the pairs
 * were built from.  Everything else as ksb_sage_attn. */
int ksb_sage_attn_pairs(const void* q8, const float* qs, const void* k8, const float* ks, const void* vt, const float* vs,
                        int64_t H, int64_t Lq, int64_t Lk, const int32_t* pair_offsets, const int32_t* pair_entries,
                        const int32_t* pair_order, void* out, int dtype, int64_t out_token_stride, int64_t out_head_stride,
                        void* const* peer_out, int n_peers, int64_t rows_per_peer, ksb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* KSANA_B200_H */
