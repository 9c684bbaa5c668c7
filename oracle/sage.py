"""Oracle Sage-style quantised attention (plain torch, CPU).  Test infrastructure only.

Arithmetic (the build's contract; the reference delegates it to the un-vendored
``sageattention`` / ``spas_sage_attn`` packages -> parity unpinned):

  km      = mean_tokens(K)                                   (K smoothing, sage_sla.py:198)
  Q8, qs  = int8 blocks of 128 tokens of  Q * (D^-1/2 * log2 e)
  K8, ks  = int8 blocks of  64 tokens of  K - km
  V8, vs  = e4m3 per (head, channel) over tokens
  per 128-row Q block, KV tiles of 128 tokens visited in ascending order, per row:
      X   = float(Q8 . K8^T) * (qs * ks)                      int32 dot, fp32 scale
      if rowmax X > r + 3.5:  a = exp2(r - rowmax X);  r = rowmax X;  l = l * a;  O = O * a
      P   = exp2(X - r + 5)
      l   = l + rowsum(P)                                     fp32, P before rounding
      O   = O + float(e4m3(P)) . float(V8)                    fp32 accumulate
  out = O / l * vs  -> input dtype

The reference point r of a row (initially -inf, so the first valid score always sets it) follows the running
row maximum lazily: it moves only when a tile's maximum exceeds it by more than REF_SLACK = 3.5 (a factor 11.3).
P carries a fixed factor 2^5 (P_SHIFT), so the largest value ever rounded to e4m3 is below 2^8.5 = 362 < 448,
and the bulk of a long, flat attention row lands in e4m3's normal range instead of its subnormals (the published
SageAttention2 recipe scales P by a static factor for the same reason); the factor cancels in O / l.  An
implementation has to move r at exactly those tiles to round P on the same e4m3 grid; after the first tile of a
row that is rare, which is the point: O is rescaled in few tiles, and the exponentials of a tile do not have to
wait for its row maximum.

Block-sparse variant: a tile mask [ceil(Lq/128), ceil(Lk/64)] (the reference's
``mask_id`` granularity, radial_sage_attn.py:155-160,174) removes whole
(128 x 64) score tiles; a Q block whose row of the mask is empty outputs zeros.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import quantizers as Qz

P_SHIFT = 5.0  # log2 of the static scale applied to P before the e4m3 rounding
REF_SLACK = 3.5  # a row's reference point moves only when the tile maximum exceeds it by more than this


def sdpa_reference(q, k, v, sm_scale=None):
    """Exact attention on [L,H,D] tensors in fp32 (SDPAImpl, backends/sdpa.py:66-77)."""
    qf, kf, vf = (t.float().permute(1, 0, 2)[None] for t in (q, k, v))
    o = F.scaled_dot_product_attention(qf, kf, vf, scale=sm_scale)
    return o[0].permute(1, 0, 2).contiguous()


def sage_prepass(q, k, v, sm_scale=None, km=None):
    """All quantised tensors of one attention call.  q:[Lq,H,D], k,v:[Lk,H,D]."""
    D = q.shape[-1]
    if km is None:
        km = Qz.k_mean(k)
    q8, qs = Qz.int8_block_quant(q, Qz.Q_BLOCK, premul=Qz.q_premul(D, sm_scale))
    k8, ks = Qz.int8_block_quant(k, Qz.K_BLOCK, mean=km)
    vt8, vs = Qz.v_quant_fp8(v)
    return dict(q8=q8, qs=qs, k8=k8, ks=ks, vt8=vt8, vs=vs, km=km)


def sage_core(pp, Lq, Lk, tile_mask=None, out_dtype=torch.float32, q_blocks=None):
    """Online-softmax INT8-QK / FP8-PV core on pre-quantised tensors -> [Lq,H,D].

    q_blocks: optional list of 128-row Q block numbers; only those are computed and the result is
    [len(q_blocks) * 128, H, D] (rows past Lq included) -- the sampled check of sequences too long to do whole."""
    q8, qs, k8, ks, vt8, vs = pp["q8"], pp["qs"], pp["k8"], pp["ks"], pp["vt8"], pp["vs"]
    H, Lqp, D = q8.shape
    Lkp = k8.shape[1]
    nq, nkv = Lqp // 128, Lkp // 128
    qf = q8.float().view(H, nq, 128, D)
    if q_blocks is not None:
        sel = torch.as_tensor(list(q_blocks), dtype=torch.long)
        qf, qs = qf[:, sel], qs[:, sel]
        if tile_mask is not None:
            tile_mask = torch.as_tensor(tile_mask)[sel]
        nq = len(sel)
    kf = k8.float()
    vf = vt8.float()  # [H, D, Lkp]
    m = torch.full((H, nq, 128), float("-inf"))
    l = torch.zeros(H, nq, 128)
    O = torch.zeros(H, nq, 128, D)
    col = torch.arange(128)
    for j in range(nkv):
        kt = kf[:, j * 128 : (j + 1) * 128]  # [H,128,D]
        S = torch.einsum("hqrd,hcd->hqrc", qf, kt)  # exact: integers < 2^24
        sc = qs[:, :, None, None] * ks[:, 2 * j : 2 * j + 2].repeat_interleave(64, dim=1)[:, None, None, :]
        X = S * sc
        valid = ((j * 128 + col) < Lk)[None, None, None, :].expand(1, nq, 1, 128)
        if tile_mask is not None:
            tm = tile_mask[:, 2 * j : 2 * j + 2].to(torch.bool).repeat_interleave(64, dim=1)  # [nq,128]
            valid = valid & tm[None, :, None, :]
        X = torch.where(valid, X, torch.full_like(X, float("-inf")))
        m_tile = X.amax(dim=-1)
        move = m_tile > m + REF_SLACK  # true for the first valid score of a row (m = -inf), never for a fully masked tile
        m_new = torch.where(move, m_tile, m)
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        P = torch.exp2(X - safe[..., None] + P_SHIFT)
        a = torch.where(move, torch.exp2(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - safe)), torch.ones_like(m))
        l = l * a + P.sum(dim=-1)
        P8 = P.to(torch.float8_e4m3fn).float()
        vt = vf[:, :, j * 128 : (j + 1) * 128]  # [H,D,128]
        O = O * a[..., None] + torch.einsum("hqrc,hdc->hqrd", P8, vt)
        m = m_new
    lsafe = torch.where(l > 0, l, torch.ones_like(l))
    out = O / lsafe[..., None] * vs[:, None, None, :]
    if q_blocks is not None:
        return out.reshape(H, nq * 128, D).permute(1, 0, 2).contiguous().to(out_dtype)
    out = out.view(H, Lqp, D)[:, :Lq].permute(1, 0, 2).contiguous()
    return out.to(out_dtype)


def sage_attention(q, k, v, sm_scale=None, tile_mask=None):
    """Full oracle: pre-passes + core.  Returns [Lq,H,D] in q.dtype."""
    pp = sage_prepass(q, k, v, sm_scale)
    return sage_core(pp, q.shape[0], k.shape[0], tile_mask, out_dtype=q.dtype)


def masked_sdpa_reference(q, k, v, tile_mask, sm_scale=None):
    """Exact fp32 attention under the same (128 x 64) tile mask (for sparse tolerance checks)."""
    Lq, H, D = q.shape
    Lk = k.shape[0]
    sc = D**-0.5 if sm_scale is None else sm_scale
    full = tile_mask.to(torch.bool).repeat_interleave(128, 0).repeat_interleave(64, 1)[:Lq, :Lk]
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) * sc
    s = s.masked_fill(~full[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("hqk,khd->qhd", p, v.float())
