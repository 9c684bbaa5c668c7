"""GPU parity of the attention pre-pass with the RMSNorm and the rotary embedding folded into the K mean and the INT8
quantisers, and of the projection that hands them the norm factors.

* the projection with row statistics writes the same output as the plain GEMM, and its per-tile sums of squares give
  the 1 / rms table of an RMSNorm over the leading channels;
* given the same 1 / rms table and the same K mean, the folded quantisers produce the bytes and scales of the
  sequence "normalise (+ rotate) in place, then quantise", exactly: Q blocks of 128, K blocks of 64 with the mean
  subtracted, ragged lengths, a sequence-parallel position offset, the per-head norm with the one-position-for-all-axes
  rotation of text tokens, and no rotation at all (cross-attention Q);
* the K mean of the folded pass agrees with the mean of the normalised tensor.
"""

import pytest
import torch

from oracle import quantizers as Qz

pytestmark = pytest.mark.gpu


def test_projection_with_row_statistics():
    from ksanadit_b200 import _lib, ops
    M, K, C = 300, 512, 512  # 3 row tiles (the last one ragged); Q and K thirds of two 256-column tiles each
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = torch.randn(3 * C, K, generator=g) * 0.05
    bias = (torch.randn(3 * C, generator=g) * 0.1).to(torch.bfloat16).cuda()
    wq, sw = Qz.weight_quant_fp8_channelwise(w)
    xq, sx = ops.quant_fp8_rowwise(x)
    plain = ops.fp8_gemm(xq, sx, wq.cuda(), sw.cuda(), bias)
    out, sums = ops.fp8_gemm_rowstats(xq, sx, wq.cuda(), sw.cuda(), bias, 2 * C)
    _lib.assert_device_ok()
    assert torch.equal(out, plain)
    assert sums.shape == (2 * C // 256, M)
    want = out[:, :2 * C].float().view(M, 2 * C // 256, 256).pow(2).sum(-1).t()
    assert torch.allclose(sums, want, rtol=1e-5, atol=0)
    rstd = ops.rowsumsq_to_rstd(sums, C, 1e-6)
    ref = torch.rsqrt(out[:, :2 * C].float().view(M, 2, C).pow(2).mean(-1) + 1e-6).t()
    assert rstd.shape == (2, M) and torch.allclose(rstd, ref, rtol=1e-5, atol=0)


@pytest.mark.parametrize("L,heads,grid,pos0", [(300, 3, (3, 10, 10), 0), (1560, 2, (1, 30, 52), 0), (64, 1, (4, 8, 8), 128), (130, 2, None, 0)])
def test_folded_quantisers_equal_the_in_place_sequence(L, heads, grid, pos0):
    from ksanadit_b200 import _lib, ops
    C = heads * 128
    g = torch.Generator().manual_seed(L + heads)
    qkv = (torch.randn(L, 3 * C, generator=g) * 2 + 0.3 * torch.randn(1, 3 * C, generator=g)).to(torch.bfloat16).cuda()
    wq = (1 + 0.1 * torch.randn(C, generator=g)).cuda()
    wk = (1 + 0.1 * torch.randn(C, generator=g)).cuda()
    rstd = torch.rsqrt(qkv[:, :2 * C].float().view(L, 2, C).pow(2).mean(-1) + 1e-6).t().contiguous()  # any table will do
    rope = ops.wan_rope_table(128, 1024) if grid is not None else None
    t = qkv.view(L, 3, heads, 128)
    # folded: the projection output is only read
    before = qkv.clone()
    km_f = ops.sage_kmean_normed(t[:, 1], wk, 1e-6, rope, grid, pos0=pos0, row_rstd=rstd[1])
    # in place, on a copy
    ref = qkv.clone()
    km_r = ops.rmsnorm_rope_inplace(ref[:, C:2 * C], wk, 1e-6, rope, grid, pos0=pos0, want_mean=True, row_rstd=rstd[1]).view(heads, 128)
    ops.rmsnorm_rope_inplace(ref[:, :C], wq, 1e-6, rope, grid, pos0=pos0, row_rstd=rstd[0])
    r = ref.view(L, 3, heads, 128)
    assert torch.allclose(km_f, km_r, rtol=0, atol=1e-5 * max(1.0, float(km_r.abs().max())))
    q8_r, qs_r = ops.sage_quant_int8(r[:, 0], ops.Q_BLOCK, premul=ops.q_premul(128))
    k8_r, ks_r = ops.sage_quant_int8(r[:, 1], ops.K_BLOCK, mean=km_r)
    q8_f, qs_f = ops.sage_quant_int8_normed(t[:, 0], ops.Q_BLOCK, wq, premul=ops.q_premul(128), rope=rope, grid=grid, pos0=pos0, row_rstd=rstd[0])
    k8_f, ks_f = ops.sage_quant_int8_normed(t[:, 1], ops.K_BLOCK, wk, mean=km_r, rope=rope, grid=grid, pos0=pos0, row_rstd=rstd[1])
    _lib.assert_device_ok()
    assert torch.equal(qkv, before)
    assert torch.equal(q8_f, q8_r) and torch.equal(qs_f, qs_r)
    assert torch.equal(k8_f, k8_r) and torch.equal(ks_f, ks_r)


def test_folded_quantisers_with_the_per_head_norm():
    """The Qwen-Image form: RMSNorm over each head's 128 channels, image rows rotated by (frame, row, column), text rows
    by one running position on all three axes."""
    from ksanadit_b200 import _lib, ops
    heads, grid, Lt = 3, (1, 6, 10), 7
    g = torch.Generator().manual_seed(4)
    w = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16).float().cuda()
    img_tab, txt_tab = ops.qwen_rope_tables(grid, Lt)
    for L, tab, gr, diag in ((grid[1] * grid[2], img_tab, grid, False), (Lt, txt_tab, (Lt, 1, 1), True)):
        x = (torch.randn(L, heads * 128, generator=g) * 2).to(torch.bfloat16).cuda()
        ref = x.clone()
        km_r = ops.rmsnorm_rope_inplace(ref, w, 1e-6, tab, gr, per_head=True, diag=diag, want_mean=True).view(heads, 128)
        k8_r, ks_r = ops.sage_quant_int8(ref.view(L, heads, 128), ops.K_BLOCK, mean=km_r)
        q8_r, qs_r = ops.sage_quant_int8(ref.view(L, heads, 128), ops.Q_BLOCK, premul=ops.q_premul(128))
        x3 = x.view(L, heads, 128)
        km_f = ops.sage_kmean_normed(x3, w, 1e-6, tab, gr, per_head=True, diag=diag)
        k8_f, ks_f = ops.sage_quant_int8_normed(x3, ops.K_BLOCK, w, mean=km_r, rope=tab, grid=gr, per_head=True, diag=diag)
        q8_f, qs_f = ops.sage_quant_int8_normed(x3, ops.Q_BLOCK, w, premul=ops.q_premul(128), rope=tab, grid=gr, per_head=True, diag=diag)
        _lib.assert_device_ok()
        assert torch.allclose(km_f, km_r, rtol=0, atol=1e-5 * max(1.0, float(km_r.abs().max())))
        assert torch.equal(k8_f, k8_r) and torch.equal(ks_f, ks_r)
        assert torch.equal(q8_f, q8_r) and torch.equal(qs_f, qs_r)


def test_folded_quantiser_rejects_a_missing_table():
    from ksanadit_b200 import _lib, ops
    x = torch.zeros(128, 1, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(128, device="cuda")
    with pytest.raises((AssertionError, _lib.KsanaB200Error)):
        ops.sage_quant_int8_normed(x, ops.Q_BLOCK, w)  # a norm over all heads without row_rstd
