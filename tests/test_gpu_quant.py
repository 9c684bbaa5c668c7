"""GPU parity: HBM-bound quantiser kernels vs the oracle.  FP8 / INT8 bytes must match bit for bit."""

import pytest
import torch

from conftest import cosine
from oracle import dit_ops as D
from oracle import quantizers as Qz

pytestmark = pytest.mark.gpu


def _ops():
    from ksanadit_b200 import _lib, ops
    return _lib, ops


@pytest.mark.parametrize("M,K", [(1, 16), (7, 5120), (300, 1536), (129, 13824), (64, 16384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rowwise_fp8_bit_exact(M, K, dtype):
    _lib, ops = _ops()
    x = D.make_activations(M, K, seed=M + K, dtype=dtype)
    if M > 3:
        x[3] = 0
    q_ref, s_ref = Qz.act_quant_fp8_rowwise(x)
    q, s = ops.quant_fp8_rowwise(x.cuda())
    _lib.assert_device_ok()
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_rowwise_fp8_strided_rows_and_empty():
    _lib, ops = _ops()
    x = D.make_activations(40, 3 * 256, seed=9)
    xs = x.cuda()[:, 256:512]  # a column slice: row stride 768
    q, s = ops.quant_fp8_rowwise(xs)
    q_ref, s_ref = Qz.act_quant_fp8_rowwise(x[:, 256:512].contiguous())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s.cpu(), s_ref)
    q0, s0 = ops.quant_fp8_rowwise(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert q0.shape == (0, 64) and s0.shape == (0,)
    with pytest.raises(_lib.KsanaB200Error):
        ops.quant_fp8_rowwise(torch.empty(4, 24, dtype=torch.bfloat16, device="cuda"))  # K % 16 != 0
    with pytest.raises(_lib.KsanaB200Error):
        ops.quant_fp8_rowwise(torch.empty(4, 32, dtype=torch.bfloat16))  # CPU tensor: no fallback


def test_static_quantisers_match_reference_vectors(golden):
    _lib, ops = _ops()
    g = golden["fp8_pt"]
    q, s = ops.quant_fp8_static(g["x"].reshape(-1, 64).cuda(), g["si"].reshape(1).cuda())
    assert torch.equal(q.cpu().view(torch.uint8), g["xq"]) and bool((s.cpu() == g["si"]).all())
    u = golden["fp8_unscaled"]
    q, s = ops.quant_fp8_static(u["x"].cuda(), None)
    assert torch.equal(q.cpu().view(torch.uint8), u["xq"]) and bool((s.cpu() == 1).all())


@pytest.mark.parametrize("M,K,rows", [(50, 1536, 1), (33, 5120, 33)])
def test_adaln_quant(M, K, rows):
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(5)
    x = D.make_activations(M, K, seed=1)
    shift = (torch.randn(rows, K, generator=g) * 0.1).to(torch.bfloat16)
    scale = (torch.randn(rows, K, generator=g) * 0.1).to(torch.bfloat16)
    h_ref = D.modulate(x, shift, scale)
    q_ref, s_ref = Qz.act_quant_fp8_rowwise(h_ref)
    q, s, h = ops.adaln_quant_fp8(x.cuda(), shift.cuda(), scale.cuda(), want_h=True)
    _lib.assert_device_ok()
    # LayerNorm statistics are fp32 reductions (order differs from the CPU): tolerance on h, then the
    # quantiser applied to the kernel's own h must be bit exact.
    assert (h.cpu().float() - h_ref.float()).abs().max() <= 2 ** -6 * h_ref.float().abs().max()
    assert cosine(h.cpu(), h_ref) > 0.99999
    q2, s2 = Qz.act_quant_fp8_rowwise(h.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s.cpu(), s2)
    frac = (q.cpu().view(torch.uint8) == q_ref.view(torch.uint8)).float().mean()
    assert frac > 0.99


def test_layernorm_affine_quant():
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(6)
    M, K = 40, 1536
    x = D.make_activations(M, K, seed=2)
    w = 1 + 0.1 * torch.randn(K, generator=g)
    b = 0.1 * torch.randn(K, generator=g)
    h_ref = D.layernorm_affine_fp32(x, w, b)
    q, s, h = ops.layernorm_quant_fp8(x.cuda(), w.cuda(), b.cuda(), want_h=True)
    assert cosine(h.cpu(), h_ref) > 0.99999
    q2, s2 = Qz.act_quant_fp8_rowwise(h.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s.cpu(), s2)


@pytest.mark.parametrize("L,H", [(1, 1), (63, 2), (200, 3), (1560, 12)])
def test_sage_prepass_bit_exact(L, H):
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(L)
    q = torch.randn(L, H, 128, generator=g).to(torch.bfloat16)
    k = (torch.randn(L, H, 128, generator=g) + 0.5 * torch.randn(1, H, 128, generator=g)).to(torch.bfloat16)
    v = torch.randn(L, H, 128, generator=g).to(torch.bfloat16)
    km = ops.sage_kmean(k.cuda())
    km_ref = Qz.k_mean(k)
    assert (km.cpu() - km_ref).abs().max() <= 1e-5 * max(1.0, float(km_ref.abs().max()))
    # the quantisers take the mean as an input, so they can be compared bit for bit
    pm = Qz.q_premul(128)
    assert pm == ops.q_premul(128)
    q8, qs = ops.sage_quant_int8(q.cuda(), 128, premul=pm)
    q8r, qsr = Qz.int8_block_quant(q, 128, premul=pm)
    assert torch.equal(q8.cpu(), q8r) and torch.equal(qs.cpu(), qsr)
    k8, ks = ops.sage_quant_int8(k.cuda(), 64, mean=km_ref.cuda())
    k8r, ksr = Qz.int8_block_quant(k, 64, mean=km_ref)
    assert torch.equal(k8.cpu(), k8r) and torch.equal(ks.cpu(), ksr)
    vt, vs = ops.sage_quant_v(v.cuda())
    vtr, vsr = Qz.v_quant_fp8(v)
    assert torch.equal(vs.cpu(), vsr) and torch.equal(vt.cpu().view(torch.uint8), vtr.view(torch.uint8))
    _lib.assert_device_ok()


def test_sage_prepass_on_fused_qkv_views():
    """Q/K/V given as strided views into one [L, 3*H*128] projection output."""
    _lib, ops = _ops()
    L, H = 300, 2
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(L, 3 * H * 128, generator=g).to(torch.bfloat16)
    qv, kv, vv = (qkv[:, i * H * 128:(i + 1) * H * 128].reshape(L, H, 128) for i in range(3))
    dq, dk, dv = (qkv.cuda()[:, i * H * 128:(i + 1) * H * 128].unflatten(1, (H, 128)) for i in range(3))
    q8, qs = ops.sage_quant_int8(dq, 128, premul=Qz.q_premul(128))
    q8r, qsr = Qz.int8_block_quant(qv, 128, premul=Qz.q_premul(128))
    assert torch.equal(q8.cpu(), q8r) and torch.equal(qs.cpu(), qsr)
    vt, vs = ops.sage_quant_v(dv)
    vtr, vsr = Qz.v_quant_fp8(vv)
    assert torch.equal(vt.cpu().view(torch.uint8), vtr.view(torch.uint8))
    km = ops.sage_kmean(dk)
    assert (km.cpu() - Qz.k_mean(kv)).abs().max() < 1e-5


def test_gate_residual():
    _lib, ops = _ops()
    g = torch.Generator().manual_seed(8)
    x, y = (torch.randn(70, 256, generator=g).to(torch.bfloat16) for _ in range(2))
    gate = torch.randn(1, 256, generator=g).to(torch.bfloat16)
    o = ops.gate_residual(x.cuda(), y.cuda(), gate.cuda())
    assert torch.equal(o.cpu(), D.gate_residual(x, y, gate))
