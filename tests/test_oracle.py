"""CPU tests: the oracle against the golden vectors made from the reference's own torch code,
plus the internal consistency of the quantiser definitions."""

import numpy as np
import pytest
import torch

from conftest import cosine, max_abs_rel
from oracle import dit_ops as D
from oracle import quantizers as Qz
from oracle import radial_mask as R
from oracle import sage as Sg
from oracle import ulysses as U


def test_per_tensor_fp8_linear_matches_reference(golden):
    g = golden["fp8_pt"]
    xq = Qz.act_quant_fp8_static(g["x"].reshape(-1, 64), g["si"])
    assert torch.equal(xq.view(torch.uint8), g["xq"])
    y = Qz.fp8_linear_emulated(g["x"], g["wq"].view(torch.float8_e4m3fn), g["sw"], g["bias"], xq=xq, s_x=g["si"])
    assert (y.float() - g["y"].float()).abs().max() <= 2e-3
    u = golden["fp8_unscaled"]
    assert torch.equal(Qz.act_quant_fp8_static(u["x"], None).view(torch.uint8), u["xq"])


def test_rowwise_quantiser_definition():
    x = D.make_activations(64, 512, seed=2)
    x[5] = 0  # all-zero row -> scale 1, zeros out
    q, s = Qz.act_quant_fp8_rowwise(x)
    # numpy restatement of the same definition: IEEE fp32 divides, bf16 product, RNE e4m3 cast
    xf = x.float().numpy()
    amax = np.abs(xf).max(axis=1)
    s_np = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32)
    assert np.array_equal(s.numpy(), s_np)
    inv = torch.from_numpy((np.float32(1.0) / s_np)).to(torch.bfloat16)
    prod = (x.float() * inv.float()[:, None]).to(torch.bfloat16)  # exact fp32 product, one rounding
    assert torch.equal(q.view(torch.uint8), prod.to(torch.float8_e4m3fn).view(torch.uint8))
    assert s[5] == 1 and int(q[5].view(torch.uint8).max()) == 0
    assert float(q.float().abs().max()) <= 448
    # dequantised error is bounded by half an e4m3 step (2^-4 relative) of the row max
    err = (q.float() * s[:, None] - x.float()).abs().amax(dim=1)
    assert bool((err <= x.float().abs().amax(dim=1) * 2**-4 + 1e-6).all())


def test_rowwise_fp8_linear_close_to_fp32():
    x = D.make_activations(96, 256, seed=3)
    lp = D.LinearParams((torch.randn(128, 256) * 0.02).to(torch.bfloat16), (torch.randn(128) * 0.02).to(torch.bfloat16))
    assert cosine(lp.fp8(x), lp.fp32(x)) > 0.999


def test_rope_matches_reference(golden):
    g = golden["rope"]
    y = D.apply_wan_rope(g["x"], tuple(g["grid"].tolist()))
    assert torch.equal(y, g["y"])


def test_wan_block_matches_reference(golden):
    g = golden["wan_block"]
    p = D.make_wan_block_params(g["dim"], g["ffn"], g["heads"], seed=g["seed_params"])
    grid = tuple(g["grid"].tolist())
    x = D.make_activations(grid[0] * grid[1] * grid[2], g["dim"], seed=g["seed_x"])[None]
    y = D.wan_block_forward(p, x, g["e"], g["ctx"], grid, linear="fp32", attn="sdpa")
    assert max_abs_rel(y.float(), g["y"].float()) <= 1e-2 and cosine(y, g["y"]) > 0.9999
    # the quantised path (emulated FP8 Linear + Sage emulation) stays within the block tolerance
    yq = D.wan_block_forward(p, x, g["e"], g["ctx"], grid, linear="fp8", attn="sage")
    assert cosine(yq, g["y"]) > 0.999


def test_qwen_block_matches_reference(golden):
    g = golden["qwen_block"]
    p = D.make_qwen_block_params(g["dim"], g["ffn"], g["heads"], seed=g["seed_params"])
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        p[nm] = p[nm].to(torch.bfloat16)
    grid = tuple(g["grid"].tolist())
    img = D.make_activations(grid[0] * grid[1] * grid[2], g["dim"], seed=g["seed_x"])
    ia, ta = D.qwen_rope_angles(grid, g["txt"].shape[1])
    i, t = D.qwen_block_forward(p, img, g["txt"][0], g["temb"][0], ia, ta, linear="fp32", attn="sdpa")
    assert max_abs_rel(i.float(), g["img_y"].float()) <= 1.5e-2
    assert max_abs_rel(t.float(), g["txt_y"].float()) <= 1.5e-2


def test_radial_masks_match_reference(golden):
    for key, packed in golden["radial_masks"].items():
        vt, nf, bs, decay, s = key.split("_")
        vt, nf, bs, s, decay = int(vt), int(nf), int(bs), int(s), float(decay)
        m = R.radial_log_mask(s, vt, nf, bs, decay)
        ref = np.unpackbits(packed.numpy())[: m.size].reshape(m.shape).astype(bool)
        assert np.array_equal(m, ref), key


def test_tile_lists_roundtrip():
    m = R.bernoulli_frame_mask(128 * 37 + 5, 900, seed=1)
    m64 = R.expand_to_q128_k64(m, 128)
    offs, ent = R.tile_lists(m64)
    back = np.zeros_like(m64)
    for r in range(m64.shape[0]):
        for e in ent[offs[r]:offs[r + 1]]:
            t, h = e // 4, e % 4
            back[r, 2 * t] = h & 1
            back[r, 2 * t + 1] = (h >> 1) & 1
    assert np.array_equal(back.astype(bool), m64)
    assert bool(np.diag(m).all())


def test_sage_emulation_within_reference_bound():
    """The bound the reference's own test puts on its Sage backend vs SDPA
    (tests/ksana/attention_op_test.py:157-186): B,L,H,D = 2,32,64,128 fp16, max<1e-1, mean<1e-2."""
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 32, 64, 128, generator=g).to(torch.float16) for _ in range(3))
    for b in range(2):
        o = Sg.sage_attention(q[b], k[b], v[b]).float()
        r = Sg.sdpa_reference(q[b], k[b], v[b])
        d = (o - r).abs()
        assert d.max() < 1e-1 and d.mean() < 1e-2


@pytest.mark.parametrize("L", [1, 63, 129, 300])
def test_sage_emulation_ragged_lengths(L):
    g = torch.Generator().manual_seed(L)
    q = torch.randn(L, 2, 128, generator=g).to(torch.bfloat16)
    k = (torch.randn(L, 2, 128, generator=g) + torch.randn(1, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
    v = torch.randn(L, 2, 128, generator=g).to(torch.bfloat16)
    o = Sg.sage_attention(q, k, v).float()
    r = Sg.sdpa_reference(q, k, v)
    assert cosine(o, r) > 0.999


def test_sage_sparse_matches_masked_sdpa():
    g = torch.Generator().manual_seed(7)
    L = 128 * 5 + 40
    q, k, v = (torch.randn(L, 2, 128, generator=g).to(torch.bfloat16) for _ in range(3))
    m = R.expand_to_q128_k64(R.bernoulli_frame_mask(L, 200, seed=3), 128)
    o = Sg.sage_attention(q, k, v, tile_mask=torch.from_numpy(m)).float()
    r = Sg.masked_sdpa_reference(q, k, v, torch.from_numpy(m))
    assert cosine(o, r) > 0.999


def test_int8_and_v_quantisers():
    g = torch.Generator().manual_seed(11)
    k = (torch.randn(200, 3, 128, generator=g) + 0.5).to(torch.bfloat16)
    km = Qz.k_mean(k)
    k8, ks = Qz.int8_block_quant(k, 64, mean=km)
    assert k8.shape == (3, 256, 128) and ks.shape == (3, 4)
    assert int(k8[:, 200:].abs().max()) == 0 and bool((ks[:, 3] > 0).all())
    deq = k8.float()[:, :200] * ks.repeat_interleave(64, dim=1)[:, :200, None]
    ref = (k.float() - km[None]).permute(1, 0, 2)
    assert (deq - ref).abs().max() <= ks.max() * 0.5 + 1e-6
    assert int(k8.abs().max()) == 127
    vt8, vs = Qz.v_quant_fp8(k)
    assert vt8.shape == (3, 128, 256) and float(vt8.float().abs().max()) == 448.0


def test_all_to_all_layout_is_an_involution():
    P, L, H, Dh = 4, 24, 8, 16
    xs = [torch.randn(1, L // P, H, Dh) for _ in range(P)]
    fwd = U.all_to_all_emulated(xs, scatter_dim=2, gather_dim=1)
    assert fwd[0].shape == (1, L, H // P, Dh)
    full = torch.cat(xs, dim=1)
    for r in range(P):
        assert torch.equal(fwd[r], full[:, :, r * (H // P):(r + 1) * (H // P)])
    back = U.all_to_all_emulated(fwd, scatter_dim=1, gather_dim=2)
    for r in range(P):
        assert torch.equal(back[r], xs[r])
