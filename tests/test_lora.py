"""LoRA merge into FP8 / high-precision state dicts (host logic, CPU)."""

import torch

from ksanadit_b200.linear import quantize_weight_per_channel
from ksanadit_b200.lora import dequantize_weight, merge_lora_weight


def _lora(n, k, r, g, prefix=""):
    return {prefix + "blk.q.lora_down.weight": torch.randn(r, k, generator=g) * 0.05,
            prefix + "blk.q.lora_up.weight": torch.randn(n, r, generator=g) * 0.05,
            prefix + "blk.q.alpha": torch.tensor(4.0)}


def test_fp8_weight_is_requantised_per_channel():
    g = torch.Generator().manual_seed(0)
    n, k, r = 48, 64, 8
    w = torch.randn(n, k, generator=g) * 0.02
    wq, s = quantize_weight_per_channel(w)
    sd = {"blk.q.weight": wq, "blk.q.scale_weight": s, "blk.q.bias": torch.zeros(n), "blk.o.weight": wq.clone(),
          "blk.o.scale_weight": s.clone()}
    lora = _lora(n, k, r, g)
    want = dequantize_weight(sd, "blk.q.weight") + 0.5 * (4.0 / r) * lora["blk.q.lora_up.weight"] @ lora["blk.q.lora_down.weight"]
    merge_lora_weight(sd, lora, torch.bfloat16, strength=0.5)
    assert sd["blk.q.weight"].dtype == torch.float8_e4m3fn and sd["blk.q.scale_weight"].shape == (n,)
    got = dequantize_weight(sd, "blk.q.weight")
    # e4m3 has 3 mantissa bits: every element within 2^-4 of its channel's largest magnitude
    assert ((got - want).abs() <= want.abs().amax(dim=1, keepdim=True) * 2.0 ** -4 + 1e-12).all()
    assert torch.allclose(sd["blk.q.scale_weight"], want.abs().amax(dim=1) / 448, rtol=1e-6)
    # a weight the LoRA file does not cover is left alone
    assert torch.equal(sd["blk.o.weight"].view(torch.uint8), wq.view(torch.uint8))


def test_per_tensor_scale_and_native_prefix():
    g = torch.Generator().manual_seed(1)
    n, k, r = 32, 32, 4
    w = torch.randn(n, k, generator=g) * 0.02
    s0 = w.abs().max() / 448
    sd = {"blk.q.weight": (w / s0).to(torch.float8_e4m3fn), "blk.q.scale_weight": s0.clone()}
    lora = _lora(n, k, r, g, prefix="diffusion_model.")
    want = dequantize_weight(sd, "blk.q.weight") + (4.0 / r) * lora["diffusion_model.blk.q.lora_up.weight"] @ lora["diffusion_model.blk.q.lora_down.weight"]
    merge_lora_weight(sd, lora, torch.bfloat16)
    got = dequantize_weight(sd, "blk.q.weight")
    assert ((got - want).abs() <= want.abs().amax(dim=1, keepdim=True) * 2.0 ** -4 + 1e-12).all()


def test_high_precision_weight_matches_reference_formula():
    g = torch.Generator().manual_seed(2)
    n, k, r = 16, 24, 4
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16)
    sd = {"blk.q.weight": w.clone()}
    lora = _lora(n, k, r, g)
    del lora["blk.q.alpha"]  # no alpha: factor 1 (lora.py:102-108)
    merge_lora_weight(sd, lora, torch.bfloat16, strength=2.0)
    want = (w.float() + 2.0 * lora["blk.q.lora_up.weight"] @ lora["blk.q.lora_down.weight"]).to(torch.bfloat16)
    assert torch.equal(sd["blk.q.weight"], want)
