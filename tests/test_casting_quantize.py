"""Host logic (CPU): weight casting, seeded stochastic FP8 rounding, and the dynamic-FP8 model walk."""

import torch

from ksanadit_b200 import casting, linear, quantize


def test_stochastic_rounding_matches_reference_vectors(golden):
    """Bytes produced by the reference's ``stochastic_rounding`` (ksana/utils/ops.py:161-180) on the CPU."""
    for name in ("e4m3", "e5m2"):
        v = golden["stochastic_rounding"][name]
        dt = torch.float8_e4m3fn if name == "e4m3" else torch.float8_e5m2
        got = casting.stochastic_rounding(v["x"].clone(), dt, seed=int(v["seed"]))
        assert got.dtype == dt and torch.equal(got.view(torch.uint8), v["y"])
        other = casting.stochastic_rounding(v["x"].clone(), dt, seed=int(v["seed"]) + 1)
        assert not torch.equal(other.view(torch.uint8), v["y"])


def test_stochastic_rounding_is_unbiased_and_stays_on_neighbours():
    x = torch.full((4096, 16), 1.3)  # between the e4m3 neighbours 1.25 and 1.375
    y = casting.stochastic_rounding(x, torch.float8_e4m3fn, seed=5).float()
    assert set(y.unique().tolist()) == {1.25, 1.375}
    assert abs(float(y.mean()) - 1.3) < 2e-3  # P(up) = 0.4
    assert torch.equal(casting.stochastic_rounding(x, torch.float8_e4m3fn, seed=5).float(), y)
    big = casting.stochastic_rounding(torch.tensor([[1e4, -1e4, 0.0]]), torch.float8_e4m3fn, seed=0).float()
    assert big.tolist() == [[448.0, -448.0, 0.0]]
    assert casting.stochastic_rounding(x, torch.bfloat16).dtype == torch.bfloat16  # non-FP8 targets are plain casts


def test_cast_helpers_follow_the_reference_contract():
    w = torch.randn(4, 4)
    assert casting.cast_to(w) is w and casting.cast_to(w, torch.float32, torch.device("cpu")) is w
    c = casting.cast_to(w, copy=True)
    assert c is not w and torch.equal(c, w)
    assert casting.cast_to(w, torch.bfloat16).dtype == torch.bfloat16
    lin = torch.nn.Linear(4, 4)
    x = torch.zeros(2, 4, dtype=torch.bfloat16)
    wt, b = casting.cast_bias_weight(lin, x)
    assert wt.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    wt, b = casting.cast_bias_weight(lin, x, dtype=torch.float16, bias_dtype=torch.float32)
    assert wt.dtype == torch.float16 and b.dtype == torch.float32
    lin.bias = None
    assert casting.cast_bias_weight(lin, x)[1] is None


def test_set_weight_seeded_rounding_and_default():
    m = linear.B200Fp8Linear(32, 16, bias=False)
    w = torch.randn(16, 32) * 0.02
    wq, s = linear.quantize_weight_per_channel(w)
    m.load_state_dict({"weight": wq, "scale_weight": s}, strict=False)
    target = w + 0.001 * torch.randn(16, 32)
    m.set_weight(target, inplace_update=True)
    rne = m.weight.data.clone()
    assert torch.equal(rne.view(torch.uint8), (target / s[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8))
    m.set_weight(target, seed=3)
    a = m.weight.data.clone()
    m.set_weight(target, seed=3)
    assert torch.equal(a.view(torch.uint8), m.weight.data.view(torch.uint8))
    want = casting.stochastic_rounding(target / s[:, None], torch.float8_e4m3fn, seed=3)
    assert torch.equal(a.view(torch.uint8), want.view(torch.uint8))
    m.set_weight(target, seed=4)
    assert not torch.equal(a.view(torch.uint8), m.weight.data.view(torch.uint8))
    assert not torch.equal(a.view(torch.uint8), rne.view(torch.uint8))


class _ToyDiT(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.patch_embedding = torch.nn.Linear(64, 64)       # excluded: "embed"
        self.time_embedder = torch.nn.Sequential(torch.nn.Linear(32, 64))  # excluded: "embed"
        blk = torch.nn.Module()
        blk.q = torch.nn.Linear(64, 64)
        blk.ffn = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.GELU(), torch.nn.Linear(96, 64, bias=False))
        blk.odd = torch.nn.Linear(64, 40)                     # 40 % 16 != 0
        blk.norm = torch.nn.LayerNorm(64)
        self.blocks = torch.nn.ModuleList([blk])
        self.head = torch.nn.Module()
        self.head.head = torch.nn.Linear(64, 64)              # excluded: "head"
        self.proj_out = torch.nn.Linear(64, 64)               # excluded: "proj_out"


def test_dynamic_fp8_walk_selects_what_the_reference_selects():
    model = _ToyDiT().to(torch.bfloat16)
    assert quantize.eligible_linear_names(model) == ["blocks.0.q", "blocks.0.ffn.0", "blocks.0.ffn.2"]
    w_before = model.blocks[0].q.weight.data.float().clone()
    assert quantize.apply_dynamic_fp8_quant(model) is True
    q = model.blocks[0].q
    assert isinstance(q, linear.B200Fp8Linear) and q.weight.dtype == torch.float8_e4m3fn and q.scale_weight.shape == (64,)
    assert q.bias is not None and model.blocks[0].ffn[2].bias is None
    deq = q.weight.data.float() * q.scale_weight[:, None]
    assert (deq - w_before).abs().max() <= w_before.abs().amax() * 2.0 ** -4
    for kept in (model.patch_embedding, model.time_embedder[0], model.blocks[0].odd, model.head.head, model.proj_out):
        assert type(kept) is torch.nn.Linear and kept.weight.dtype == torch.bfloat16
    assert quantize.eligible_linear_names(model) == []  # idempotent: converted layers are not picked again
    assert quantize.apply_dynamic_fp8_quant(None) is False and quantize.apply_dynamic_fp8_quant(torch.nn.ReLU()) is False
    assert quantize.eligible_linear_names(_ToyDiT(), exclude_layers=["blocks"]) == ["patch_embedding", "time_embedder.0", "head.head", "proj_out"]
