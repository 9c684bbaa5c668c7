"""GPU parity: tcgen05 FP8 GEMM (per-token x per-channel scales, fused epilogues) vs the oracle."""

import pytest
import torch

from conftest import cosine, max_abs_rel
from oracle import dit_ops as D
from oracle import quantizers as Qz

pytestmark = pytest.mark.gpu

# tolerance of the GEMM output against the oracle's fp32-accumulated result rounded to bf16:
# one bf16 ulp of the row's largest output plus accumulation-order noise
GEMM_MAX_ABS_REL = 1e-2
GEMM_COS = 0.9999


def _mk(M, N, K, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = D.make_activations(M, K, seed=seed, dtype=dtype)
    w = (torch.randn(N, K, generator=g) * 0.02).to(dtype)
    b = (torch.randn(N, generator=g) * 0.02).to(dtype)
    xq, sx = Qz.act_quant_fp8_rowwise(x)
    wq, sw = Qz.weight_quant_fp8_channelwise(w)
    return x, xq, sx, wq, sw, b


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 128),      # exactly one tile, one k step
    (128, 256, 512),      # ring wraps once
    (1, 8, 16),           # smallest legal problem
    (80, 256, 1024),      # ragged M
    (300, 520, 144),      # ragged M, N, K
    (1560, 1536, 1536),   # Wan2.1-1.3B-shaped o-proj
    (2500, 4608, 1536),   # more tiles than SMs: persistent loop + both accumulators
])
def test_gemm_matches_oracle(M, N, K):
    from ksanadit_b200 import _lib, ops
    x, xq, sx, wq, sw, b = _mk(M, N, K, seed=M + N + K)
    ref = Qz.fp8_linear_emulated(x, wq, sw, b, xq=xq, s_x=sx)
    out = ops.fp8_gemm(xq.cuda(), sx.cuda(), wq.cuda(), sw.cuda(), b.cuda(), out_dtype=torch.bfloat16)
    _lib.assert_device_ok()
    assert max_abs_rel(out.cpu().float(), ref.float()) <= GEMM_MAX_ABS_REL
    assert cosine(out.cpu(), ref) >= GEMM_COS


def test_gemm_fp16_no_bias_and_determinism():
    from ksanadit_b200 import ops
    x, xq, sx, wq, sw, _ = _mk(200, 512, 256, seed=1, dtype=torch.float16)
    ref = Qz.fp8_linear_emulated(x, wq, sw, None, xq=xq, s_x=sx)
    a = ops.fp8_gemm(xq.cuda(), sx.cuda(), wq.cuda(), sw.cuda(), None, out_dtype=torch.float16)
    b2 = ops.fp8_gemm(xq.cuda(), sx.cuda(), wq.cuda(), sw.cuda(), None, out_dtype=torch.float16)
    assert torch.equal(a, b2)
    assert max_abs_rel(a.cpu().float(), ref.float()) <= GEMM_MAX_ABS_REL


def test_gemm_gelu_epilogue():
    from ksanadit_b200 import _lib, ops
    x, xq, sx, wq, sw, b = _mk(260, 768, 256, seed=2)
    ref = D.gelu_tanh(Qz.fp8_linear_emulated(x, wq, sw, b, xq=xq, s_x=sx))
    out = ops.fp8_gemm(xq.cuda(), sx.cuda(), wq.cuda(), sw.cuda(), b.cuda(), epilogue=_lib.EPI_GELU_TANH)
    assert max_abs_rel(out.cpu().float(), ref.float()) <= GEMM_MAX_ABS_REL


@pytest.mark.parametrize("gate_rows", [1, 260])
def test_gemm_gate_residual_epilogue(gate_rows):
    from ksanadit_b200 import _lib, ops
    M, N, K = 260, 512, 256
    x, xq, sx, wq, sw, b = _mk(M, N, K, seed=3)
    g = torch.Generator().manual_seed(4)
    resid = torch.randn(M, N, generator=g).to(torch.bfloat16)
    gate = torch.randn(gate_rows, N, generator=g).to(torch.bfloat16)
    y = Qz.fp8_linear_emulated(x, wq, sw, b, xq=xq, s_x=sx)
    ref = D.gate_residual(resid, y, gate)
    out = ops.fp8_gemm(xq.cuda(), sx.cuda(), wq.cuda(), sw.cuda(), b.cuda(), epilogue=_lib.EPI_GATE_RESIDUAL,
                       resid=resid.cuda(), gate=gate.cuda())
    assert max_abs_rel(out.cpu().float(), ref.float()) <= GEMM_MAX_ABS_REL


def test_gemm_reference_per_tensor_vector(golden):
    """The reference's own per-tensor fp8_linear output (fp8_linear.py:25-73), reproduced by expanding
    its scalar scales to vectors."""
    from ksanadit_b200 import ops
    g = golden["fp8_pt"]
    xq = g["xq"].view(torch.float8_e4m3fn).cuda()
    wq = g["wq"].view(torch.float8_e4m3fn).cuda()
    M, N = xq.shape[0], wq.shape[0]
    out = ops.fp8_gemm(xq, g["si"].expand(M).contiguous().cuda(), wq, g["sw"].expand(N).contiguous().cuda(), g["bias"].cuda())
    assert (out.cpu().float() - g["y"].reshape(M, N).float()).abs().max() <= 2e-3


def test_gemm_rejects_bad_arguments():
    from ksanadit_b200 import _lib, ops
    a = torch.zeros(4, 24, dtype=torch.float8_e4m3fn, device="cuda")
    w = torch.zeros(8, 24, dtype=torch.float8_e4m3fn, device="cuda")
    with pytest.raises(_lib.KsanaB200Error):
        ops.fp8_gemm(a, torch.ones(4, device="cuda"), w, torch.ones(8, device="cuda"))


def test_gemm_linearity_at_full_width():
    """Size-independent property at a Wan2.2-14B layer width: scaling the row scales scales the output."""
    from ksanadit_b200 import ops
    M, N, K = 1024, 5120, 5120
    g = torch.Generator(device="cuda").manual_seed(0)
    xq = (torch.randn(M, K, device="cuda", generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    wq = (torch.randn(N, K, device="cuda", generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    sx = torch.rand(M, device="cuda", generator=g) + 0.5
    sw = torch.rand(N, device="cuda", generator=g) * 1e-4
    a = ops.fp8_gemm(xq, sx, wq, sw).float()
    b2 = ops.fp8_gemm(xq, sx * 2, wq, sw).float()
    assert max_abs_rel(b2, a * 2) <= 1e-2
    ref = (xq[:64].float() @ wq.float().t()) * sx[:64, None] * sw[None]
    assert max_abs_rel(a[:64], ref) <= GEMM_MAX_ABS_REL


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 200, 80), (1000, 768, 512), (129, 520, 1040)])
@pytest.mark.parametrize("epilogue", ["none", "gelu", "gate"])
def test_cta_pair_form_gives_the_bits_of_the_single_cta_form(M, N, K, epilogue):
    """tcgen05.mma.cta_group::2 (two CTAs of a cluster on one 256-row tile, each with its own half of the operands) and
    cta_group::1 accumulate the same products in the same order: equal outputs, ragged edges included (a pair whose
    second CTA has no rows at all, a W tile cut by N, a K tail)."""
    from ksanadit_b200 import _lib, ops
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    xq = (torch.randn(M, K, device="cuda", generator=g) * 50).clamp(-448, 448).to(torch.float8_e4m3fn)
    wq = (torch.randn(N, K, device="cuda", generator=g) * 50).clamp(-448, 448).to(torch.float8_e4m3fn)
    sx, sw = torch.rand(M, device="cuda", generator=g) + 0.5, (torch.rand(N, device="cuda", generator=g) + 0.5) * 5e-4
    bias = torch.randn(N, device="cuda", generator=g).to(torch.bfloat16)
    epi = {"none": _lib.EPI_NONE, "gelu": _lib.EPI_GELU_TANH, "gate": _lib.EPI_GATE_RESIDUAL}[epilogue]
    resid = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16) if epilogue == "gate" else None
    gate = torch.randn(1, N, device="cuda", generator=g).to(torch.bfloat16) if epilogue == "gate" else None
    before = lib.ksb_gemm_pair_mode(-1)
    try:
        outs = []
        for mode in (0, 1):
            lib.ksb_gemm_pair_mode(mode)
            assert lib.ksb_gemm_pair_mode(-1) == mode
            outs.append(ops.fp8_gemm(xq, sx, wq, sw, bias, epilogue=epi, resid=resid, gate=gate))
            _lib.assert_device_ok()
    finally:
        lib.ksb_gemm_pair_mode(before)
    assert torch.equal(outs[0], outs[1])
