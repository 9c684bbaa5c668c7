"""Weight / bias casting helpers and seeded stochastic rounding to FP8, behind the names KsanaDiT's Linear uses.

Mirrors ``cast_to`` / ``cast_bias_weight`` / ``manual_stochastic_round_to_float8`` / ``stochastic_rounding``
(ksana/utils/ops.py:74-110,131-180).  These run when weights are loaded or patched (LoRA merge, ``set_weight``),
never inside a denoise step, so they are plain torch tensor expressions on whatever device the weight lives on.

Stochastic rounding follows the published scheme the reference uses: the value is taken to fp16, split into
sign, a clamped exponent and a mantissa scaled to the target's mantissa grid; a uniform draw in [0, 1) from a
seeded generator is added before flooring, so a value between two FP8 neighbours goes up with a probability
equal to its position between them.  Draws are made per slice of rows, in fp16, from ``torch.Generator``
seeded once per call -- the same stream of draws as the reference, which makes the result reproducible
against it bit for bit on the same device (checked against the reference on the CPU by the golden vectors).
"""

from __future__ import annotations

import torch

_FP8_LAYOUT = {torch.float8_e4m3fn: (4, 3, 7), torch.float8_e5m2: (5, 2, 15)}  # exponent bits, mantissa bits, bias
_ROWS_PER_DRAW = 4096 * 4096  # elements per generator draw: large weights are rounded in row slices of about this size


def cast_to(weight, dtype=None, device=None, non_blocking=False, copy=False, stream=None):
    """``weight`` as ``dtype`` on ``device``; the same tensor comes back when nothing has to change."""
    same_device = device is None or weight.device == torch.device(device)
    if same_device and not copy and (dtype is None or weight.dtype == dtype):
        return weight

    def convert():
        if same_device:
            return weight.to(dtype=dtype, copy=copy)
        out = torch.empty_like(weight, dtype=dtype, device=device)
        out.copy_(weight, non_blocking=non_blocking)
        return out

    if stream is None:
        return convert()
    with stream:
        return convert()


def cast_bias_weight(module, input=None, dtype=None, device=None, bias_dtype=None):  # noqa: A002
    """(weight, bias) of ``module`` cast for a matmul with ``input``: dtype / device default to the input's, the
    bias dtype to the weight's target dtype."""
    if input is not None:
        dtype = input.dtype if dtype is None else dtype
        bias_dtype = dtype if bias_dtype is None else bias_dtype
        device = input.device if device is None else device
    non_blocking = device is not None and torch.device(device).type == "cuda"
    bias = None if module.bias is None else cast_to(module.bias, bias_dtype, device, non_blocking=non_blocking)
    return cast_to(module.weight, dtype, device, non_blocking=non_blocking), bias


def _round_slice(x, dtype, generator):
    e_bits, m_bits, bias = _FP8_LAYOUT[dtype]
    h = x.half()
    mag = h.abs()
    sign = torch.sign(h)
    sign = torch.where(mag == 0, torch.zeros_like(sign), sign)
    expo = torch.clamp(torch.floor(torch.log2(mag)) + bias, 0, 2 ** e_bits - 1)
    normal = expo != 0
    # position on the mantissa grid of the value's binade (normal) or of the subnormal range
    grid = torch.where(normal, (mag / (2.0 ** (expo - bias)) - 1.0) * (2 ** m_bits), mag / (2.0 ** (1 - bias - m_bits)))
    grid = grid + torch.rand(grid.size(), dtype=grid.dtype, layout=grid.layout, device=grid.device, generator=generator)
    frac = grid.floor() / (2 ** m_bits)
    out = sign * torch.where(normal, (2.0 ** (expo - bias)) * (1.0 + frac), (2.0 ** (1 - bias)) * frac)
    lim = torch.finfo(dtype)
    return torch.clamp(out, min=lim.min, max=lim.max)


def manual_stochastic_round_to_float8(x, dtype, generator=None):
    """fp16 tensor on the FP8 grid of ``dtype`` (not yet cast), one uniform draw per element from ``generator``."""
    if dtype not in _FP8_LAYOUT:
        raise ValueError("Unsupported dtype")
    return _round_slice(x, dtype, generator)


def stochastic_rounding(value, dtype, seed=0):
    """``value`` in ``dtype``; FP8 targets are rounded stochastically with a generator seeded with ``seed``."""
    if dtype not in _FP8_LAYOUT:
        return value.to(dtype=dtype)
    gen = torch.Generator(device=value.device)
    gen.manual_seed(seed)
    out = torch.empty_like(value, dtype=dtype)
    n_slices = max(1, value.numel() / _ROWS_PER_DRAW)
    step = max(1, round(value.shape[0] / n_slices))
    for r0 in range(0, value.shape[0], step):
        out[r0:r0 + step].copy_(_round_slice(value[r0:r0 + step], dtype, gen))
    return out
