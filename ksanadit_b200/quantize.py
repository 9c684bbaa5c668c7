"""Dynamic FP8 quantisation of a loaded high-precision model (the ``fp8_gemm_dynamic`` linear backend).

Mirrors ``DEFAULT_FP8_EXCLUDE_LAYERS`` / ``_apply_dynamic_fp8_quant`` / ``apply_dynamic_fp8_quant``
(ksana/utils/quantize.py:29-33,209-404,427-453): every ``torch.nn.Linear`` of the model whose two dimensions are
multiples of 16 and whose qualified name contains none of the exclude patterns is quantised; embedding layers
and the output heads (``embed``, ``proj_out``, ``head``) stay in their original precision.  The reference hands
those layers to torchao (per-tensor dynamic FP8); here each is replaced by a ``B200Fp8Linear`` holding e4m3
weights with one scale per output channel, and activations are quantised per token at run time -- a finer
granularity over the same selection of layers.  Nothing is swallowed: a layer that cannot be converted raises.
"""

from __future__ import annotations

import torch

from .linear import B200Fp8Linear

DEFAULT_FP8_EXCLUDE_LAYERS: list[str] = ["embed", "proj_out", "head"]


def is_eligible_linear(name: str, module: torch.nn.Module, exclude_layers=None) -> bool:
    """The reference's filter (quantize.py:324-346): a plain Linear, both dims % 16 == 0, no exclude pattern in its name."""
    if not isinstance(module, torch.nn.Linear) or isinstance(module, B200Fp8Linear):
        return False
    if module.in_features % 16 != 0 or module.out_features % 16 != 0:
        return False
    patterns = DEFAULT_FP8_EXCLUDE_LAYERS if exclude_layers is None else exclude_layers
    return not any(p in name for p in patterns)


def eligible_linear_names(model: torch.nn.Module, exclude_layers=None) -> list[str]:
    return [n for n, m in model.named_modules() if is_eligible_linear(n, m, exclude_layers)]


def _apply_dynamic_fp8_quant(model: torch.nn.Module, exclude_layers=None, dtype=None) -> list[str]:
    """Replaces every eligible Linear in place; returns the qualified names that were converted."""
    names = eligible_linear_names(model, exclude_layers)
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, leaf)
        run_dtype = dtype or (old.weight.dtype if old.weight.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16)
        setattr(parent, leaf, B200Fp8Linear.from_float(old, dtype=run_dtype))
    return names


def apply_dynamic_fp8_quant(model: torch.nn.Module, load_device=None) -> bool:
    """quantize.py:427-453: move the model to ``load_device`` when it is a CUDA device, then quantise.

    Returns False (and changes nothing) for a missing or parameter-less model, True otherwise."""
    if model is None:
        return False
    try:
        current = next(model.parameters()).device
    except StopIteration:
        return False
    if current.type != "cuda" and load_device is not None and torch.device(load_device).type == "cuda":
        model.to(torch.device(load_device))
    _apply_dynamic_fp8_quant(model)
    return True
