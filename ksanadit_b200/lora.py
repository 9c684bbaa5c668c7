"""LoRA merge into FP8 checkpoints at load time (host-side torch, runs on whatever device the state dict is on).

Mirror of KsanaDiT's ``merge_lora_weight`` (ksana/utils/lora.py:85-126) with one difference that matters for
FP8: the reference writes ``W * scale_weight + delta`` back into the e4m3 tensor while leaving ``scale_weight`` as
it was; here the merged matrix is re-quantised with a fresh scale per output channel (the granularity the
B200 GEMM consumes), and ``<name>.scale_weight`` is replaced by that ``[N]`` vector.  High-precision weights are
merged exactly as in the reference.  Name conventions (``diffusion_model.`` prefix of native LoRA files,
``.lora_down.weight`` / ``.lora_up.weight`` / ``.alpha``) are the reference's (lora.py:46-51).
"""

from __future__ import annotations

import torch

from .linear import quantize_weight_per_channel

FP8_TYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def build_lora_names(key: str, lora_down_key: str, lora_up_key: str, is_native_weight: bool):
    base = "diffusion_model." if is_native_weight else ""
    stem = key[: -len(".weight")]
    return base + stem + lora_down_key, base + stem + lora_up_key, base + stem + ".alpha"


def dequantize_weight(model_sd: dict, key: str) -> torch.Tensor:
    """fp32 value of ``model_sd[key]``: FP8 weights times their ``scale_weight`` (0-d or per output channel)."""
    w = model_sd[key]
    if w.dtype not in FP8_TYPES:
        return w.float()
    s = model_sd.get(key[: -len(".weight")] + ".scale_weight")
    wf = w.float()
    if s is None:
        return wf
    s = s.float().to(w.device)
    return wf * (s.reshape(-1, 1) if s.dim() > 0 and s.numel() > 1 else s.reshape(()))


def merge_lora_weight(model_sd: dict, lora_sd: dict, run_dtype: torch.dtype, lora_down_key: str = ".lora_down.weight",
                      lora_up_key: str = ".lora_up.weight", strength: float = 1.0, seed: int | None = None) -> dict:
    """Adds ``strength * alpha / rank * up @ down`` to every weight of ``model_sd`` the LoRA file covers, in place.

    e4m3 weights come back as e4m3 with a per-output-channel ``scale_weight``; other dtypes come back in
    ``run_dtype``.  ``seed``: round the re-quantised e4m3 weights stochastically (seeded, one stream per weight:
    ``seed`` + its position in the state dict) instead of to nearest even.  Returns ``model_sd``.
    """
    is_native_weight = any("diffusion_model." in k for k in lora_sd)
    for index, key in enumerate([k for k in model_sd if k.endswith(".weight")]):
        down_name, up_name, alpha_name = build_lora_names(key, lora_down_key, lora_up_key, is_native_weight)
        if down_name not in lora_sd:
            continue
        if up_name not in lora_sd:
            raise KeyError(f"{down_name} has no matching {up_name}")
        value = model_sd[key]
        down = lora_sd[down_name].to(value.device, torch.float32)
        up = lora_sd[up_name].to(value.device, torch.float32)
        factor = float(lora_sd[alpha_name]) / down.shape[0] if alpha_name in lora_sd else 1.0
        if up.shape[0] != value.shape[0] or down.shape[1] != value.shape[1] or up.shape[1] != down.shape[0]:
            raise ValueError(f"LoRA shapes {tuple(up.shape)} x {tuple(down.shape)} do not fit {key} {tuple(value.shape)}")
        merged = dequantize_weight(model_sd, key).addmm_(up, down, alpha=strength * factor)
        if value.dtype in FP8_TYPES:
            if value.dtype != torch.float8_e4m3fn:
                raise ValueError(f"{key}: only float8_e4m3fn weights are supported, got {value.dtype}")
            wq, s = quantize_weight_per_channel(merged, seed=None if seed is None else seed + index)
            model_sd[key] = wq
            model_sd[key[: -len(".weight")] + ".scale_weight"] = s
        else:
            model_sd[key] = merged.to(run_dtype)
    return model_sd
