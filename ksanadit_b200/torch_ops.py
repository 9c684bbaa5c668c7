"""``torch.library`` registrations of the two contractions, so that code traced by ``torch.compile`` (KsanaDiT
breaks the graph at its attention op, ksana/operations/attention/attention_op.py:72) sees them as opaque
operators with known output shapes instead of ctypes calls it cannot trace:

    torch.ops.ksana_b200.fp8_linear(x, weight_e4m3, weight_scale, bias)  -> [..., N] in x.dtype
    torch.ops.ksana_b200.sage_attention(q, k, v)                        -> [L, H, 128] in q.dtype

The real implementations are the CUDA kernels (no CPU implementation is registered: calling the operators on
CPU tensors raises); the fake implementations only describe shapes and dtypes.
"""

from __future__ import annotations

import torch

from . import ops


@torch.library.custom_op("ksana_b200::fp8_linear", mutates_args=(), device_types="cuda")
def fp8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Per-token e4m3 quantisation of ``x`` + FP8 GEMM against ``weight`` [N, K] (e4m3) with per-channel scales."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    xq, sx = ops.quant_fp8_rowwise(x2)
    ws = weight_scale.float()
    ws = (ws.expand(weight.shape[0]) if ws.dim() == 0 else ws.reshape(weight.shape[0])).contiguous()
    out = ops.fp8_gemm(xq, sx, weight, ws, bias, out_dtype=x.dtype)
    return out.reshape(*shape[:-1], weight.shape[0])


@fp8_linear.register_fake
def _(x, weight, weight_scale, bias=None):
    return x.new_empty(*x.shape[:-1], weight.shape[0])


@torch.library.custom_op("ksana_b200::sage_attention", mutates_args=(), device_types="cuda")
def sage_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [Lq, H, 128], k / v [Lk, H, 128] (bf16 / fp16) -> [Lq, H, 128]; softmax scale 128^-0.5."""
    return ops.sage_attention(q, k, v)


@sage_attention.register_fake
def _(q, k, v):
    return q.new_empty(q.shape)
