"""Oracle quantisers (plain torch, CPU).  Test infrastructure only.

These functions *define* the bit patterns the CUDA quantisers must reproduce.
Every floating-point step is an elementwise IEEE fp32 (or bf16/fp16) operation
or an order-independent max, so the result does not depend on reduction order
and can be matched bit-for-bit on the GPU.

Reference anchors
-----------------
* activation expression order ``(x * (1/scale).to(x.dtype)).to(float8_e4m3fn)``:
  ``ksana/operations/linear/fp8_linear.py:52-58``
* unscaled path ``clamp(x, -448, 448)`` then cast: ``fp8_linear.py:48-51``
* e4m3 is always the activation format: ``fp8_linear.py:46-47``
* GEMM ``_scaled_mm(a, w.t(), scale_a, scale_b, bias, out_dtype=x.dtype)``:
  ``fp8_linear.py:60-63``
* offline weight re-quantisation ``weight / scale_weight`` -> fp8:
  ``fp8_linear.py:145-150``
* Sage pre-pass shapes (K mean over tokens, Q block 128 / K block 64 INT8 with
  fp32 scales, per-(head, channel) V scale): the in-tree call sites
  ``ksana/operations/attention/backends/sage_sla.py:79,189-190,198-228``.
  The arithmetic itself lives in an un-vendored dependency: the definitions
  below are this build's contract (parity unpinned).
"""

from __future__ import annotations

import math

import torch

E4M3_MAX = 448.0
INT8_MAX = 127.0
LOG2E = 1.4426950408889634
Q_BLOCK = 128  # tokens per INT8 scale block of Q
K_BLOCK = 64  # tokens per INT8 scale block of K
KV_TILE = 128  # token padding granularity of the quantised K / V buffers


def _div(a: torch.Tensor, b: float) -> torch.Tensor:
    """IEEE fp32 division by a constant (forces a true elementwise divide)."""
    return a / torch.full_like(a, b)


# --------------------------------------------------------------------------- FP8 Linear


def act_quant_fp8_rowwise(x: torch.Tensor):
    """Per-token e4m3 quantisation of a [M, K] bf16/fp16 activation.

    s_m = absmax_k(x[m]) / 448 (fp32, 1.0 for an all-zero row);
    q = (x * (1/s_m).to(x.dtype)).to(e4m3)  -- the reference's expression order
    (fp8_linear.py:53-57) applied row-wise.
    Returns (q [M,K] float8_e4m3fn, s [M] fp32).
    """
    assert x.dim() == 2 and x.dtype in (torch.bfloat16, torch.float16)
    amax = x.float().abs().amax(dim=-1)
    s = torch.where(amax > 0, _div(amax, E4M3_MAX), torch.ones_like(amax))
    inv = (torch.ones_like(s) / s).to(x.dtype)
    q = (x * inv[:, None]).to(torch.float8_e4m3fn)
    return q, s


def act_quant_fp8_static(x: torch.Tensor, scale_input: torch.Tensor | None):
    """The reference's own per-tensor activation quantiser (fp8_linear.py:48-58).

    scale_input None  -> clamp(+-448) then cast (unscaled fp8 checkpoints);
    scale_input 0-d   -> (x * (1/scale).to(x.dtype)).to(e4m3), saturated at +-448
    (the CPU cast is non-saturating, the GPU kernel saturates; values are clamped
    here so both agree).
    """
    if scale_input is None:
        return torch.clamp(x, min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)
    y = x * (1.0 / scale_input.float()).to(x.dtype)
    return torch.clamp(y, min=-E4M3_MAX, max=E4M3_MAX).to(torch.float8_e4m3fn)


def weight_quant_fp8_channelwise(w: torch.Tensor):
    """Offline per-output-channel e4m3 quantisation of a [N, K] weight.

    s_n = absmax_k(W[n]) / 448; Wq = (W / s_n).to(e4m3).  Returns (Wq, s [N] fp32).
    """
    wf = w.float()
    amax = wf.abs().amax(dim=-1)
    s = torch.where(amax > 0, _div(amax, E4M3_MAX), torch.ones_like(amax))
    wq = (wf / s[:, None]).to(torch.float8_e4m3fn)
    return wq, s


def fp8_linear_emulated(x, wq, s_w, bias=None, out_dtype=None, s_x=None, xq=None):
    """y = (sum_k q[m,k] * Wq[n,k])_fp32 * s_m * s_n + bias[n] -> out_dtype.

    x: [..., K] bf16/fp16 (quantised per token here unless xq/s_x are given).
    s_w: [N] (per channel) or 0-d (per tensor, the reference's granularity).
    """
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if xq is None:
        xq, s_x = act_quant_fp8_rowwise(x2)
    acc = xq.float() @ wq.float().t()
    s_x = s_x.float().reshape(-1, 1) if s_x.dim() > 0 else s_x.float()
    s_w = s_w.float().reshape(1, -1) if s_w.dim() > 0 else s_w.float()
    y = acc * s_x * s_w
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype or x.dtype).reshape(*shape[:-1], wq.shape[0])


# --------------------------------------------------------------------------- Sage pre-passes


def q_premul(head_dim: int, sm_scale: float | None = None) -> float:
    """fp32 constant folded into Q before INT8 quantisation: softmax scale * log2(e).

    The Sage backend ignores a custom softmax_scale and uses head_dim**-0.5
    (sage_attn.py:75-81; attention_op.py:39).
    """
    sc = (head_dim**-0.5) if sm_scale is None else sm_scale
    return float(torch.tensor(sc * LOG2E, dtype=torch.float64).to(torch.float32))


def k_mean(k: torch.Tensor) -> torch.Tensor:
    """K smoothing vector: fp32 mean over all tokens, per (head, channel).  k: [L,H,D] -> [H,D].

    (sage_sla.py:198 ``km = k.mean(dim=-2)``.)  The sum is an fp32 reduction whose
    order is unspecified, so this is compared with a tolerance, and the INT8
    quantiser below takes the mean as an input.
    """
    return k.float().mean(dim=0)


def int8_block_quant(x: torch.Tensor, block: int, premul: float | None = None, mean: torch.Tensor | None = None):
    """Per-(head, token-block) INT8 quantisation.

    x: [L, H, D] bf16/fp16.  xf = float(x) (- mean[h,d]) (* premul), all fp32.
    scale[h,b] = absmax over the block's (tokens x D) / 127 (1.0 if the block is zero);
    q = clamp(round_half_even(xf * inv), -127, 127) with inv = 127 / absmax (1.0 if zero) -- one
    fp32 divide per block, one multiply per element.
    Returns (q8 [H, Lpad, D] int8 zero-padded to a multiple of 128 tokens,
             scale [H, Lpad // block] fp32 with 1.0 in fully padded blocks).
    """
    L, H, D = x.shape
    xf = x.float()
    if mean is not None:
        xf = xf - mean.float()[None]
    if premul is not None:
        xf = xf * torch.full((), premul, dtype=torch.float32)
    Lpad = (L + KV_TILE - 1) // KV_TILE * KV_TILE
    xp = torch.zeros(Lpad, H, D, dtype=torch.float32)
    xp[:L] = xf
    nb = Lpad // block
    xb = xp.view(nb, block, H, D)
    amax = xb.abs().amax(dim=(1, 3))  # [nb, H]
    scale = torch.where(amax > 0, _div(amax, INT8_MAX), torch.ones_like(amax))
    inv = torch.where(amax > 0, torch.full_like(amax, INT8_MAX) / amax, torch.ones_like(amax))
    q = torch.round(xb * inv[:, None, :, None]).clamp_(-INT8_MAX, INT8_MAX).to(torch.int8)
    q8 = q.view(Lpad, H, D).permute(1, 0, 2).contiguous()
    return q8, scale.t().contiguous()


def v_quant_fp8(v: torch.Tensor):
    """Per-(head, channel) e4m3 quantisation of V with the token axis made contiguous.

    v: [L,H,D].  s[h,d] = absmax over tokens / 448 (1.0 if zero); v8 = (float(v) * inv).to(e4m3) with
    inv = 448 / absmax (1.0 if zero), saturated at +-448.
    Returns (vt8 [H, D, Lpad] e4m3, zero padded to a multiple of 128 tokens; s [H, D] fp32).
    (Shape follows sage_sla.py:222-228: transpose + pad + per-(b,h,d) scale.)
    """
    L, H, D = v.shape
    vf = v.float()
    amax = vf.abs().amax(dim=0)  # [H, D]
    s = torch.where(amax > 0, _div(amax, E4M3_MAX), torch.ones_like(amax))
    inv = torch.where(amax > 0, torch.full_like(amax, E4M3_MAX) / amax, torch.ones_like(amax))
    v8 = (vf * inv[None]).clamp_(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    Lpad = (L + KV_TILE - 1) // KV_TILE * KV_TILE
    out = torch.zeros(H, D, Lpad, dtype=torch.uint8)
    out[:, :, :L] = v8.view(torch.uint8).permute(1, 2, 0)
    return out.view(torch.float8_e4m3fn), s


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def gemm_flops(M: int, N: int, K: int) -> float:
    return 2.0 * M * N * K


def attn_flops(H: int, Lq: int, Lk: int, D: int) -> float:
    return 4.0 * H * Lq * Lk * D


__all__ = [n for n in dir() if not n.startswith("_")] + ["_div"]
_ = math
