"""FP8 quantized Linear for the B200 kernels behind KsanaDiT's Linear contract.

Mirrors ``Fp8Linear`` / ``scaled_fp8_ops().ScaledFp8Linear`` / ``pick_linear`` / ``find_fp8_info``
(ksana/operations/linear/fp8_linear.py:25-156, ksana/operations/linear/pick_linear.py:26-76):
same constructor, same parameter names (``weight`` [N,K] float8_e4m3fn, ``bias``, ``scale_weight``,
``scale_input``), ``reset_parameters`` that initialises nothing, ``forward`` on 2-D or 3-D input
returning ``input.dtype``.  Differences, all deliberate:

* scales may be per output channel (``scale_weight`` [N]) and activations are quantised per token
  unless a static ``scale_input`` is loaded -- a superset of the reference's per-tensor scalars, which
  are accepted and broadcast;
* failures raise.  The reference swallows any exception and silently runs an fp16 ``F.linear``
  (fp8_linear.py:82-92); here there is no other path.
"""

from __future__ import annotations

import torch

from . import _lib, ops
from .casting import stochastic_rounding
from .config import KsanaLinearBackend, backend_value

FP8 = torch.float8_e4m3fn
E4M3_MAX = 448.0


def quantize_weight_per_channel(w: torch.Tensor, seed: int | None = None):
    """Offline per-output-channel e4m3 quantisation: s_n = absmax_k / 448, Wq = (W / s_n) -> e4m3.

    ``seed`` None rounds to nearest even; an integer rounds stochastically with a generator seeded with it
    (``stochastic_rounding``, ksana/utils/ops.py:161-180), which keeps the expected value of a patched weight
    unbiased when small updates are merged repeatedly."""
    wf = w.float()
    amax = wf.abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / torch.full_like(amax, E4M3_MAX), torch.ones_like(amax))
    scaled = wf / s[:, None]
    return (scaled.to(FP8) if seed is None else stochastic_rounding(scaled, FP8, seed=seed)), s


def find_fp8_info(state_dict):
    """pick_linear.py:26-44: first fp8 dtype in the state dict, and whether scale_weight keys exist."""
    fp8_dtype, is_scaled = None, False
    for v in state_dict.values():
        if hasattr(v, "dtype") and v.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            fp8_dtype = v.dtype
            break
    for k in state_dict.keys():
        if k.endswith("scale_weight"):
            is_scaled = True
            break
    state_dict.pop("scaled_fp8", None)
    return fp8_dtype, is_scaled


class B200Fp8Linear(torch.nn.Linear):
    """Drop-in for ``operations.Linear`` when the checkpoint (or the dynamic backend) is FP8."""

    static_input_scale = False  # class switch set by b200_fp8_ops(scale_input=True)

    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=FP8)
        self.compute_dtype = dtype if dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        if self.bias is not None:
            self.bias = torch.nn.Parameter(torch.empty(out_features, device=device, dtype=self.compute_dtype), requires_grad=False)
        self.weight.requires_grad_(False)
        self._w_scale_vec = None

    def reset_parameters(self):
        # like the reference, nothing is initialised; the scale parameters are created so that a state
        # dict can be loaded without missing keys (ksana/utils/load.py:234-240 rejects missing keys)
        if not hasattr(self, "scale_weight"):
            self.scale_weight = torch.nn.Parameter(torch.ones((), device=self.weight.device, dtype=torch.float32), requires_grad=False)
        if not hasattr(self, "scale_input"):
            self.scale_input = (
                torch.nn.Parameter(torch.ones((), device=self.weight.device, dtype=torch.float32), requires_grad=False)
                if self.static_input_scale else None
            )
        return None

    # -- loading helpers -----------------------------------------------------------------------
    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        key = prefix + "scale_weight"
        if key in state_dict and state_dict[key].shape != self.scale_weight.shape:
            self.scale_weight = torch.nn.Parameter(torch.empty_like(state_dict[key], dtype=torch.float32, device=self.weight.device), requires_grad=False)
        self._w_scale_vec = None
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    @classmethod
    def from_float(cls, linear: torch.nn.Linear, dtype=torch.bfloat16):
        """Dynamic backend: quantise a high-precision Linear per output channel (replaces the torchao
        per-tensor path of ksana/utils/quantize.py:209-221)."""
        m = cls(linear.in_features, linear.out_features, bias=linear.bias is not None, device=linear.weight.device, dtype=dtype)
        wq, s = quantize_weight_per_channel(linear.weight.data)
        m.weight = torch.nn.Parameter(wq, requires_grad=False)
        m.scale_weight = torch.nn.Parameter(s, requires_grad=False)
        if linear.bias is not None:
            m.bias = torch.nn.Parameter(linear.bias.data.to(dtype), requires_grad=False)
        return m

    def weight_scale_vector(self) -> torch.Tensor:
        """[N] fp32 scale vector the GEMM consumes (a per-tensor scalar is broadcast once and cached)."""
        sw = self.scale_weight
        if self._w_scale_vec is None or self._w_scale_vec.device != self.weight.device:
            v = sw.detach().float().to(self.weight.device)
            self._w_scale_vec = (v.expand(self.out_features) if v.dim() == 0 else v.reshape(self.out_features)).contiguous()
        return self._w_scale_vec

    # -- forward --------------------------------------------------------------------------------
    def quantize_input(self, x2: torch.Tensor):
        if self.scale_input is not None:
            return ops.quant_fp8_static(x2, self.scale_input.detach().reshape(1).float())
        return ops.quant_fp8_rowwise(x2)

    def forward(self, input: torch.Tensor, epilogue=_lib.EPI_NONE, resid=None, gate=None) -> torch.Tensor:  # noqa: A002
        if self.weight.dtype != FP8:
            raise _lib.KsanaB200Error(f"B200Fp8Linear needs an e4m3 weight, found {self.weight.dtype}")
        if input.dim() not in (2, 3):
            raise ValueError(f"expected a 2-D or 3-D input, got {tuple(input.shape)}")  # fp8_linear.py:30-37 returns None here
        if input.dtype not in (torch.bfloat16, torch.float16):
            raise TypeError(f"expected bf16/fp16 activations, got {input.dtype}")
        shape = input.shape
        x2 = input.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        xq, sx = self.quantize_input(x2)
        bias = None if self.bias is None else self.bias
        if resid is not None:
            resid = resid.reshape(-1, self.out_features)
        out = ops.fp8_gemm(xq, sx, self.weight.data, self.weight_scale_vector(), bias, out_dtype=input.dtype, epilogue=epilogue,
                           resid=resid, gate=gate)
        return out.reshape(*shape[:-1], self.out_features)

    def forward_quantized(self, xq, sx, out_dtype, epilogue=_lib.EPI_NONE, resid=None, gate=None, out=None):
        """GEMM on an already quantised activation (used by the fused block path)."""
        return ops.fp8_gemm(xq, sx, self.weight.data, self.weight_scale_vector(), self.bias, out_dtype=out_dtype, epilogue=epilogue,
                            resid=resid, gate=gate, out=out)

    def forward_quantized_rowstats(self, xq, sx, out_dtype, sumsq_cols):
        """forward_quantized that also returns the per-tile row sums of squares of the first ``sumsq_cols`` output
        columns ([sumsq_cols / 256, M] fp32): the statistics of an RMSNorm that follows this projection."""
        return ops.fp8_gemm_rowstats(xq, sx, self.weight.data, self.weight_scale_vector(), self.bias, sumsq_cols, out_dtype=out_dtype)

    # API kept from ScaledFp8Linear (fp8_linear.py:138-154)
    def convert_weight(self, weight, inplace=False, **kwargs):
        s = self.weight_scale_vector().to(weight.dtype)[:, None]
        if inplace:
            weight *= s
            return weight
        return weight * s

    def set_weight(self, weight, inplace_update=False, seed=None, **kwargs):
        """Re-quantises ``weight`` with the scales already loaded (fp8_linear.py:145-154).  With an integer ``seed``
        the rounding is the reference's seeded stochastic rounding; without one (the reference would fail on a
        None seed) it is round-to-nearest-even."""
        scaled = weight.float() / self.weight_scale_vector().to(weight.device)[:, None]
        if seed is None:
            wq = scaled.clamp(-E4M3_MAX, E4M3_MAX).to(FP8)
        else:
            wq = stochastic_rounding(scaled, FP8, seed=int(seed))
        if inplace_update:
            self.weight.data.copy_(wq)
        else:
            self.weight = torch.nn.Parameter(wq, requires_grad=False)


def b200_fp8_ops(scale_input: bool = False, override_dtype=None):
    """Class factory with the shape of ``scaled_fp8_ops`` (fp8_linear.py:95-156)."""
    if override_dtype not in (None, FP8):
        raise _lib.KsanaB200Error(f"only float8_e4m3fn weights are supported, got {override_dtype}")

    class B200ScaledFp8Linear(B200Fp8Linear):
        static_input_scale = bool(scale_input)

    return B200ScaledFp8Linear


def pick_linear(run_dtype, state_dict, linear_backend, load_device=None):
    """pick_linear.py:48-76 for this library: which Linear class the Ops registry gets.

    FP8 checkpoints (or the FP8_GEMM backends) get the B200 class; anything else is outside this
    library and is reported, not silently replaced.
    """
    fp8_dtype, is_scaled = find_fp8_info(state_dict)
    lb = backend_value(linear_backend)
    if lb == KsanaLinearBackend.FP8_GEMM.value and fp8_dtype is None:
        raise ValueError("Could not find fp8 dtype in state_dict when linear_backend is fp8_gemm")
    if lb == KsanaLinearBackend.FP8_GEMM_DYNAMIC.value:
        return B200Fp8Linear  # weights are quantised at load with B200Fp8Linear.from_float
    if fp8_dtype is not None and lb in (KsanaLinearBackend.DEFAULT.value, KsanaLinearBackend.FP8_GEMM.value):
        if fp8_dtype != FP8:
            raise _lib.KsanaB200Error(f"{fp8_dtype} checkpoints are not supported (e4m3 only)")
        return b200_fp8_ops(scale_input=False, override_dtype=fp8_dtype) if is_scaled else B200Fp8Linear
    raise _lib.KsanaB200Error(f"linear_backend={lb} without an fp8 checkpoint is not an FP8 path; keep KsanaDiT's own Linear for it")
