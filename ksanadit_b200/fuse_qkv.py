"""QKV-fused projection for the FP8 Linear, behind KsanaDiT's fusion switch and state-dict remap.

Mirrors ``MODEL_QKV_PATTERNS`` / ``should_use_qkv_fusion`` / ``remap_qkv_weights`` /
``remap_state_dict_for_model`` / ``QKVProjectionMixin`` (ksana/operations/fuse_qkv/fuse_qkv.py:25-233).
The reference disables fusion globally (fuse_qkv.py:36-38) and its remap concatenates only ``.weight``
and ``.bias`` (fuse_qkv.py:84-128); here fusion is on for the B200 Linear, and the three projections'
``scale_weight`` (scalars or vectors) become one per-output-channel vector of length 3*dim, which is
what lets checkpoints whose q/k/v carry different per-tensor scales share one GEMM.
"""

from __future__ import annotations

import torch

MODEL_QKV_PATTERNS = {
    "wan": [(".self_attn.q", ".self_attn.k", ".self_attn.v", ".self_attn.qkv")],
    "qwen": [(".to_q", ".to_k", ".to_v", ".to_qkv"), (".add_q_proj", ".add_k_proj", ".add_v_proj", ".add_qkv_proj")],
}


def should_use_qkv_fusion(operations) -> bool:
    """True when the registry's Linear is the B200 FP8 Linear (or no registry is given)."""
    if operations is None:
        return True
    from .linear import B200Fp8Linear
    cls = getattr(operations, "Linear", None)
    return isinstance(cls, type) and issubclass(cls, B200Fp8Linear)


def _scale_vec(t, n):
    t = t.float()
    return t.expand(n).clone() if t.dim() == 0 else t.reshape(n)


def remap_qkv_weights(state_dict, patterns, inplace=True):
    """Concatenates q|k|v rows of weight / bias / scale_weight under the fused name.  scale_input (static
    activation scales) cannot be merged unless equal; unequal ones are dropped in favour of per-token scales."""
    sd = state_dict if inplace else dict(state_dict)
    for q_sfx, k_sfx, v_sfx, f_sfx in patterns:
        for key in [k for k in list(sd.keys()) if k.endswith(q_sfx + ".weight")]:
            prefix = key[: -len(q_sfx + ".weight")]
            names = [prefix + s for s in (q_sfx, k_sfx, v_sfx)]
            if not all(n + ".weight" in sd for n in names):
                continue
            ws = [sd.pop(n + ".weight") for n in names]
            fused = prefix + f_sfx
            sd[fused + ".weight"] = torch.cat([w.view(torch.uint8) for w in ws], dim=0).view(ws[0].dtype) if ws[0].dtype.itemsize == 1 else torch.cat(ws, dim=0)
            if all(n + ".bias" in sd for n in names):
                sd[fused + ".bias"] = torch.cat([sd.pop(n + ".bias") for n in names], dim=0)
            if any(n + ".scale_weight" in sd for n in names):
                vecs = []
                for n, w in zip(names, ws):
                    s = sd.pop(n + ".scale_weight", torch.ones((), dtype=torch.float32))
                    vecs.append(_scale_vec(s, w.shape[0]))
                sd[fused + ".scale_weight"] = torch.cat(vecs, dim=0)
            si = [sd.pop(n + ".scale_input", None) for n in names]
            if all(s is not None for s in si) and all(torch.equal(si[0], s) for s in si[1:]):
                sd[fused + ".scale_input"] = si[0]
    return sd


def remap_state_dict_for_model(model, state_dict, model_name):
    """fuse_qkv.py:153-194: remap when any module of the model was built fused."""
    fused = any(getattr(m, "qkv_fused", False) for m in model.modules())
    if not fused:
        return state_dict
    key = "wan" if "wan" in model_name.lower() else "qwen" if "qwen" in model_name.lower() else None
    if key is None:
        return state_dict
    return remap_qkv_weights(state_dict, MODEL_QKV_PATTERNS[key])


class QKVProjectionMixin:
    """fuse_qkv.py:197-233, unchanged in shape: one fused Linear(dim, 3*dim) or three Linear(dim, dim)."""

    def _setup_qkv_projection(self, dim, operations, device=None, dtype=None, bias=True, fused_name="qkv",
                              separate_names=("q", "k", "v"), prefix=""):
        fused = should_use_qkv_fusion(operations)
        if not hasattr(self, "_qkv_configs"):
            self._qkv_configs = {}
        self._qkv_configs[prefix] = {"fused": fused, "fused_name": fused_name, "separate_names": separate_names}
        self.qkv_fused = getattr(self, "qkv_fused", False) or fused
        if fused:
            setattr(self, fused_name, operations.Linear(dim, dim * 3, bias=bias, device=device, dtype=dtype))
        else:
            for n in separate_names:
                setattr(self, n, operations.Linear(dim, dim, bias=bias, device=device, dtype=dtype))

    def compute_qkv(self, x, prefix=""):
        cfg = self._qkv_configs[prefix]
        if cfg["fused"]:
            return getattr(self, cfg["fused_name"])(x).chunk(3, dim=-1)
        q, k, v = cfg["separate_names"]
        return getattr(self, q)(x), getattr(self, k)(x), getattr(self, v)(x)
