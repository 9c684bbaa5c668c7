"""Registers the B200 implementations into a running KsanaDiT process, without editing KsanaDiT.

Hooks (all are module-level names KsanaDiT looks up at call time):

* attention-backend registry: ``get_backend_mapping()`` builds a dict once
  (ksana/operations/attention/backends/base.py:24-48); the entries for ``SAGE_ATTN`` and
  ``RADIAL_SAGE_ATTN`` are replaced, so ``KsanaAttentionConfig(backend=SAGE_ATTN)`` keeps working;
* quantized-linear selection: ``build_ops`` calls the name ``pick_linear`` imported into
  ksana/operations/ops.py:18 -> replaced by a wrapper that returns the B200 class for FP8 checkpoints and
  defers to KsanaDiT's own function otherwise;
* QKV fusion switch: ``should_use_qkv_fusion`` is looked up as a global of
  ksana/operations/fuse_qkv/fuse_qkv.py at :209 -> replaced; ``remap_qkv_weights`` gains scale handling;
* collectives: ``all_to_all`` as imported by the model modules (wan_model.py:13, qwen/attention.py:27-28);
* with ``fused_blocks=True`` also ``WanAttentionBlock.forward`` (wan_model.py:325-393) and
  ``QwenImageTransformerBlock.forward`` (qwen/transformer.py:196-241): blocks built from the
  operators above run as the fused kernel sequence on their own parameters (``adopt.py``), so the adaLN / RMSNorm /
  RoPE / GELU / gated-residual passes between the operator calls are fused too; other blocks keep their forward.

``uninstall()`` restores everything.
"""

from __future__ import annotations

import importlib

from . import attention, distribute, fuse_qkv, linear

_saved: dict = {}


def _ksana(name):
    try:
        return importlib.import_module(name)
    except Exception as exc:  # KsanaDiT is not importable in this process
        raise RuntimeError(f"KsanaDiT module {name} is not importable: {exc}") from exc


def install(patch_collectives: bool = True, fused_blocks: bool = False) -> None:
    if _saved:
        return
    base = _ksana("ksana.operations.attention.backends.base")
    cfg = _ksana("ksana.config")
    mapping = base.get_backend_mapping()
    _saved["mapping"] = (mapping, dict(mapping))

    def bind(impl, member):
        # the registry is keyed by KsanaDiT's enum members and check_config() compares against type()
        return type(impl.__name__, (impl, base.KsanaAttentionBackendImpl), {"type": staticmethod(lambda: member)})

    mapping[cfg.KsanaAttentionBackend.SAGE_ATTN] = bind(attention.B200SageAttentionImpl, cfg.KsanaAttentionBackend.SAGE_ATTN)
    mapping[cfg.KsanaAttentionBackend.RADIAL_SAGE_ATTN] = bind(attention.B200RadialSageAttentionImpl, cfg.KsanaAttentionBackend.RADIAL_SAGE_ATTN)

    ops_mod = _ksana("ksana.operations.ops")
    ref_pick = ops_mod.pick_linear
    _saved["pick_linear"] = (ops_mod, ref_pick)

    def pick_linear(run_dtype, state_dict, linear_backend, load_device=None):
        fp8_dtype, _ = linear.find_fp8_info(dict(state_dict))
        lb = linear.backend_value(linear_backend)
        if fp8_dtype is not None or lb in ("fp8_gemm", "fp8_gemm_dynamic"):
            return linear.pick_linear(run_dtype, state_dict, linear_backend, load_device)
        return ref_pick(run_dtype, state_dict, linear_backend, load_device)

    ops_mod.pick_linear = pick_linear

    fq = _ksana("ksana.operations.fuse_qkv.fuse_qkv")
    _saved["fuse"] = (fq, fq.should_use_qkv_fusion, fq.remap_qkv_weights)
    fq.should_use_qkv_fusion = fuse_qkv.should_use_qkv_fusion
    fq.remap_qkv_weights = fuse_qkv.remap_qkv_weights

    if patch_collectives:
        mods = []
        for name in ("ksana.models.wan.wan_model", "ksana.models.qwen.attention"):
            try:
                m = _ksana(name)
            except RuntimeError:
                continue
            mods.append((m, m.all_to_all))
            m.all_to_all = distribute.all_to_all
        _saved["a2a"] = mods

    if fused_blocks:
        from . import adopt
        wm = _ksana("ksana.models.wan.wan_model")
        original = wm.WanAttentionBlock.forward
        _saved["wan_forward"] = (wm.WanAttentionBlock, original)
        wm.WanAttentionBlock.forward = adopt.make_fused_wan_forward(original)
        try:
            qt = _ksana("ksana.models.qwen.transformer")
        except RuntimeError:
            qt = None
        if qt is not None:
            q_original = qt.QwenImageTransformerBlock.forward
            _saved["qwen_forward"] = (qt.QwenImageTransformerBlock, q_original)
            qt.QwenImageTransformerBlock.forward = adopt.make_fused_qwen_forward(q_original)


def uninstall() -> None:
    if not _saved:
        return
    mapping, old = _saved["mapping"]
    mapping.clear()
    mapping.update(old)
    mod, fn = _saved["pick_linear"]
    mod.pick_linear = fn
    fq, a, b = _saved["fuse"]
    fq.should_use_qkv_fusion, fq.remap_qkv_weights = a, b
    for m, fn in _saved.get("a2a", []):
        m.all_to_all = fn
    for key in ("wan_forward", "qwen_forward"):
        if key in _saved:
            cls, fn = _saved[key]
            cls.forward = fn
    _saved.clear()
