"""Runs KsanaDiT's own block modules through the fused B200 kernel sequence, on the modules' own parameters.

``install(fused_blocks=True)`` replaces ``WanAttentionBlock.forward`` (ksana/models/wan/wan_model.py:325-393) by
``fused_wan_forward`` below, and ``QwenImageTransformerBlock.forward`` (ksana/models/qwen/transformer.py:196-241) by
``fused_qwen_forward`` in the same way.  A block built through the B200 operator registry (FP8 Linears of this package, fused
QKV projection, a Sage attention backend, 128-wide heads, RMSNorm on q / k) is *adopted*: a ``B200WanBlock`` is
created around the block's existing sub-modules -- ``self_attn.qkv / o / norm_q / norm_k``, ``cross_attn.q / k / v / o /
norm_q / norm_k``, ``norm3``, ``ffn[0]``, ``ffn[2]``, ``modulation`` are the same objects, nothing is copied and the
state dict of the model is unchanged -- and the call runs adaLN+quant, the QKV GEMM, RMSNorm+RoPE, the Sage
quantisers, attention, the gated-residual and GELU GEMM epilogues instead of the eager LayerNorm / addcmul /
RMSNorm / fp64 RoPE / GELU passes between the operator calls.  Any block or call that does not qualify (other Linear
classes, separate q / k / v, FETA, CPU tensors, a modulation layout the fused path does not take) goes through the
block's original forward.
"""

from __future__ import annotations

import torch

from . import attention
from .config import backend_value
from .linear import B200Fp8Linear
from .qwen_block import B200QwenBlock
from .wan_block import HEAD, B200WanBlock

_ADOPTED = "_ksana_b200_adopted"
SAGE_BACKENDS = ("sage_attention", "radial_sage_attention")


class AdoptedWanBlock(B200WanBlock):
    """A ``B200WanBlock`` whose sub-modules are those of an existing Wan block module (no new parameters)."""

    def __init__(self, block):
        torch.nn.Module.__init__(self)
        sa, ca = block.self_attn, block.cross_attn
        self.dim, self.ffn_dim, self.num_heads = block.dim, block.ffn_dim, block.num_heads
        self.block_id, self.eps = block.block_id, block.eps
        self.dtype = block.modulation.dtype
        self.self_attn, self.cross_attn = sa, ca
        self.cross_attn_norm = bool(block.cross_attn_norm)
        self.norm3 = block.norm3
        self.ffn = block.ffn
        self.modulation = block.modulation
        self.tile_lists = None
        self.cache_context = False
        self.peer_exchange = None
        self._ones = None
        self._ctx_cache = None
        cfg = getattr(sa.attention, "attention_config", None)
        self.attention_config = cfg
        self._radial = None
        if cfg is not None and backend_value(cfg.backend) == "radial_sage_attention":
            self._radial = attention.B200RadialSageAttentionImpl(attention_config=cfg, num_heads=self.num_heads, head_size=HEAD, causal=False,
                                                                 softmax_scale=None)


def why_not_adoptable(block) -> str | None:
    """None when the fused sequence can take this block module over, else the reason."""
    sa, ca = getattr(block, "self_attn", None), getattr(block, "cross_attn", None)
    if sa is None or ca is None or not hasattr(block, "modulation") or not hasattr(block, "ffn"):
        return "not a Wan attention block"
    if not hasattr(sa, "qkv"):
        return "q / k / v are separate Linears (build the model with the B200 fusion switch installed)"
    linears = [sa.qkv, sa.o, ca.q, ca.k, ca.v, ca.o, block.ffn[0], block.ffn[2]]
    if not all(isinstance(m, B200Fp8Linear) for m in linears):
        return "a Linear of the block is not the B200 FP8 Linear"
    if block.dim != block.num_heads * HEAD:
        return f"head size {block.dim // block.num_heads} (only {HEAD})"
    for n in (sa.norm_q, sa.norm_k, ca.norm_q, ca.norm_k):
        w = getattr(n, "weight", None)
        if w is None or w.dtype != torch.float32 or w.numel() != block.dim:
            return "q / k RMSNorm without an fp32 weight over all channels"
    if block.cross_attn_norm and getattr(block.norm3, "weight", None) is None:
        return "norm3 without affine parameters"
    if block.modulation.dtype not in (torch.bfloat16, torch.float16):
        return f"modulation in {block.modulation.dtype}"
    cfg = getattr(getattr(sa, "attention", None), "attention_config", None)
    if cfg is None or backend_value(cfg.backend) not in SAGE_BACKENDS:
        return "the block's attention backend is not a Sage backend"
    if hasattr(sa, "proj_l"):
        return "sparse-linear attention projection present"
    return None


def adopt(block):
    """The cached ``AdoptedWanBlock`` of a block module, or None when it does not qualify."""
    cached = block.__dict__.get(_ADOPTED)
    if cached is None:
        cached = (AdoptedWanBlock(block),) if why_not_adoptable(block) is None else (None,)
        block.__dict__[_ADOPTED] = cached  # in the instance dict, outside the module tree and the state dict
    return cached[0]


def _radial_lists(ab: AdoptedWanBlock, x, seq_lens, step_iter, latent_shape):
    """Tile lists for this call, or None for dense attention -- RadialSageAttentionImpl.forward's switch
    (radial_sage_attn.py:92-100) with the block's own block_id."""
    r = ab._radial
    if r is None:
        return None
    if step_iter is None or step_iter < r.dense_attn_steps or ab.block_id < r.dense_blocks_num:
        return None
    if not bool((seq_lens == seq_lens[0]).all().item()):
        raise ValueError("k_lens must be the same for all tokens")
    _, _, num_frame, l_h, l_w = latent_shape
    if l_h % (r.block_size // 8) != 0 or l_w % (r.block_size // 8) != 0:
        raise ValueError(f"output's width and height must be divisible by block size {r.block_size}")
    from . import distribute
    total = x.shape[1] * distribute.get_world_size()
    return r.tile_lists_for(total, int(seq_lens[0].item()), int(num_frame), x.device)


def make_fused_wan_forward(original_forward):
    def fused_wan_forward(self, x, e, seq_lens, grid_sizes, freqs, context, context_lens, step_iter=None, latent_shape=None,
                          rope_func="default", feta_enabled=False, feta_weight=2.0, num_frames=1):
        ab = adopt(self)
        takes = (ab is not None and not feta_enabled and x.is_cuda and x.dtype == ab.dtype and e.ndim == 4 and context is not None
                 and not torch.is_grad_enabled())
        if not takes:
            return original_forward(self, x, e, seq_lens, grid_sizes, freqs, context, context_lens, step_iter=step_iter,
                                    latent_shape=latent_shape, rope_func=rope_func, feta_enabled=feta_enabled, feta_weight=feta_weight,
                                    num_frames=num_frames)
        ab.tile_lists = _radial_lists(ab, x, seq_lens, step_iter, latent_shape)
        return ab(x, e, grid_sizes=grid_sizes, context=context, rope_func=rope_func)

    fused_wan_forward.__wrapped__ = original_forward
    return fused_wan_forward


# ----------------------------------------------------------------------------- Qwen-Image dual-stream block

_QWEN_NORMS = ("norm_q", "norm_k", "norm_added_q", "norm_added_k")


class AdoptedQwenBlock(B200QwenBlock):
    """A ``B200QwenBlock`` whose sub-modules are those of an existing QwenImageTransformerBlock module."""

    def __init__(self, block):
        torch.nn.Module.__init__(self)
        self.zero_cond_t = bool(getattr(block, "zero_cond_t", False))
        self.dim, self.num_heads = block.dim, block.num_attention_heads
        self.eps = float(getattr(block.img_norm1, "eps", 1e-6))
        self.img_mod, self.txt_mod, self.attn = block.img_mod, block.txt_mod, block.attn
        self.img_mlp, self.txt_mlp = block.img_mlp, block.txt_mlp
        self.dtype = block.img_mod[1].compute_dtype
        self.ffn_dim = block.img_mlp.net[0].proj.out_features
        self._mod_fused = None
        self._norm_cache = {}

    def _norm_weight(self, name):
        # the reference keeps these weights in the run dtype; the kernel takes fp32 (one converted copy per weight version)
        w = getattr(self.attn, name).weight
        hit = self._norm_cache.get(name)
        if hit is None or hit[0] != (w.data_ptr(), w._version):
            hit = ((w.data_ptr(), w._version), w.detach().float().contiguous())
            self._norm_cache[name] = hit
        return hit[1]


def why_not_adoptable_qwen(block) -> str | None:
    a = getattr(block, "attn", None)
    if a is None or not hasattr(block, "img_mod") or not hasattr(block, "txt_mlp"):
        return "not a Qwen-Image transformer block"
    if not hasattr(a, "to_qkv") or not hasattr(a, "add_qkv_proj"):
        return "q / k / v are separate Linears (build the model with the B200 fusion switch installed)"
    linears = [block.img_mod[1], block.txt_mod[1], a.to_qkv, a.add_qkv_proj, a.to_out[0], a.to_add_out,
               block.img_mlp.net[0].proj, block.img_mlp.net[2], block.txt_mlp.net[0].proj, block.txt_mlp.net[2]]
    if not all(isinstance(m, B200Fp8Linear) for m in linears):
        return "a Linear of the block is not the B200 FP8 Linear"
    if block.attention_head_dim != HEAD or block.dim != block.num_attention_heads * HEAD:
        return f"head size {block.attention_head_dim} (only {HEAD})"
    for n in _QWEN_NORMS:
        w = getattr(getattr(a, n), "weight", None)
        if w is None or w.numel() != HEAD:
            return "q / k RMSNorm without a per-head weight"
    cfg = getattr(getattr(a, "attention", None), "attention_config", None)
    if cfg is None or backend_value(cfg.backend) != "sage_attention":
        return "the block's attention backend is not the Sage backend"
    return None


def adopt_qwen(block):
    cached = block.__dict__.get(_ADOPTED)
    if cached is None:
        cached = (AdoptedQwenBlock(block),) if why_not_adoptable_qwen(block) is None else (None,)
        block.__dict__[_ADOPTED] = cached
    return cached[0]


def make_fused_qwen_forward(original_forward):
    def fused_qwen_forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None, modulate_index=None):
        ab = adopt_qwen(self)
        takes = (ab is not None and hidden_states.is_cuda and hidden_states.dtype == ab.dtype and hidden_states.shape[0] == 1
                 and image_rotary_emb is not None and not torch.is_grad_enabled()
                 and (modulate_index is not None) == ab.zero_cond_t)
        if not takes:
            return original_forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=image_rotary_emb,
                                    modulate_index=modulate_index)
        return ab(hidden_states, encoder_hidden_states, temb, image_rotary_emb=image_rotary_emb, modulate_index=modulate_index)

    fused_qwen_forward.__wrapped__ = original_forward
    return fused_qwen_forward
