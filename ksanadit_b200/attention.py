"""Attention backends for KsanaDiT's attention-backend registry, running the B200 Sage-style kernels.

Mirrors ``KsanaAttentionBackendImpl`` (ksana/operations/attention/backends/base.py:76-128),
``SageAttentionImpl`` (backends/sage_attn.py:30-84), ``RadialSageAttentionImpl``
(backends/radial_sage_attn/radial_sage_attn.py:32-176) and ``KsanaAttentionOp``
(ksana/operations/attention/attention_op.py:24-91): same constructor arguments, ``type()`` /
``supports()`` / ``forward(query, key, value, **kwargs)`` on [B, L, H, D] tensors, unknown keyword
arguments tolerated.  There is no substitution of another backend: if the CUDA library cannot run the
request, ``supports`` is false and construction raises.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections import OrderedDict

import numpy as np
import torch

from . import _lib, ops, radial_mask
from .config import KsanaAttentionBackend, KsanaAttentionConfig, KsanaRadialSageAttentionConfig, backend_value

HEAD_SIZE = 128


class KsanaAttentionBackendImpl(ABC):
    """Same abstract surface as KsanaDiT's class of this name (base.py:76-128)."""

    @abstractmethod
    def __init__(self, attention_config, num_heads, head_size, causal, softmax_scale, num_kv_heads=None, **extra_impl_args):
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def type():  # noqa: A003
        raise NotImplementedError

    @staticmethod
    @abstractmethod
    def supports(**kwargs) -> bool:
        raise NotImplementedError

    def check_config(self):
        if backend_value(self.attention_config.backend) != backend_value(self.type()):
            raise ValueError(f"Attention config {self.attention_config.backend} does not match implementation type {self.type()}")

    def preprocess_qkv(self, qkv):
        return qkv

    def postprocess_output(self, output):
        return output

    @abstractmethod
    def forward(self, query, key, value, **kwargs):
        raise NotImplementedError


def _kernel_supports(head_size=None, dtype=None, **_) -> bool:
    if head_size is not None and head_size != HEAD_SIZE:
        return False
    if dtype is not None and dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return False
    return torch.cuda.is_available()


def _run_sage(query, key, value, tile_lists=None):
    """[B, L, H, D] in, [B, Lq, H, D] out; one kernel sequence per batch element."""
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
        raise ValueError("attention expects tensors shaped [B, L, H, D]")
    if not query.is_cuda:
        raise _lib.KsanaB200Error("the B200 attention backend needs CUDA tensors (no CPU path exists)")
    if query.shape[-1] != HEAD_SIZE:
        raise _lib.KsanaB200Error(f"head size {query.shape[-1]} is not supported (only {HEAD_SIZE})")
    if key.shape[2] != query.shape[2]:
        raise _lib.KsanaB200Error("grouped-query attention (num_kv_heads != num_heads) is not supported")
    orig = query.dtype
    if orig not in (torch.bfloat16, torch.float16):  # sage_attn.py:67-74 casts other dtypes to bf16
        query, key, value = (t.to(torch.bfloat16) for t in (query, key, value))
    B, Lq, H, D = query.shape
    out = torch.empty(B, Lq, H, D, dtype=query.dtype, device=query.device)
    offs, ents, order = tile_lists if tile_lists is not None else (None, None, None)
    for b in range(B):
        ops.sage_attention(query[b], key[b], value[b], tile_offsets=offs, tile_entries=ents, out=out[b], tile_order=order)
    return out if out.dtype == orig else out.to(orig)


class B200SageAttentionImpl(KsanaAttentionBackendImpl):
    """SAGE_ATTN: K smoothing, INT8 Q.K^T, FP8 P.V on tcgen05.  Like the reference's Sage backend it uses
    head_size**-0.5 and ignores ``softmax_scale`` / ``k_lens`` (sage_attn.py:75-81)."""

    @staticmethod
    def type():  # noqa: A003
        return KsanaAttentionBackend.SAGE_ATTN

    @staticmethod
    def supports(**kwargs) -> bool:
        return _kernel_supports(**kwargs)

    def __init__(self, attention_config, num_heads, head_size, causal, softmax_scale, num_kv_heads=None, **extra_impl_args):
        if causal:
            raise ValueError("the B200 Sage backend does not support causal attention")
        if head_size != HEAD_SIZE:
            raise _lib.KsanaB200Error(f"head size {head_size} is not supported (only {HEAD_SIZE})")
        _lib.load()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.num_heads = num_heads
        self.attention_config = attention_config
        self.check_config()

    def forward(self, query, key, value, **kwargs):
        return _run_sage(query, key, value)


class B200RadialSageAttentionImpl(KsanaAttentionBackendImpl):
    """RADIAL_SAGE_ATTN: dense for the first steps / blocks, else the same kernel walking radial tile lists."""

    _global_cache: "OrderedDict" = OrderedDict()
    _max_cache_size = 16  # FIFO, as in the reference (radial_sage_attn.py:33-34,162-166)

    @staticmethod
    def type():  # noqa: A003
        return KsanaAttentionBackend.RADIAL_SAGE_ATTN

    @staticmethod
    def supports(**kwargs) -> bool:
        return _kernel_supports(**kwargs)

    def __init__(self, attention_config, num_heads, head_size, causal, softmax_scale, num_kv_heads=None, **extra_impl_args):
        if causal:
            raise ValueError("RadialSageAttention backend does not support causal attention")
        for f in ("block_size", "decay_factor", "dense_blocks_num", "dense_attn_steps"):
            if not hasattr(attention_config, f):
                raise ValueError("KsanaRadialSageAttentionConfig must be provided")
        if head_size != HEAD_SIZE:
            raise _lib.KsanaB200Error(f"head size {head_size} is not supported (only {HEAD_SIZE})")
        _lib.load()
        self.attention_config = attention_config
        self.block_size = attention_config.block_size
        self.decay_factor = attention_config.decay_factor
        self.dense_blocks_num = attention_config.dense_blocks_num
        self.dense_attn_steps = attention_config.dense_attn_steps
        self.num_heads = num_heads
        self.check_config()

    def forward(self, query, key, value, *, dense_only=False, k_lens=None, step_iter=-1, block_id=-1, latent_shape=None, **kwargs):
        if dense_only or step_iter < self.dense_attn_steps or block_id < self.dense_blocks_num:
            return _run_sage(query, key, value)
        if k_lens is None:
            raise ValueError("k_lens is required for radial attention")
        if not bool((k_lens == k_lens[0]).all().item()):
            raise ValueError("k_lens must be the same for all tokens")
        video_tokens = int(k_lens[0].item())
        _, _, num_frame, l_h, l_w = latent_shape
        if l_h % (self.block_size // 8) != 0 or l_w % (self.block_size // 8) != 0:
            raise ValueError(f"output's width and height must be divisible by block size {self.block_size}")
        # The reference builds the mask for query.shape[1] tokens and hands the whole sequence to its kernel (its
        # `[:, :, :video_token_num]` slice acts on the head axis of an NHD tensor, radial_sage_attn.py:170-176):
        # the lists below cover exactly the length the kernel gets, and the output keeps the input's shape.
        if key.shape[1] != query.shape[1]:
            raise ValueError("radial attention is self-attention: key and query lengths must match")
        lists = self.tile_lists_for(query.shape[1], video_tokens, int(num_frame), query.device)
        return _run_sage(query, key, value, lists)

    def tile_lists_for(self, seq_len, video_tokens, num_frame, device):
        """(offsets [nq + 1], entries, order [nq]) device tensors for a sequence of ``seq_len`` tokens, nq = ceil(seq_len / 128).

        ``MaskMap`` yields seq_len // block_size rows; a ragged last block (seq_len not a multiple of 128, e.g. 21
        frames of 64 tokens) is kept dense in both directions, like every row and column past the video tokens."""
        key = (seq_len, self.block_size, self.decay_factor, video_tokens, num_frame, str(device))
        cache = B200RadialSageAttentionImpl._global_cache
        if key not in cache:
            bs = self.block_size
            if bs not in (64, 128):
                raise ValueError(f"block_size must be 64 or 128, got {bs}")
            m = radial_mask.build_radial_tile_mask(seq_len, video_tokens, num_frame, bs, self.decay_factor)
            nq = (seq_len + 127) // 128
            full = np.ones((nq * (128 // bs), nq * (128 // bs)), dtype=bool)
            full[: m.shape[0], : m.shape[1]] = m
            m = radial_mask.expand_to_kernel_granularity(full, bs)
            offs, ents = radial_mask.compact_tile_lists(m)
            order = radial_mask.longest_first_order(offs)
            # what the kernel indexes with: nq + 1 offsets, nq order entries, KV tile numbers below ceil(seq_len / 128)
            if offs.size != nq + 1 or order.size != nq or (ents.size and int((ents >> 2).max()) >= nq) or int(offs[-1]) != ents.size:
                raise _lib.KsanaB200Error("radial tile lists do not match the kernel's block counts")
            if ents.size == 0:
                ents = np.zeros(1, dtype=np.int32)  # keep a valid pointer for an all-empty mask
            if len(cache) >= self._max_cache_size:
                cache.popitem(last=False)
            cache[key] = (torch.from_numpy(offs).to(device), torch.from_numpy(ents).to(device), torch.from_numpy(order).to(device))
        return cache[key]


_BACKENDS = {
    KsanaAttentionBackend.SAGE_ATTN.value: B200SageAttentionImpl,
    KsanaAttentionBackend.RADIAL_SAGE_ATTN.value: B200RadialSageAttentionImpl,
}


def get_attention_backend_impl(attention_config, **kwargs):
    """base.py:51-73 without the silent walk through other backends: the requested one or an error."""
    name = backend_value(attention_config.backend)
    impl = _BACKENDS.get(name)
    if impl is None:
        raise ValueError(f"attn_backend:{name} is not in supported_list:{sorted(_BACKENDS)}")
    if not impl.supports(**kwargs):
        raise RuntimeError(f"attention backend {name} cannot run {kwargs} on this machine (no other backend is substituted)")
    return impl


class KsanaAttentionOp(torch.nn.Module):
    """Same module surface as KsanaDiT's KsanaAttentionOp (attention_op.py:24-91)."""

    def __init__(self, num_heads, head_size, *, num_kv_heads=None, softmax_scale=None, causal=False, attention_config=None):
        super().__init__()
        if attention_config is None:
            raise ValueError("attention_config should not be None")
        self.num_heads = num_heads
        self.head_size = head_size
        self.num_kv_heads = num_kv_heads or num_heads
        self.softmax_scale = softmax_scale if softmax_scale is not None else head_size ** -0.5
        self.causal = causal
        self.attention_config = attention_config
        self._attn_impl = None
        self._attn_impl_dtype = None

    @property
    def backend_type(self):
        return self._attn_impl.type() if self._attn_impl else None

    def _ensure_impl(self, dtype):
        if self._attn_impl is not None and dtype == self._attn_impl_dtype:
            return
        impl = get_attention_backend_impl(self.attention_config, head_size=self.head_size, dtype=dtype)
        self._attn_impl = impl(attention_config=self.attention_config, num_heads=self.num_heads, head_size=self.head_size,
                               causal=self.causal, softmax_scale=self.softmax_scale, num_kv_heads=self.num_kv_heads)
        self._attn_impl_dtype = dtype

    @torch.compiler.disable
    def forward(self, query, key, value, **backend_kwargs):
        if query.dim() != 4 or key.dim() != 4 or value.dim() != 4:
            raise ValueError("LocalAttentionOp expects tensors shaped [B, L, H, D].")
        self._ensure_impl(query.dtype)
        return self._attn_impl.forward(query, key, value, **backend_kwargs)


def pick_attn_op(attention_config):
    """ksana/operations/attention/pick_attn.py:22-23."""
    from functools import partial
    return partial(KsanaAttentionOp, attention_config=attention_config)


_ = (KsanaAttentionConfig, KsanaRadialSageAttentionConfig)
