"""GPU parity through the drop-in classes: the calls a KsanaDiT model makes, not the functional wrappers.

``KsanaAttentionOp(...)(q, k, v, **backend_kwargs)`` on [B, L, H, D] tensors for SAGE_ATTN and RADIAL_SAGE_ATTN
(ksana/operations/attention/attention_op.py:72-91, backends/radial_sage_attn/radial_sage_attn.py:78-176), and a
module built with ``QKVProjectionMixin`` + the FP8 Linear that loads an un-fused scaled-FP8 state dict through
``remap_state_dict_for_model`` (ksana/operations/fuse_qkv/fuse_qkv.py:153-233).
"""

import numpy as np
import pytest
import torch

from conftest import cosine, max_abs_rel
from oracle import quantizers as Qz
from oracle import radial_mask as R
from oracle import sage as Sg

pytestmark = pytest.mark.gpu

ATT_COS, ATT_MAR = 0.999, 2e-2  # block-output tolerance of the task against the quantised oracle


def _bqkv(B, L, H, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, L, H, 128, generator=g)
    k = torch.randn(B, L, H, 128, generator=g) + 0.5 * torch.randn(B, 1, H, 128, generator=g)
    v = torch.randn(B, L, H, 128, generator=g)
    return tuple(t.to(dtype) for t in (q, k, v))


def _oracle_batch(q, k, v, tile_mask=None):
    qb, kb, vb = (t.to(torch.bfloat16) if t.dtype == torch.float32 else t for t in (q, k, v))  # sage_attn.py:67-74
    return torch.stack([Sg.sage_attention(qb[b], kb[b], vb[b], tile_mask=tile_mask).float() for b in range(q.shape[0])])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_attention_op_sage_backend_batched(dtype):
    from ksanadit_b200 import _lib, attention
    from ksanadit_b200.config import KsanaAttentionBackend, KsanaAttentionConfig
    op = attention.KsanaAttentionOp(3, 128, attention_config=KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN))
    q, k, v = _bqkv(2, 333, 3, seed=21, dtype=dtype)
    out = op(q.cuda(), k.cuda(), v.cuda(), k_lens=torch.tensor([333, 333]), some_unknown_kwarg=1)
    _lib.assert_device_ok()
    assert out.shape == q.shape and out.dtype == dtype and op.backend_type == KsanaAttentionBackend.SAGE_ATTN
    ref = _oracle_batch(q, k, v)
    assert cosine(out.cpu().float(), ref) >= ATT_COS and max_abs_rel(out.cpu().float(), ref) <= ATT_MAR


def _kernel_mask(seq_len, video, frames, bs, decay):
    """The reference's mask (oracle restatement of MaskMap) padded to the kernel's block counts: blocks the
    floor-divided mask does not cover (a ragged tail) are dense."""
    m = R.radial_log_mask(seq_len, video, frames, bs, decay)
    nq = (seq_len + 127) // 128
    full = np.ones((nq * (128 // bs), nq * (128 // bs)), dtype=bool)
    full[: m.shape[0], : m.shape[1]] = m
    return R.expand_to_q128_k64(full, bs)


@pytest.mark.parametrize("frames,lh,lw,extra,bs", [
    (9, 16, 32, 0, 128),     # 9 frames x 128 tokens: tiles line up with frames
    (21, 16, 16, 0, 128),    # 21 frames x 64 tokens = 1344 tokens: not a multiple of 128
    (9, 16, 32, 100, 128),   # 100 tokens past the video: seq_len > video tokens, ragged tail
    (10, 16, 16, 0, 64),     # 64-token mask blocks merged pairwise into the kernel's 128-row Q blocks
])
def test_attention_op_radial_backend_matches_same_mask_oracle(frames, lh, lw, extra, bs):
    from ksanadit_b200 import _lib, attention
    from ksanadit_b200.config import KsanaRadialSageAttentionConfig
    cfg = KsanaRadialSageAttentionConfig(dense_blocks_num=1, dense_attn_steps=2, decay_factor=0.2, block_size=bs)
    op = attention.KsanaAttentionOp(2, 128, attention_config=cfg)
    video = frames * (lh // 2) * (lw // 2)
    L = video + extra
    q, k, v = _bqkv(2, L, 2, seed=frames + extra, dtype=torch.bfloat16)
    kw = dict(k_lens=torch.tensor([video, video]), latent_shape=[2, 16, frames, lh, lw])
    sparse = op(q.cuda(), k.cuda(), v.cuda(), step_iter=5, block_id=3, **kw)
    _lib.assert_device_ok()
    assert sparse.shape == q.shape  # the reference keeps the full length (its token slice is a no-op on NHD)
    mask = _kernel_mask(L, video, frames, bs, 0.2)
    assert not mask.all(), "the case must drop some tiles"
    ref = _oracle_batch(q, k, v, torch.from_numpy(mask))
    assert cosine(sparse.cpu().float(), ref) >= ATT_COS and max_abs_rel(sparse.cpu().float(), ref) <= ATT_MAR
    # dense switch: early steps, early blocks and dense_only all take the dense kernel
    dense_ref = _oracle_batch(q[:1], k[:1], v[:1])
    for extra_kw in (dict(step_iter=1, block_id=3), dict(step_iter=5, block_id=0), dict(step_iter=5, block_id=3, dense_only=True)):
        d = op(q[:1].cuda(), k[:1].cuda(), v[:1].cuda(), **extra_kw, **kw)
        assert cosine(d.cpu().float(), dense_ref) >= ATT_COS and max_abs_rel(d.cpu().float(), dense_ref) <= ATT_MAR
    assert cosine(sparse[:1].cpu().float(), dense_ref) < 0.99999  # and the sparse path really differs


def test_radial_backend_rejects_what_the_reference_rejects():
    from ksanadit_b200 import attention
    from ksanadit_b200.config import KsanaRadialSageAttentionConfig
    op = attention.KsanaAttentionOp(1, 128, attention_config=KsanaRadialSageAttentionConfig())
    q = torch.zeros(1, 256, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):  # k_lens differ
        op(q, q, q, k_lens=torch.tensor([256, 128]), latent_shape=[1, 16, 2, 16, 32], step_iter=1, block_id=1)
    with pytest.raises(ValueError):  # latent height not a multiple of block_size / 8
        op(q, q, q, k_lens=torch.tensor([256]), latent_shape=[1, 16, 2, 12, 32], step_iter=1, block_id=1)


def test_tile_list_shape_checks_raise_before_launch():
    from ksanadit_b200 import _lib, ops
    q, k, v = (t[0] for t in _bqkv(1, 300, 1, seed=2, dtype=torch.bfloat16))
    pp = Sg.sage_prepass(q, k, v)
    dev = {n: pp[n].cuda() for n in ("q8", "qs", "k8", "ks", "vt8", "vs")}
    offs = torch.zeros(3, dtype=torch.int32, device="cuda")  # needs ceil(300 / 128) + 1 = 4 offsets
    ents = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.KsanaB200Error):
        ops.sage_attn_core(dev["q8"], dev["qs"], dev["k8"], dev["ks"], dev["vt8"], dev["vs"], 300, 300, tile_offsets=offs, tile_entries=ents)
    with pytest.raises(_lib.KsanaB200Error):
        ops.sage_attn_core(dev["q8"], dev["qs"], dev["k8"], dev["ks"], dev["vt8"], dev["vs"], 300, 300,
                           tile_order=torch.zeros(2, dtype=torch.int32, device="cuda"))


def _toy_wan_model(dim, operations):
    """The smallest model shaped like WanModel's projections (wan_model.py:94-118): blocks.N.self_attn.{qkv | q,k,v} + o."""
    from ksanadit_b200.fuse_qkv import QKVProjectionMixin

    class SelfAttention(torch.nn.Module, QKVProjectionMixin):
        def __init__(self):
            super().__init__()
            self._setup_qkv_projection(dim, operations, dtype=torch.bfloat16)
            self.o = operations.Linear(dim, dim, dtype=torch.bfloat16)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = SelfAttention()

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = torch.nn.ModuleList([Block()])

    return Model()


def test_fused_qkv_module_loads_unfused_scaled_fp8_checkpoint():
    from ksanadit_b200 import fuse_qkv, linear
    from oracle import dit_ops as D
    dim = 256
    g = torch.Generator().manual_seed(5)

    class Ops:
        Linear = linear.b200_fp8_ops(scale_input=False)

    model = _toy_wan_model(dim, Ops)
    attn = model.blocks[0].self_attn
    assert attn.qkv_fused and attn.qkv.weight.shape == (3 * dim, dim)
    # a checkpoint as KsanaDiT's scaled-FP8 loaders see it: separate q / k / v, per-tensor scalar scales that differ
    sd, ws = {}, {}
    for i, n in enumerate(("q", "k", "v", "o")):
        w = torch.randn(dim, dim, generator=g) * 0.02 * (i + 1)
        s = w.abs().max() / 448.0
        ws[n] = ((w / s).to(torch.float8_e4m3fn), s, torch.randn(dim, generator=g).to(torch.bfloat16))
        pre = f"blocks.0.self_attn.{n}"
        sd[pre + ".weight"], sd[pre + ".scale_weight"], sd[pre + ".bias"] = ws[n]
    sd = fuse_qkv.remap_state_dict_for_model(model, sd, "wan2.2")
    assert "blocks.0.self_attn.qkv.weight" in sd and "blocks.0.self_attn.q.weight" not in sd
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected
    model = model.cuda()
    x = D.make_activations(200, dim, seed=1)
    xq, sx = Qz.act_quant_fp8_rowwise(x)
    q, k, v = attn.compute_qkv(x.cuda()[None])
    for got, n in ((q, "q"), (k, "k"), (v, "v")):
        wq, s, b = ws[n]
        ref = Qz.fp8_linear_emulated(x, wq, s, b, out_dtype=torch.float32, s_x=sx, xq=xq)
        assert got.shape == (1, 200, dim)
        assert cosine(got[0].cpu().float(), ref) >= 0.9999 and max_abs_rel(got[0].cpu().float(), ref) <= 1e-2
    wq, s, b = ws["o"]
    o = attn.o(x.cuda())
    ref = Qz.fp8_linear_emulated(x, wq, s, b, out_dtype=torch.float32, s_x=sx, xq=xq)
    assert cosine(o.cpu().float(), ref) >= 0.9999 and max_abs_rel(o.cpu().float(), ref) <= 1e-2
