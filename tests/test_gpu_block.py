"""GPU parity: the fused Wan block (all kernels chained) vs the oracle's block, and the norm/RoPE kernel."""

import os
import sys

import pytest
import torch

from conftest import cosine, max_abs_rel
from oracle import dit_ops as D

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from __graft_entry__ import block_state_dict  # noqa: E402

pytestmark = pytest.mark.gpu

# block-output tolerance stated by the task: cosine >= 0.999 and max-abs-rel <= 2e-2
BLOCK_COS, BLOCK_MAR = 0.999, 2e-2


@pytest.mark.parametrize("L,grid,heads,pos0", [(48, (2, 4, 6), 2, 0), (300, (3, 10, 10), 3, 0), (64, (4, 8, 8), 1, 128), (40, (1, 5, 6), 2, 0)])
def test_rmsnorm_rope_inplace(L, grid, heads, pos0):
    from ksanadit_b200 import ops
    C = heads * 128
    g = torch.Generator().manual_seed(L)
    x = (torch.randn(L, 3 * C, generator=g) * 2).to(torch.bfloat16)
    w = 1 + 0.1 * torch.randn(C, generator=g)
    xs = x[:, C:2 * C]
    n = D.rmsnorm_fp32(xs, w)
    F = grid[0] * grid[1] * grid[2]
    if pos0:
        ref = D.apply_wan_rope(n.view(L, heads, 128), grid, sp_rank=pos0 // L, sp_size=max(2, F // L)).reshape(L, C)
    else:
        ref = D.apply_wan_rope(n.view(L, heads, 128), grid).reshape(L, C)
    xd = x.cuda()
    mean = ops.rmsnorm_rope_inplace(xd[:, C:2 * C], w.cuda(), 1e-6, ops.wan_rope_table(128, 1024), grid, pos0=pos0, want_mean=True)
    out = xd[:, C:2 * C].cpu()
    assert torch.equal(xd[:, :C].cpu(), x[:, :C]) and torch.equal(xd[:, 2 * C:].cpu(), x[:, 2 * C:])  # neighbours untouched
    # fp32 rotation vs the reference's fp64: at most one bf16 ulp on a few elements
    d = (out.float() - ref.float()).abs()
    assert float(d.max()) <= 2 ** -7 * float(ref.float().abs().max())
    assert float((d > 0).float().mean()) < 0.02
    assert (mean.cpu() - out.float().mean(dim=0)).abs().max() < 1e-4
    # no rotation: bit exact against the fp32 RMSNorm
    xd2 = x.cuda()
    ops.rmsnorm_rope_inplace(xd2[:, C:2 * C], w.cuda(), 1e-6)
    assert (xd2[:, C:2 * C].cpu().float() - n.float()).abs().max() <= 2 ** -7 * float(n.float().abs().max())


@pytest.mark.parametrize("dim,ffn,heads,grid,ctx", [(256, 768, 2, (2, 6, 8), 40), (1536, 8960, 12, (1, 30, 52), 512)])
def test_wan_block_matches_oracle(dim, ffn, heads, grid, ctx):
    """Second case is the Wan2.1-1.3B-shaped block of the benchmark's CPU configuration (1560 tokens)."""
    from ksanadit_b200 import _lib
    from ksanadit_b200.wan_block import B200WanBlock
    L = grid[0] * grid[1] * grid[2]
    p = D.make_wan_block_params(dim, ffn, heads, seed=0)
    x = D.make_activations(L, dim, seed=0)[None]
    g = torch.Generator().manual_seed(0)
    e = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16)
    c = torch.randn(1, ctx, dim, generator=g).to(torch.bfloat16)
    ref = D.wan_block_forward(p, x, e, c, grid, linear="fp8", attn="sage").float()
    blk = B200WanBlock(dim, ffn, heads, device="cuda").load_block_state_dict(block_state_dict(p))
    with torch.no_grad():
        out = blk(x.cuda(), e.cuda(), grid_sizes=[grid], context=c.cuda()).float().cpu()
        out2 = blk(x.cuda(), e.cuda(), grid_sizes=[grid], context=c.cuda()).float().cpu()
    _lib.assert_device_ok()
    assert torch.equal(out, out2)  # deterministic
    assert cosine(out, ref) >= BLOCK_COS and max_abs_rel(out, ref) <= BLOCK_MAR
    # the change the block makes to its input (the residual branch) is itself close, not just x + small
    assert cosine(out - x[0].float(), ref - x[0].float()) >= 0.995
    exact = D.wan_block_forward(p, x, e, c, grid, linear="fp32", attn="sdpa").float()
    assert cosine(out, exact) >= BLOCK_COS


def test_wan_block_against_reference_golden_subsample(golden):
    """Config-1 block output of the reference's own modules (fp32 Linear + SDPA), stored as a strided subsample."""
    from ksanadit_b200.wan_block import B200WanBlock
    g1 = golden["wan_block_cfg1"]
    dim, ffn, heads, grid = 1536, 8960, 12, (1, 30, 52)
    p = D.make_wan_block_params(dim, ffn, heads, seed=0)
    x = D.make_activations(1560, dim, seed=0)[None]
    gg = torch.Generator().manual_seed(0)
    e = (torch.randn(1, 1, 6, dim, generator=gg) * 0.1).to(torch.bfloat16)
    c = torch.randn(1, 512, dim, generator=gg).to(torch.bfloat16)
    assert torch.equal(e, g1["e"])
    blk = B200WanBlock(dim, ffn, heads, device="cuda").load_block_state_dict(block_state_dict(p))
    with torch.no_grad():
        out = blk(x.cuda(), e.cuda(), grid_sizes=[grid], context=c.cuda()).cpu()
    sub = out[0, ::97, ::31].float()
    assert cosine(sub, g1["y_sub"].float()) >= BLOCK_COS
    assert abs(float(out.float().abs().mean()) - float(g1["absmean"])) <= 2e-2 * float(g1["absmean"])


def test_linear_module_forward_2d_3d():
    from ksanadit_b200 import linear
    from oracle import quantizers as Qz
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(256, 128, generator=g) * 0.02).to(torch.bfloat16)
    b = (torch.randn(256, generator=g) * 0.02).to(torch.bfloat16)
    lin = linear.B200Fp8Linear.from_float(torch.nn.Linear(128, 256).requires_grad_(False).to(torch.bfloat16).cuda())
    lin.weight.data, lin.scale_weight.data = (t.cuda() for t in Qz.weight_quant_fp8_channelwise(w))
    lin.bias.data = b.cuda()
    lin._w_scale_vec = None
    x = D.make_activations(2 * 33, 128, seed=2).view(2, 33, 128)
    ref = D.LinearParams(w, b).fp8(x)
    out = lin(x.cuda())
    assert out.shape == (2, 33, 256) and out.dtype == torch.bfloat16
    assert max_abs_rel(out.cpu().float(), ref.float()) <= 1e-2
    assert lin(x[0].cuda()).shape == (33, 256)


def _qwen_state_dict(p):
    """Oracle Qwen block parameters -> a state dict with QwenImageTransformerBlock's parameter names."""
    sd = {}
    for a, b in (("img_mod.1", "img_mod"), ("txt_mod.1", "txt_mod"), ("attn.to_q", "to_q"), ("attn.to_k", "to_k"),
                 ("attn.to_v", "to_v"), ("attn.add_q_proj", "add_q_proj"), ("attn.add_k_proj", "add_k_proj"),
                 ("attn.add_v_proj", "add_v_proj"), ("attn.to_out.0", "to_out"), ("attn.to_add_out", "to_add_out"),
                 ("img_mlp.net.0.proj", "img_mlp.0"), ("img_mlp.net.2", "img_mlp.2"),
                 ("txt_mlp.net.0.proj", "txt_mlp.0"), ("txt_mlp.net.2", "txt_mlp.2")):
        sd[a + ".weight"] = p[b].w
        sd[a + ".bias"] = p[b].b
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        sd[f"attn.{nm}.weight"] = p[nm]
    return sd


@pytest.mark.parametrize("dim,ffn,heads,grid,Lt", [(256, 1024, 2, (1, 6, 8), 10), (1024, 4096, 8, (1, 24, 20), 77)])
def test_qwen_block_matches_oracle(dim, ffn, heads, grid, Lt):
    from ksanadit_b200 import _lib
    from ksanadit_b200.qwen_block import B200QwenBlock
    p = D.make_qwen_block_params(dim, ffn, heads, seed=5)
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        p[nm] = p[nm].to(torch.bfloat16)  # the reference keeps these weights in the run dtype
    Li = grid[0] * grid[1] * grid[2]
    g = torch.Generator().manual_seed(9)
    img = D.make_activations(Li, dim, seed=6)
    txt = torch.randn(Lt, dim, generator=g).to(torch.bfloat16)
    temb = torch.randn(dim, generator=g).to(torch.bfloat16)
    ia, ta = D.qwen_rope_angles(grid, Lt)
    i_ref, t_ref = D.qwen_block_forward(p, img, txt, temb, ia, ta, linear="fp8", attn="sage")
    blk = B200QwenBlock(dim, heads, ffn, device="cuda").load_block_state_dict(_qwen_state_dict(p))
    with torch.no_grad():
        t_out, i_out = blk(img[None].cuda(), txt[None].cuda(), temb[None].cuda(), img_grid=grid)
    _lib.assert_device_ok()
    for out, ref in ((i_out[0].cpu().float(), i_ref.float()), (t_out[0].cpu().float(), t_ref.float())):
        assert cosine(out, ref) >= BLOCK_COS and max_abs_rel(out, ref) <= BLOCK_MAR
    i_exact, t_exact = D.qwen_block_forward(p, img, txt, temb, ia, ta, linear="fp32", attn="sdpa")
    assert cosine(i_out[0].cpu().float(), i_exact.float()) >= BLOCK_COS


def test_per_head_rmsnorm_and_qwen_rope():
    from ksanadit_b200 import ops
    heads, grid, Lt = 3, (1, 6, 10), 7
    Li = grid[1] * grid[2]
    g = torch.Generator().manual_seed(4)
    w = (1 + 0.1 * torch.randn(128, generator=g))
    ia, ta = D.qwen_rope_angles(grid, Lt)
    img_tab, txt_tab = ops.qwen_rope_tables(grid, Lt)
    for L, ang, tab, gr, diag in ((Li, ia, img_tab, grid, False), (Lt, ta, txt_tab, (Lt, 1, 1), True)):
        x = (torch.randn(L, heads * 128, generator=g) * 2).to(torch.bfloat16)
        n = D.rmsnorm_heads(x.view(L, heads, 128), w.to(torch.bfloat16))
        ref = D.apply_rope_angles(n, ang).reshape(L, heads * 128)
        xd = x.cuda()
        ops.rmsnorm_rope_inplace(xd, w.to(torch.bfloat16).float().cuda(), 1e-6, tab, gr, per_head=True, diag=diag)
        d = (xd.cpu().float() - ref.float()).abs()
        assert float(d.max()) <= 2 ** -6 * float(ref.float().abs().max())
        assert cosine(xd.cpu(), ref) > 0.99999


def test_comfy_rope_table_matches_reference_formulation(golden):
    """rope_func="comfy" (ksana/utils/rope.py:151-212): the kernel rotates with a table of bf16-rounded cos / sin, like
    the reference's 2x2 matrices held in the activation dtype.  The reference rounds twice per output (product, then
    addcmul), the kernel once, so single outputs may differ by one bf16 ulp."""
    from ksanadit_b200 import ops
    v = golden["comfy_rope"]["bf16"]
    x, grid, ref = v["x"], tuple(int(t) for t in v["grid"]), v["y"]
    L, N, Dh = x.shape
    assert torch.equal(D.apply_comfy_rope(x, grid), ref)  # the oracle restatement is the reference, bit for bit
    xd = x.reshape(L, N * Dh).clone().cuda()
    ones = torch.ones(N * Dh)
    # unit RMSNorm weight on unit-RMS rows would still rescale: rotate rows that are already normalised instead
    n = D.rmsnorm_fp32(x.reshape(L, N * Dh), ones)
    want = D.apply_comfy_rope(n.view(L, N, Dh), grid).reshape(L, N * Dh)
    ops.rmsnorm_rope_inplace(xd, ones.cuda(), 1e-6, ops.comfy_rope_table(Dh, 1024, dtype=torch.bfloat16), grid)
    d = (xd.cpu().float() - want.float()).abs()
    assert float(d.max()) <= 2 ** -7 * float(want.float().abs().max())
    assert float((d > 0).float().mean()) < 0.25
    dflt = D.apply_wan_rope(n.view(L, N, Dh), grid).reshape(L, N * Dh)
    assert float((xd.cpu().float() - want.float()).abs().mean()) < float((dflt.float() - want.float()).abs().mean())


def test_wan_block_with_comfy_rope_matches_oracle():
    from ksanadit_b200 import _lib
    from ksanadit_b200.wan_block import B200WanBlock
    dim, ffn, heads, grid, ctx = 256, 768, 2, (2, 6, 8), 40
    L = grid[0] * grid[1] * grid[2]
    p = D.make_wan_block_params(dim, ffn, heads, seed=0)
    x = D.make_activations(L, dim, seed=0)[None]
    g = torch.Generator().manual_seed(0)
    e = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16)
    c = torch.randn(1, ctx, dim, generator=g).to(torch.bfloat16)
    ref = D.wan_block_forward(p, x, e, c, grid, linear="fp8", attn="sage", rope="comfy").float()
    blk = B200WanBlock(dim, ffn, heads, device="cuda").load_block_state_dict(block_state_dict(p))
    with torch.no_grad():
        out = blk(x.cuda(), e.cuda(), grid_sizes=[grid], context=c.cuda(), rope_func="comfy").float().cpu()
        with pytest.raises(_lib.KsanaB200Error):
            blk(x.cuda(), e.cuda(), grid_sizes=[grid], context=c.cuda(), rope_func="something else")
    _lib.assert_device_ok()
    assert cosine(out, ref) >= BLOCK_COS and max_abs_rel(out, ref) <= BLOCK_MAR


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_qwen_block_zero_cond_t_per_token_modulation(dtype, golden):
    """zero_cond_t blocks (qwen/transformer.py:171-188,206-208): per-token choice between two modulation rows."""
    from ksanadit_b200 import _lib
    from ksanadit_b200.qwen_block import B200QwenBlock
    dim, ffn, heads, grid, Lt = 256, 1024, 2, (1, 6, 8), 10
    p = D.make_qwen_block_params(dim, ffn, heads, seed=5, dtype=dtype)
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        p[nm] = p[nm].to(dtype)
    gz = golden["qwen_block_zero_cond"]
    Li = grid[1] * grid[2]
    g = torch.Generator().manual_seed(9)
    img = D.make_activations(Li, dim, seed=6, dtype=dtype)
    txt = torch.randn(Lt, dim, generator=g).to(dtype)
    temb2, index = gz["temb"].to(dtype), gz["index"]
    ia, ta = D.qwen_rope_angles(grid, Lt)
    i_ref, t_ref = D.qwen_block_forward(p, img, txt, temb2, ia, ta, linear="fp8", attn="sage", modulate_index=index)
    blk = B200QwenBlock(dim, heads, ffn, device="cuda", dtype=dtype, zero_cond_t=True).load_block_state_dict(_qwen_state_dict(p))
    with torch.no_grad():
        t_out, i_out = blk(img[None].cuda(), txt[None].cuda(), temb2.cuda(), img_grid=grid, modulate_index=index[None].cuda())
        with pytest.raises(_lib.KsanaB200Error):
            blk(img[None].cuda(), txt[None].cuda(), temb2.cuda(), img_grid=grid)  # a zero_cond_t block needs the index
    _lib.assert_device_ok()
    for out, ref in ((i_out[0].cpu().float(), i_ref.float()), (t_out[0].cpu().float(), t_ref.float())):
        assert cosine(out, ref) >= BLOCK_COS and max_abs_rel(out, ref) <= BLOCK_MAR
    # every token on row 0 gives a different image stream: the index really selects
    i_all0, _ = D.qwen_block_forward(p, img, txt, temb2, ia, ta, linear="fp8", attn="sage", modulate_index=torch.zeros_like(index))
    assert max_abs_rel(i_out[0].cpu().float(), i_all0.float()) > max_abs_rel(i_out[0].cpu().float(), i_ref.float())
    if dtype == torch.bfloat16:  # the reference's own block output (fp32 Linear + SDPA) on the same inputs
        assert cosine(i_out[0].cpu().float(), gz["img_y"].float()) >= BLOCK_COS


def test_wan_block_cfg_batch_folds_into_rows():
    """Two samples (cond / uncond: own modulation and own text context, same grid) folded into the row dimension give what
    the two samples give one at a time -- every element is computed by the same arithmetic, only the launches differ --
    and both match the oracle (generator.py:356-375: the reference concatenates cond and uncond on the batch axis)."""
    from ksanadit_b200 import _lib, ops
    from ksanadit_b200.wan_block import B200WanBlock
    dim, ffn, heads, grid, ctx = 256, 768, 2, (2, 6, 9), 40
    L = grid[0] * grid[1] * grid[2]  # 108 tokens: a ragged last tile inside every sample
    p = D.make_wan_block_params(dim, ffn, heads, seed=0)
    g = torch.Generator().manual_seed(1)
    x = torch.stack([D.make_activations(L, dim, seed=s) for s in (3, 4)])
    e = (torch.randn(2, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16)
    c = torch.randn(2, ctx, dim, generator=g).to(torch.bfloat16)
    blk = B200WanBlock(dim, ffn, heads, device="cuda").load_block_state_dict(block_state_dict(p))
    with torch.no_grad():
        launches0 = ops.STATS.kernels
        both = blk(x.cuda(), e.cuda(), grid_sizes=[grid, grid], context=c.cuda())
        n_batched = ops.STATS.kernels - launches0
        single = [blk(x[b:b + 1].cuda(), e[b:b + 1].cuda(), grid_sizes=[grid], context=c[b:b + 1].cuda()) for b in range(2)]
        n_single = ops.STATS.kernels - launches0 - n_batched
    _lib.assert_device_ok()
    assert both.shape == (2, L, dim)
    for b in range(2):
        assert torch.equal(both[b], single[b][0]), f"sample {b}: batched and one-at-a-time results differ"
        ref = D.wan_block_forward(p, x[b:b + 1], e[b:b + 1], c[b:b + 1], grid, linear="fp8", attn="sage").float()
        assert cosine(both[b].cpu().float(), ref[0]) >= BLOCK_COS and max_abs_rel(both[b].cpu().float(), ref[0]) <= BLOCK_MAR
    assert n_batched < n_single  # one GEMM and one attention launch per stage for both samples


def test_context_cache_is_keyed_on_the_tensor_object():
    from ksanadit_b200.wan_block import B200WanBlock
    dim, ffn, heads, grid = 256, 768, 2, (1, 6, 8)
    L = 48
    blk = B200WanBlock(dim, ffn, heads, device="cuda", cache_context=True).random_init(3)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, L, dim, generator=g).to(torch.bfloat16).cuda()
    e = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16).cuda()
    c1 = torch.randn(1, 24, dim, generator=g).to(torch.bfloat16).cuda()
    with torch.no_grad():
        y1 = blk(x, e, grid_sizes=[grid], context=c1)
        assert torch.equal(blk(x, e, grid_sizes=[grid], context=c1), y1)  # second call takes the cached K / V
        c2 = torch.randn(1, 24, dim, generator=g).to(torch.bfloat16).cuda()
        addr = c1.data_ptr()
        c1.copy_(c2)  # same storage, new prompt: the version counter moves and the entry is not reused
        assert c1.data_ptr() == addr
        y2 = blk(x, e, grid_sizes=[grid], context=c1)
        fresh = B200WanBlock(dim, ffn, heads, device="cuda").random_init(3)(x, e, grid_sizes=[grid], context=c2)
    assert torch.equal(y2, fresh) and not torch.equal(y2, y1)


class _RefShapedWanBlock(torch.nn.Module):
    """A module with the attribute layout of KsanaDiT's WanAttentionBlock built from the B200 operators (wan_model.py:
    61-133,254-323): what `install(fused_blocks=True)` meets inside a loaded model.  Its forward is never used."""

    def __init__(self, dim, ffn, heads, attention_config):
        super().__init__()
        from ksanadit_b200.linear import B200Fp8Linear

        def rms():
            m = torch.nn.Module()
            m.weight = torch.nn.Parameter(torch.ones(dim, dtype=torch.float32), requires_grad=False)
            return m

        def attn(separate):
            a = torch.nn.Module()
            if separate:
                a.q, a.k, a.v = (B200Fp8Linear(dim, dim) for _ in range(3))
            else:
                a.qkv = B200Fp8Linear(dim, 3 * dim)
            a.o, a.norm_q, a.norm_k = B200Fp8Linear(dim, dim), rms(), rms()
            a.attention = torch.nn.Module()
            a.attention.attention_config = attention_config
            return a

        self.dim, self.ffn_dim, self.num_heads, self.block_id, self.eps, self.cross_attn_norm = dim, ffn, heads, 2, 1e-6, True
        self.self_attn, self.cross_attn = attn(False), attn(True)
        self.norm3 = torch.nn.LayerNorm(dim, 1e-6, elementwise_affine=True, dtype=torch.float32)
        self.ffn = torch.nn.Sequential(B200Fp8Linear(dim, ffn), torch.nn.GELU(approximate="tanh"), B200Fp8Linear(ffn, dim))
        self.modulation = torch.nn.Parameter(torch.zeros(1, 6, dim, dtype=torch.bfloat16), requires_grad=False)


@pytest.mark.parametrize("radial", [False, True])
def test_fused_forward_on_an_adopted_reference_shaped_block(radial):
    """The fused sequence running on a reference-shaped module's own parameters gives what B200WanBlock gives with the same
    weights, for the Sage backend and for the radial one (dense in early steps, tile lists afterwards)."""
    from ksanadit_b200 import _lib, adopt
    from ksanadit_b200.config import KsanaAttentionBackend, KsanaAttentionConfig, KsanaRadialSageAttentionConfig
    from ksanadit_b200.wan_block import B200WanBlock
    dim, ffn, heads = 256, 768, 2
    frames, lh, lw = 9, 16, 32
    grid = (frames, lh // 2, lw // 2)
    L = grid[0] * grid[1] * grid[2]  # 1152 tokens
    cfg = KsanaRadialSageAttentionConfig(dense_blocks_num=1, dense_attn_steps=2, decay_factor=0.2, block_size=128) if radial \
        else KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN)
    ours = B200WanBlock(dim, ffn, heads, block_id=2, device="cuda").random_init(11)
    ref_like = _RefShapedWanBlock(dim, ffn, heads, cfg).cuda()
    sd = {k: v for k, v in ours.state_dict().items()}
    missing, unexpected = ref_like.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    for a, b in ((ref_like.self_attn.qkv, ours.self_attn.qkv), (ref_like.ffn[0], ours.ffn[0])):
        assert torch.equal(a.weight.view(torch.uint8), b.weight.view(torch.uint8)) and torch.equal(a.scale_weight, b.scale_weight)
    assert adopt.why_not_adoptable(ref_like) is None
    fused = adopt.make_fused_wan_forward(lambda *a, **k: (_ for _ in ()).throw(AssertionError("the original forward must not run")))
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, L, dim, generator=g).to(torch.bfloat16).cuda()
    e = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16).cuda()
    c = torch.randn(1, 40, dim, generator=g).to(torch.bfloat16).cuda()
    kw = dict(seq_lens=torch.tensor([L]), grid_sizes=torch.tensor([grid]), freqs=None, context=c, context_lens=None,
              latent_shape=[1, 16, frames, lh, lw])
    with torch.no_grad():
        dense = ours(x, e, grid_sizes=[grid], context=c)
        early = fused(ref_like, x, e, step_iter=0, **kw)
        late = fused(ref_like, x, e, step_iter=5, **kw)
    _lib.assert_device_ok()
    assert torch.equal(early, dense)
    if not radial:
        assert torch.equal(late, dense)
    else:
        impl = adopt.adopt(ref_like)._radial
        ours.tile_lists = impl.tile_lists_for(L, L, frames, x.device)
        with torch.no_grad():
            sparse = ours(x, e, grid_sizes=[grid], context=c)
        assert torch.equal(late, sparse) and not torch.equal(late, dense)
    # a call the fused path does not take goes to the original forward
    with pytest.raises(AssertionError, match="original forward"):
        fused(ref_like, x, e, step_iter=0, feta_enabled=True, **kw)


class _RefShapedQwenBlock(torch.nn.Module):
    """Attribute layout of KsanaDiT's QwenImageTransformerBlock built from the B200 operators (qwen/transformer.py:122-169,
    qwen/attention.py:221-281): per-head RMSNorm weights in the run dtype, `attention.attention_config`, LayerNorms."""

    def __init__(self, dim, heads, ffn, attention_config, zero_cond_t=False):
        super().__init__()
        from ksanadit_b200.linear import B200Fp8Linear
        self.dim, self.num_attention_heads, self.attention_head_dim, self.zero_cond_t = dim, heads, dim // heads, zero_cond_t
        self.img_mod = torch.nn.Sequential(torch.nn.SiLU(), B200Fp8Linear(dim, 6 * dim))
        self.txt_mod = torch.nn.Sequential(torch.nn.SiLU(), B200Fp8Linear(dim, 6 * dim))
        self.img_norm1 = torch.nn.LayerNorm(dim, 1e-6, elementwise_affine=False)
        a = torch.nn.Module()
        a.to_qkv, a.add_qkv_proj = B200Fp8Linear(dim, 3 * dim), B200Fp8Linear(dim, 3 * dim)
        a.to_out = torch.nn.ModuleList([B200Fp8Linear(dim, dim), torch.nn.Dropout(0.0)])
        a.to_add_out = B200Fp8Linear(dim, dim)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            m = torch.nn.Module()
            m.weight = torch.nn.Parameter(torch.ones(128, dtype=torch.bfloat16), requires_grad=False)
            setattr(a, n, m)
        a.attention = torch.nn.Module()
        a.attention.attention_config = attention_config
        self.attn = a
        for s in ("img_mlp", "txt_mlp"):
            mlp, act = torch.nn.Module(), torch.nn.Module()
            act.proj = B200Fp8Linear(dim, ffn)
            mlp.net = torch.nn.ModuleList([act, torch.nn.Identity(), B200Fp8Linear(ffn, dim)])
            setattr(self, s, mlp)


def test_fused_forward_on_an_adopted_reference_shaped_qwen_block():
    """The adopted block takes its rotation tables from the caller's `image_rotary_emb` (complex, one row per token) and
    gives what B200QwenBlock gives from the grid with the same weights; both match the oracle."""
    from ksanadit_b200 import _lib, adopt
    from ksanadit_b200.config import KsanaAttentionBackend, KsanaAttentionConfig
    from ksanadit_b200.qwen_block import B200QwenBlock
    dim, ffn, heads, grid, Lt = 256, 1024, 2, (1, 6, 8), 10
    Li = grid[1] * grid[2]
    p = D.make_qwen_block_params(dim, ffn, heads, seed=5)
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        p[nm] = p[nm].to(torch.bfloat16)
    ours = B200QwenBlock(dim, heads, ffn, device="cuda").load_block_state_dict(_qwen_state_dict(p))
    ref_like = _RefShapedQwenBlock(dim, heads, ffn, KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN)).cuda()
    missing, unexpected = ref_like.load_state_dict(ours.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    assert adopt.why_not_adoptable_qwen(ref_like) is None
    fused = adopt.make_fused_qwen_forward(lambda *a, **k: (_ for _ in ()).throw(AssertionError("the original forward must not run")))
    g = torch.Generator().manual_seed(9)
    img = D.make_activations(Li, dim, seed=6)
    txt = torch.randn(Lt, dim, generator=g).to(torch.bfloat16)
    temb = torch.randn(dim, generator=g).to(torch.bfloat16)
    ia, ta = D.qwen_rope_angles(grid, Lt)  # [L, 64] angles -> the complex per-token rows the reference's rope module returns
    rotary = tuple(torch.polar(torch.ones_like(a_.float()), a_.float()).cuda() for a_ in (ia, ta))
    with torch.no_grad():
        t_grid, i_grid = ours(img[None].cuda(), txt[None].cuda(), temb[None].cuda(), img_grid=grid)
        t_rot, i_rot = fused(ref_like, img[None].cuda(), txt[None].cuda(), temb[None].cuda(), image_rotary_emb=rotary)
    _lib.assert_device_ok()
    i_ref, t_ref = D.qwen_block_forward(p, img, txt, temb, ia, ta, linear="fp8", attn="sage")
    for out, ref in ((i_rot[0].cpu().float(), i_ref.float()), (t_rot[0].cpu().float(), t_ref.float())):
        assert cosine(out, ref) >= BLOCK_COS and max_abs_rel(out, ref) <= BLOCK_MAR
    # same kernels, tables built two ways (fp64 formula vs the caller's fp32 cos / sin): equal up to the table's last bit
    assert cosine(i_rot.cpu().float(), i_grid.cpu().float()) > 0.99999 and cosine(t_rot.cpu().float(), t_grid.cpu().float()) > 0.99999
    with pytest.raises(AssertionError, match="original forward"):  # no rotary embeddings: not a call the fused path takes
        fused(ref_like, img[None].cuda(), txt[None].cuda(), temb[None].cuda())
