"""Generate the golden vectors under tests/golden/ from the reference's own torch code.

Run where the KsanaDiT source tree is importable (default path below, or
``KSANA_REFERENCE=/path/to/KsanaDiT``):

    python tests/golden/make_golden.py

It imports the reference's modules on CPU (five optional third-party imports of
the reference are stubbed, none is on the DiT-block path), runs them on small
seeded inputs, checks the oracle against them and writes ``reference_vectors.pt``.
The tests then compare the oracle (and, on a GPU, the CUDA kernels) with those
vectors without needing the reference tree.
"""

from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("KSANA_REFERENCE", "/root/reference")


def _stub(name, **attrs):
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def install_stubs():
    import yaml

    class _Profiler:
        def __init__(self, *a, **k):
            pass

    class OmegaConf:
        load = staticmethod(lambda p: yaml.safe_load(open(p)))
        to_container = staticmethod(lambda c, **k: c)
        create = staticmethod(lambda c=None: c or {})

        @staticmethod
        def merge(*a):
            out = {}
            for d in a:
                out.update(d or {})
            return out

    _stub("pyinstrument", Profiler=_Profiler)
    _stub("omegaconf", OmegaConf=OmegaConf, DictConfig=dict, ListConfig=list)
    _stub("imageio")
    _stub("ftfy")
    _stub("diffusers")
    _stub("diffusers.configuration_utils", ConfigMixin=type("ConfigMixin", (), {}), register_to_config=lambda f: f)
    _stub("diffusers.models")
    _stub("diffusers.models.modeling_utils", ModelMixin=torch.nn.Module)
    sys.path.insert(0, REF)


def cos(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


def max_abs_rel(a, b):
    return float((a.double() - b.double()).abs().max() / (b.double().abs().max() + 1e-30))


def main():
    install_stubs()
    import ksana  # noqa: F401  (prints and swallows its optional 'ray' import error)
    from ksana.config import KsanaAttentionBackend, KsanaAttentionConfig
    from ksana.models.qwen.attention import QwenEmbedRope
    from ksana.models.qwen.transformer import QwenImageTransformerBlock
    from ksana.models.wan.wan_model import WanAttentionBlock, rope_params
    from ksana.operations.attention.backends.radial_sage_attn.attn_mask import MaskMap
    from ksana.operations.attention.backends.sdpa import SDPAImpl
    from ksana.operations.attention.pick_attn import pick_attn_op
    from ksana.operations.linear.fp8_linear import scaled_fp8_ops
    from ksana.operations.linear.linear import Linear
    from ksana.operations.ops import LayerNorm, Ops, RMSNorm
    from ksana.utils.rope import apply_default_rope

    from oracle import dit_ops as D
    from oracle import quantizers as Qz
    from oracle import radial_mask as R

    SDPAImpl.supports = staticmethod(lambda **_: True)  # reference gates SDPA on CUDA presence (sdpa.py:27-29)
    gold = {}
    torch.manual_seed(0)

    # ---- (1) the reference's per-tensor FP8 Linear (fp8_linear.py:25-73) -----------------
    g = torch.Generator().manual_seed(1)
    cls = scaled_fp8_ops(fp8_matrix_mult=True, scale_input=True, override_dtype=torch.float8_e4m3fn)
    lin = cls(64, 48, bias=True)
    w = torch.randn(48, 64, generator=g) * 0.02
    sw = w.abs().max() / 448.0
    lin.weight = torch.nn.Parameter((w / sw).to(torch.float8_e4m3fn), requires_grad=False)
    lin.bias = torch.nn.Parameter((torch.randn(48, generator=g) * 0.02).to(torch.bfloat16), requires_grad=False)
    lin.scale_weight = torch.nn.Parameter(sw.float(), requires_grad=False)
    x = (torch.randn(2, 24, 64, generator=g) * 2).to(torch.bfloat16)
    si = (x.float().abs().max() / 448.0).float()
    lin.scale_input = torch.nn.Parameter(si, requires_grad=False)
    lin.eval()
    y_ref = lin(x.clone())
    xq = Qz.act_quant_fp8_static(x.reshape(-1, 64), si)
    y_or = Qz.fp8_linear_emulated(x, lin.weight.data, sw.float(), lin.bias.data, xq=xq, s_x=si)
    d = (y_ref.float() - y_or.float()).abs().max().item()
    print(f"[1] per-tensor fp8_linear: max|ref-oracle| = {d:.3e}")
    assert d <= 2e-3
    gold["fp8_pt"] = dict(x=x, wq=lin.weight.data.view(torch.uint8), sw=sw.float(), si=si, bias=lin.bias.data,
                          xq=xq.view(torch.uint8), y=y_ref)
    # unscaled path (clamp then cast)
    lin2 = cls(64, 48, bias=False)
    lin2.weight = torch.nn.Parameter(lin.weight.data.clone(), requires_grad=False)
    lin2.scale_weight = torch.nn.Parameter(sw.float(), requires_grad=False)
    lin2.scale_input = None
    lin2.eval()
    xb = (torch.randn(24, 64, generator=g) * 300).to(torch.bfloat16)
    y2 = lin2(xb.clone())
    xq2 = Qz.act_quant_fp8_static(xb, None)
    y2o = Qz.fp8_linear_emulated(xb, lin2.weight.data, sw.float(), None, xq=xq2, s_x=torch.ones(()))
    d = max_abs_rel(y2o.float(), y2.float())
    print(f"[1b] unscaled fp8_linear: max-abs-rel = {d:.3e}")
    assert d <= 1e-2
    gold["fp8_unscaled"] = dict(x=xb, xq=xq2.view(torch.uint8), y=y2)

    # ---- (2) Wan RoPE (rope.py:62-128) ---------------------------------------------------
    grid = (3, 4, 6)
    L = grid[0] * grid[1] * grid[2]
    dd = 128
    freqs = torch.cat([rope_params(1024, dd - 4 * (dd // 6)), rope_params(1024, 2 * (dd // 6)),
                       rope_params(1024, 2 * (dd // 6))], dim=1)
    xr = torch.randn(1, L, 2, dd, generator=g).to(torch.bfloat16)
    r_ref = apply_default_rope(xr, torch.tensor([grid]), freqs)
    r_or = D.apply_wan_rope(xr[0], grid)
    assert torch.equal(r_ref[0], r_or), "rope sp=1"
    for rank in range(2):
        xs = xr[:, rank * (L // 2):(rank + 1) * (L // 2)]
        a = apply_default_rope(xs, torch.tensor([grid]), freqs, sp_rank=rank, sp_size=2)
        b = D.apply_wan_rope(xs[0], grid, sp_rank=rank, sp_size=2)
        assert torch.equal(a[0], b), "rope sp=2"
    print("[2] Wan RoPE: oracle == reference (bit-exact, sp 1 and 2)")
    gold["rope"] = dict(x=xr[0], grid=torch.tensor(grid), y=r_ref[0])

    # ---- (3) Wan block with the reference modules (wan_model.py:254-393) ------------------
    def ref_wan_block(p, dim, ffn, heads, x, e, ctx, grid):
        ops = Ops()
        ops.register("Linear", Linear)
        ops.register("LayerNorm", LayerNorm)
        ops.register("RMSNorm", RMSNorm)
        ops.register("Attn", pick_attn_op(KsanaAttentionConfig(backend=KsanaAttentionBackend.TORCH_SDPA)))
        st = {"operations": ops, "device": "cpu", "dtype": torch.bfloat16, "rms_dtype": None}
        blk = WanAttentionBlock(dim, ffn, heads, block_id=0, qk_norm=True, cross_attn_norm=True, eps=1e-6,
                                operation_settings=st)
        sd = {"modulation": p["modulation"], "norm3.weight": p["norm3.w"], "norm3.bias": p["norm3.b"]}
        for a, b in (("self_attn", "self"), ("cross_attn", "cross")):
            for nm in "qkvo":
                sd[f"{a}.{nm}.weight"] = p[f"{b}.{nm}"].w
                sd[f"{a}.{nm}.bias"] = p[f"{b}.{nm}"].b
            sd[f"{a}.norm_q.weight"] = p[f"{b}.norm_q"]
            sd[f"{a}.norm_k.weight"] = p[f"{b}.norm_k"]
        for i in (0, 2):
            sd[f"ffn.{i}.weight"] = p[f"ffn.{i}"].w
            sd[f"ffn.{i}.bias"] = p[f"ffn.{i}"].b
        missing, unexpected = blk.load_state_dict(sd, strict=False)
        assert not missing and not unexpected, (missing, unexpected)
        blk.eval()
        with torch.no_grad():
            return blk(x, e, seq_lens=torch.tensor([x.shape[1]]), grid_sizes=torch.tensor([grid]), freqs=freqs,
                       context=ctx, context_lens=None, step_iter=0, latent_shape=[1, 16, grid[0], 8, 8])

    dim, ffn, heads = 256, 512, 2
    p = D.make_wan_block_params(dim, ffn, heads, seed=3)
    xw = D.make_activations(L, dim, seed=4)[None]
    ew = (torch.randn(1, 1, 6, dim, generator=g) * 0.1).to(torch.bfloat16)
    cw = torch.randn(1, 16, dim, generator=g).to(torch.bfloat16)
    yw_ref = ref_wan_block(p, dim, ffn, heads, xw, ew, cw, grid)
    yw_or = D.wan_block_forward(p, xw, ew, cw, grid, linear="fp32", attn="sdpa")
    d = max_abs_rel(yw_or.float(), yw_ref.float())
    print(f"[3] Wan block (fp32 Linear + SDPA): max-abs-rel = {d:.3e}, cos = {cos(yw_or, yw_ref):.6f}")
    assert d <= 1e-2 and cos(yw_or, yw_ref) > 0.9999
    gold["wan_block"] = dict(seed_params=3, seed_x=4, dim=dim, ffn=ffn, heads=heads, grid=torch.tensor(grid), e=ew,
                             ctx=cw, y=yw_ref)

    # config 1 of the benchmark (Wan2.1-1.3B-shaped block, 1560 tokens): timed + stats only
    import time
    dim1, ffn1, heads1, grid1 = 1536, 8960, 12, (1, 30, 52)
    p1 = D.make_wan_block_params(dim1, ffn1, heads1, seed=0)
    x1 = D.make_activations(1560, dim1, seed=0)[None]
    g1 = torch.Generator().manual_seed(0)
    e1 = (torch.randn(1, 1, 6, dim1, generator=g1) * 0.1).to(torch.bfloat16)
    c1 = torch.randn(1, 512, dim1, generator=g1).to(torch.bfloat16)
    t0 = time.time()
    y1_ref = ref_wan_block(p1, dim1, ffn1, heads1, x1, e1, c1, grid1)
    t_ref = time.time() - t0
    y1_or = D.wan_block_forward(p1, x1, e1, c1, grid1, linear="fp32", attn="sdpa")
    d = max_abs_rel(y1_or.float(), y1_ref.float())
    print(f"[3b] config-1 Wan block: ref {t_ref:.2f}s on {torch.get_num_threads()} threads; "
          f"max-abs-rel = {d:.3e}, cos = {cos(y1_or, y1_ref):.6f}")
    assert d <= 1e-2
    gold["wan_block_cfg1"] = dict(y_sub=y1_ref[0, ::97, ::31].clone(), absmean=y1_ref.float().abs().mean(),
                                  seed=0, e=e1, ctx_seed=0)

    # ---- (4) radial tile mask (attn_mask.py) ---------------------------------------------
    import ksana.operations.attention.backends.radial_sage_attn.attn_mask as am
    am.tqdm = lambda it, **k: it
    masks = {}
    for (vt, nf, bs, decay, s) in [(8 * 16 * 16, 8, 128, 0.5, 8 * 256), (12 * 24 * 16, 12, 128, 0.2, 12 * 384 + 256),
                                   (9 * 16 * 24, 9, 64, 0.5, 9 * 384), (21 * 1280, 21, 128, 0.02, 21 * 1280),
                                   (10 * 360, 10, 128, 0.5, 10 * 360 + 77)]:  # last: frames that do not end on tile edges
        mm = MaskMap(video_token_num=vt, num_frame=nf, block_size=bs, device="cpu")
        ref_m = mm.query_log_mask(s, "radial", block_size=bs, decay_factor=decay).numpy()
        or_m = R.radial_log_mask(s, vt, nf, bs, decay)
        assert np.array_equal(ref_m, or_m), (vt, nf, bs, decay)
        masks[f"{vt}_{nf}_{bs}_{decay}_{s}"] = torch.from_numpy(np.packbits(ref_m))
        print(f"[4] radial mask vt={vt} nf={nf} bs={bs} decay={decay}: equal, density {ref_m.mean():.3f}")
    gold["radial_masks"] = masks

    # ---- (5) Qwen-Image dual-stream block (qwen/transformer.py:122-241) ------------------
    qdim, qffn, qheads = 256, 1024, 2
    qp = D.make_qwen_block_params(qdim, qffn, qheads, seed=5)
    ops = Ops()
    for nm, c in (("Linear", Linear), ("LayerNorm", LayerNorm), ("RMSNorm", RMSNorm)):
        ops.register(nm, c)
    ops.register("Attn", pick_attn_op(KsanaAttentionConfig(backend=KsanaAttentionBackend.TORCH_SDPA)))
    st = {"operations": ops, "device": "cpu", "dtype": torch.bfloat16, "rms_dtype": None}
    qb = QwenImageTransformerBlock(qdim, qheads, qdim // qheads, operation_settings=st)
    sd = {}
    for a, b in (("img_mod.1", "img_mod"), ("txt_mod.1", "txt_mod"), ("attn.to_q", "to_q"), ("attn.to_k", "to_k"),
                 ("attn.to_v", "to_v"), ("attn.add_q_proj", "add_q_proj"), ("attn.add_k_proj", "add_k_proj"),
                 ("attn.add_v_proj", "add_v_proj"), ("attn.to_out.0", "to_out"), ("attn.to_add_out", "to_add_out"),
                 ("img_mlp.net.0.proj", "img_mlp.0"), ("img_mlp.net.2", "img_mlp.2"),
                 ("txt_mlp.net.0.proj", "txt_mlp.0"), ("txt_mlp.net.2", "txt_mlp.2")):
        sd[a + ".weight"] = qp[b].w
        sd[a + ".bias"] = qp[b].b
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        sd[f"attn.{nm}.weight"] = qp[nm].to(torch.bfloat16)
    missing, unexpected = qb.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    qb.eval()
    qgrid, Lt = (1, 6, 8), 10
    Li = qgrid[0] * qgrid[1] * qgrid[2]
    img = D.make_activations(Li, qdim, seed=6)[None]
    txt = torch.randn(1, Lt, qdim, generator=g).to(torch.bfloat16)
    temb = torch.randn(1, qdim, generator=g).to(torch.bfloat16)
    rope = QwenEmbedRope(theta=10000, axes_dim=[16, 56, 56], scale_rope=True)
    vf, tf = rope(qgrid, [Lt], torch.device("cpu"))
    with torch.no_grad():
        t_ref, i_ref = qb(img, txt, temb, image_rotary_emb=(vf, tf))
    ia, ta = D.qwen_rope_angles(qgrid, Lt)
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        qp[nm] = qp[nm].to(torch.bfloat16)
    i_or, t_or = D.qwen_block_forward(qp, img[0], txt[0], temb[0], ia, ta, linear="fp32", attn="sdpa")
    di, dt = max_abs_rel(i_or.float(), i_ref[0].float()), max_abs_rel(t_or.float(), t_ref[0].float())
    print(f"[5] Qwen block: img max-abs-rel {di:.3e} cos {cos(i_or, i_ref[0]):.6f}; txt {dt:.3e} cos {cos(t_or, t_ref[0]):.6f}")
    assert di <= 1.5e-2 and dt <= 1.5e-2
    gold["qwen_block"] = dict(seed_params=5, seed_x=6, dim=qdim, ffn=qffn, heads=qheads, grid=torch.tensor(qgrid), txt=txt,
                              temb=temb, img_y=i_ref[0], txt_y=t_ref[0])

    # ---- (6) seeded stochastic rounding to FP8 (utils/ops.py:131-180) ---------------------
    from ksana.utils.ops import stochastic_rounding as ref_sr

    from ksanadit_b200 import casting
    sr = {}
    for nm, dt, shape in (("e4m3", torch.float8_e4m3fn, (96, 64)), ("e5m2", torch.float8_e5m2, (33, 40))):
        xs = torch.randn(*shape, generator=g) * 30
        xs[0, :8] = torch.tensor([0, 1e-4, -1e-3, 0.0019, 500, -600, 448, 0.0156])
        y_ref = ref_sr(xs.clone(), dt, seed=11)
        y_own = casting.stochastic_rounding(xs.clone(), dt, seed=11)
        assert torch.equal(y_ref.view(torch.uint8), y_own.view(torch.uint8)), nm
        sr[nm] = dict(x=xs, seed=11, y=y_ref.view(torch.uint8))
    print("[6] stochastic rounding: product == reference (bit-exact, e4m3 and e5m2)")
    gold["stochastic_rounding"] = sr

    # ---- (7) ComfyUI RoPE (utils/rope.py:151-212, wan_model.py:724-741) --------------------
    from ksana.utils.rope import EmbedND, apply_comfyui_rope
    cgrid = (3, 4, 6)
    emb = EmbedND(dim=dd, theta=10000.0, axes_dim=[dd - 4 * (dd // 6), 2 * (dd // 6), 2 * (dd // 6)])
    comfy = {}
    for nm, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        f_, h_, w_ = cgrid
        ids = torch.zeros((f_, h_, w_, 3), dtype=dt)
        ids[:, :, :, 0] += torch.linspace(0, f_ - 1, steps=f_, dtype=dt).reshape(-1, 1, 1)
        ids[:, :, :, 1] += torch.linspace(0, h_ - 1, steps=h_, dtype=dt).reshape(1, -1, 1)
        ids[:, :, :, 2] += torch.linspace(0, w_ - 1, steps=w_, dtype=dt).reshape(1, 1, -1)
        cf = emb(ids.reshape(1, -1, 3)).movedim(1, 2).to(dtype=dt)  # WanModel._rope_encode
        xc = torch.randn(1, f_ * h_ * w_, 2, dd, generator=g).to(dt)
        y_ref = apply_comfyui_rope(xc, cf)
        assert torch.equal(y_ref[0], D.apply_comfy_rope(xc[0], cgrid)), nm
        comfy[nm] = dict(x=xc[0], grid=torch.tensor(cgrid), y=y_ref[0])
    print("[7] ComfyUI RoPE: oracle == reference (bit-exact, bf16 and fp16)")
    gold["comfy_rope"] = comfy

    # ---- (8) Qwen block with zero_cond_t / modulate_index (qwen/transformer.py:171-188,206-208) ----
    qz = QwenImageTransformerBlock(qdim, qheads, qdim // qheads, zero_cond_t=True, operation_settings=st)
    qz.load_state_dict(sd, strict=False)
    qz.eval()
    temb2 = torch.randn(2, qdim, generator=g).to(torch.bfloat16)
    index = (torch.rand(1, Li, generator=g) < 0.4).to(torch.int64)
    with torch.no_grad():
        tz_ref, iz_ref = qz(img, txt, temb2, image_rotary_emb=(vf, tf), modulate_index=index)
    iz_or, tz_or = D.qwen_block_forward(qp, img[0], txt[0], temb2, ia, ta, linear="fp32", attn="sdpa", modulate_index=index[0])
    di, dt_ = max_abs_rel(iz_or.float(), iz_ref[0].float()), max_abs_rel(tz_or.float(), tz_ref[0].float())
    print(f"[8] Qwen block zero_cond_t: img max-abs-rel {di:.3e}; txt {dt_:.3e}")
    assert di <= 1.5e-2 and dt_ <= 1.5e-2
    with torch.no_grad():  # every token on row 0 / row 1: the per-token choice must matter
        _, i_all0 = qz(img, txt, temb2, image_rotary_emb=(vf, tf), modulate_index=torch.zeros_like(index))
    assert float((iz_ref != i_all0).float().mean()) > 0.2, "the index must change the image stream"
    gold["qwen_block_zero_cond"] = dict(temb=temb2, index=index[0], img_y=iz_ref[0], txt_y=tz_ref[0])

    # ---- (9) block-level step cache (cache/dbcache.py:60-450) on a toy block stack ----------
    from ksana.cache.dbcache import DBCache
    from ksana.config.cache_config.dbcache import DBCacheConfig as RefDBCfg
    from ksana.models.model_key import KsanaModelKey

    from ksanadit_b200.step_cache import B200DBCache, DBCacheConfig

    def eager_diff(x_new, x_old, prev):
        r = x_new - x_old
        if prev is None or prev.shape != r.shape:
            return r, None
        cm, pm = torch.abs(r).mean() + 1e-8, torch.abs(prev).mean() + 1e-8
        return r, float(torch.abs(r - prev).mean() / ((cm + pm) / 2))

    nb = 6
    gw = torch.Generator().manual_seed(21)
    toy_w = [torch.randn(32, 32, generator=gw) * 0.05 for _ in range(nb)]
    toy_blocks = [(lambda x, scale=1.0, w=w: x + torch.tanh(x.float() @ w).to(x.dtype) * scale) for w in toy_w]
    x_toy = torch.randn(16, 32, generator=gw).to(torch.bfloat16)
    dbc = {"weights": torch.stack(toy_w), "x": x_toy, "cases": []}
    for (fn, bn, thr, tay) in [(2, 1, 0.3, False), (1, 0, 0.08, False), (1, 0, 0.5, True), (0, 2, 0.2, False)]:
        kw = dict(fn_compute_blocks=fn, bn_compute_blocks=bn, residual_diff_threshold=thr, max_warmup_steps=2, warmup_interval=1,
                  max_cached_steps=5, max_continuous_cached_steps=2, num_blocks=nb, enable_taylorseer=tay)
        ref_c = DBCache(KsanaModelKey.Wan2_2_T2V_14B, RefDBCfg(**kw))
        own_c = B200DBCache(DBCacheConfig(**kw), diff_fn=eager_diff)
        outs = []
        for step in range(14):
            for phase in ("cond", "uncond"):
                xin = (x_toy * (1 + 0.02 * step) + (0.3 if phase == "uncond" else 0)).to(torch.bfloat16)
                a = ref_c(phase, xin.clone(), step, 1000 - step * 10, toy_blocks, scale=1.0 + 0.001 * step)
                b = own_c(phase, xin.clone(), step, 1000 - step * 10, toy_blocks, scale=1.0 + 0.001 * step)
                assert torch.equal(a, b), (fn, bn, thr, tay, step, phase)
                outs.append(a)
        rs = ref_c.get_stats_summary()
        assert rs["cond_cached_steps"] == own_c.get_stats_summary()["cond_cached_steps"] and rs["cond_cached_steps"] > 0
        dbc["cases"].append(dict(cfg=kw, outs=torch.stack(outs), cond_cached=rs["cond_cached_steps"], uncond_cached=rs["uncond_cached_steps"],
                                 diffs=torch.tensor(ref_c._diff_history)))
    print("[9] DBCache on a toy block stack: product state machine == reference (outputs bit-equal, same hits; 4 settings)")
    gold["dbcache"] = dbc

    out = os.path.join(HERE, "reference_vectors.pt")
    torch.save(gold, out)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
