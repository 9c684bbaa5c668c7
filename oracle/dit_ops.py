"""Oracle for the non-GEMM passes and the block wiring (plain torch, CPU).  Test infrastructure only.

Restates:
* LayerNorm / RMSNorm dtype rules            ksana/operations/ops.py:41-87
* adaLN modulate ``shift + LN(x) * (1+scale)``  ksana/models/wan/wan_model.py:374,391
* gated residual ``x + y * gate``             wan_model.py:385,392
* Wan 3-axis RoPE (complex, fp64)            ksana/utils/rope.py:22-24,43-58,62-128 ;
                                              table: wan_model.py:51-58,676-684
* WanSelfAttention / WanCrossAttention / WanAttentionBlock forward
                                              wan_model.py:148-206,233-251,325-393
* Qwen-Image dual-stream block               ksana/models/qwen/transformer.py:171-241,
                                              ksana/models/qwen/attention.py:31-59,320-371
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import quantizers as Qz
from . import sage as Sg

# --------------------------------------------------------------------------- norms / elementwise


def layernorm_noaffine(x, eps=1e-6):
    """ops.LayerNorm with elementwise_affine=False -> F.layer_norm in x.dtype (ops.py:48-52)."""
    return F.layer_norm(x, (x.shape[-1],), None, None, eps)


def layernorm_affine_fp32(x, w, b, eps=1e-6):
    """ops.LayerNorm with an fp32 weight -> computed in fp32, cast back (ops.py:45-50)."""
    return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float() if b is not None else None, eps).type_as(x)


def rmsnorm_fp32(x, w, eps=1e-6):
    """RMSNorm.float_rmsnorm (ops.py:64-70): x.float() * rsqrt(mean(x^2)+eps) * w -> x.dtype."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps) * w.float()).type_as(x)


def modulate(x, shift, scale, eps=1e-6):
    """torch.addcmul(shift, LN(x), 1 + scale) in x.dtype (wan_model.py:374)."""
    return torch.addcmul(shift.to(x.dtype), layernorm_noaffine(x, eps), 1 + scale.to(x.dtype))


def gate_residual(x, y, gate):
    """torch.addcmul(x, y, gate) (wan_model.py:385,392)."""
    return torch.addcmul(x, y, gate.to(x.dtype))


def gelu_tanh(x):
    return F.gelu(x, approximate="tanh")


# --------------------------------------------------------------------------- RoPE


def rope_params(max_seq_len, dim, theta=10000):
    """wan_model.py:51-58 -- complex128 table [max_seq_len, dim//2]."""
    freqs = torch.outer(
        torch.arange(max_seq_len),
        1.0 / torch.pow(theta, torch.arange(0, dim, 2).to(torch.float64).div(dim)),
    )
    return torch.polar(torch.ones_like(freqs), freqs)


def wan_freqs(head_dim=128, max_len=1024):
    """wan_model.py:676-684 -- cat of three axis tables with dims d-4(d//6), 2(d//6), 2(d//6)."""
    d = head_dim
    return torch.cat(
        [rope_params(max_len, d - 4 * (d // 6)), rope_params(max_len, 2 * (d // 6)), rope_params(max_len, 2 * (d // 6))],
        dim=1,
    )


def wan_rope_angles(grid, head_dim=128, theta=10000.0):
    """Per-token rotation angles [F*H*W, head_dim//2] in fp64 (what the tables above encode).

    Pair p of a head uses axis f for p < n_f, h for the next n_h, w for the rest,
    where (n_f, n_h, n_w) = (half - 2*(half//3), half//3, half//3)  (rope.py:22-24).
    """
    Fr, Hh, Ww = grid
    half = head_dim // 2
    n_h = n_w = half // 3
    n_f = half - 2 * n_h
    dims = [head_dim - 4 * (head_dim // 6), 2 * (head_dim // 6), 2 * (head_dim // 6)]
    inv = [1.0 / torch.pow(theta, torch.arange(0, d, 2).to(torch.float64).div(d)) for d in dims]
    assert [len(i) for i in inv] == [n_f, n_h, n_w]
    f = torch.arange(Fr, dtype=torch.float64).view(Fr, 1, 1, 1).expand(Fr, Hh, Ww, 1)
    h = torch.arange(Hh, dtype=torch.float64).view(1, Hh, 1, 1).expand(Fr, Hh, Ww, 1)
    w = torch.arange(Ww, dtype=torch.float64).view(1, 1, Ww, 1).expand(Fr, Hh, Ww, 1)
    ang = torch.cat([f * inv[0], h * inv[1], w * inv[2]], dim=-1)
    return ang.reshape(Fr * Hh * Ww, half)


def apply_wan_rope(x, grid, sp_rank=0, sp_size=1):
    """apply_default_rope for one sample (rope.py:62-128).  x: [L_local, N, D].

    Tokens past F*H*W pass through unchanged (sp_size == 1) or are rotated by 1+1j,
    i.e. the reference's ones-padding of the table (rope.py:30-40,108-112).
    """
    L, N, D = x.shape
    ang = wan_rope_angles(grid, D)
    cis = torch.polar(torch.ones_like(ang), ang)  # complex128 [S, D/2]
    S = cis.shape[0]
    if sp_size > 1:
        tgt = L * sp_size
        if S < tgt:
            cis = torch.cat([cis, torch.ones(tgt - S, D // 2, dtype=cis.dtype)], dim=0)
        cis = cis[sp_rank * L : (sp_rank + 1) * L]
        n_rot = L
    else:
        n_rot = min(S, L)
        cis = cis[:n_rot]
    xc = torch.view_as_complex(x[:n_rot].to(torch.float64).reshape(n_rot, N, D // 2, 2))
    y = torch.view_as_real(xc * cis[:, None, :]).flatten(2)
    y = torch.cat([y, x[n_rot:].to(torch.float64)])
    return y.type_as(x)


# --------------------------------------------------------------------------- linears used by the blocks


class LinearParams:
    """One Linear's parameters in the forms the different oracles need."""

    def __init__(self, w, b=None):
        self.w = w  # [N,K] high precision
        self.b = b
        self.wq, self.sw = Qz.weight_quant_fp8_channelwise(w)

    def fp32(self, x):
        return F.linear(x.float(), self.w.float(), None if self.b is None else self.b.float()).to(x.dtype)

    def fp8(self, x):
        return Qz.fp8_linear_emulated(x, self.wq, self.sw, self.b, out_dtype=x.dtype)


def comfy_rope_matrices(grid, head_dim=128, theta=10000.0, dtype=torch.bfloat16):
    """``WanModel._rope_encode`` + ``EmbedND`` + ``_comfy_rope`` (wan_model.py:724-741, rope.py:151-180):
    [L, head_dim/2, 2, 2] rotation matrices [[cos, -sin], [sin, cos]] for the (f, h, w) position of every token.
    Position ids are made in ``dtype``, angles in fp64 from fp32 positions, matrices rounded to fp32 then ``dtype``."""
    f, h, w = grid
    ids = torch.zeros(f, h, w, 3, dtype=dtype)
    ids[..., 0] += torch.linspace(0, f - 1, steps=f, dtype=dtype).reshape(-1, 1, 1)
    ids[..., 1] += torch.linspace(0, h - 1, steps=h, dtype=dtype).reshape(1, -1, 1)
    ids[..., 2] += torch.linspace(0, w - 1, steps=w, dtype=dtype).reshape(1, 1, -1)
    ids = ids.reshape(-1, 3)
    d = head_dim
    mats = []
    for axis, dd in enumerate([d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)]):
        omega = 1.0 / (theta ** torch.linspace(0, (dd - 2) / dd, steps=dd // 2, dtype=torch.float64))
        ang = torch.einsum("n,d->nd", ids[:, axis].to(torch.float32), omega)
        m = torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1)
        mats.append(m.reshape(*m.shape[:-1], 2, 2).to(torch.float32))
    return torch.cat(mats, dim=-3).to(dtype)


def apply_comfy_rope(x, grid, theta=10000.0):
    """``apply_comfyui_rope`` (rope.py:183-212) on x [L, N, D]: out = M[..., 0] * x0 + M[..., 1] * x1 per channel pair,
    in the dtype of the matrices (= x's), the second term through ``addcmul_``."""
    L, N, D = x.shape
    M = comfy_rope_matrices(grid, D, theta, x.dtype)[:L, None]  # [L, 1, D/2, 2, 2]
    x_ = x.to(M.dtype).reshape(L, N, D // 2, 1, 2)
    out = M[..., 0] * x_[..., 0]
    out.addcmul_(M[..., 1], x_[..., 1])
    return out.reshape(L, N, D).type_as(x)


def make_linear_fn(mode):
    return (lambda lp, x: lp.fp8(x)) if mode == "fp8" else (lambda lp, x: lp.fp32(x))


def make_attn_fn(mode):
    """mode 'sdpa' (exact) or 'sage' (quantised emulation).  Tensors [B,L,H,D]."""

    def run(q, k, v):
        outs = []
        for b in range(q.shape[0]):
            if mode == "sage":
                outs.append(Sg.sage_attention(q[b], k[b], v[b]))
            else:
                outs.append(Sg.sdpa_reference(q[b], k[b], v[b]).to(q.dtype))
        return torch.stack(outs)

    return run


# --------------------------------------------------------------------------- Wan block


def wan_block_forward(p, x, e, context, grid, linear="fp8", attn="sage", eps=1e-6, sp_rank=0, sp_size=1, a2a=None, rope="default"):
    """WanAttentionBlock.forward (wan_model.py:325-393) on x [B,L,C], e [B,1,6,C], context [B,Lc,C].

    p: dict with 'modulation' [1,6,C]; LinearParams under 'self.q','self.k','self.v','self.o',
    'cross.q','cross.k','cross.v','cross.o','ffn.0','ffn.2'; fp32 vectors 'self.norm_q','self.norm_k',
    'cross.norm_q','cross.norm_k','norm3.w','norm3.b'; int 'num_heads'.
    a2a: optional (scatter_heads_gather_seq, scatter_seq_gather_heads) pair for Ulysses.
    rope: "default" (complex fp64, rope.py:62-128) or "comfy" (2x2 matrices in the activation dtype, rope.py:151-212).
    """
    lin = make_linear_fn(linear)
    att = make_attn_fn(attn)
    B, L, C = x.shape
    n = p["num_heads"]
    d = C // n
    em = (p["modulation"].unsqueeze(0) + e).unbind(2)  # 6 x [B,1,C]   (wan_model.py:366-369)

    h = modulate(x, em[0], em[1], eps)
    q = rmsnorm_fp32(lin(p["self.q"], h), p["self.norm_q"], eps).view(B, L, n, d)
    k = rmsnorm_fp32(lin(p["self.k"], h), p["self.norm_k"], eps).view(B, L, n, d)
    v = lin(p["self.v"], h).view(B, L, n, d)
    if rope == "comfy":
        assert sp_size == 1
        q = torch.stack([apply_comfy_rope(q[b], grid) for b in range(B)])
        k = torch.stack([apply_comfy_rope(k[b], grid) for b in range(B)])
    else:
        q = torch.stack([apply_wan_rope(q[b], grid, sp_rank, sp_size) for b in range(B)])
        k = torch.stack([apply_wan_rope(k[b], grid, sp_rank, sp_size) for b in range(B)])
    if a2a is not None:
        q, k, v = (a2a[0](t) for t in (q, k, v))
    y = att(q, k, v)
    if a2a is not None:
        y = a2a[1](y)
    y = lin(p["self.o"], y.flatten(2))
    x = gate_residual(x, y, em[2])

    xn = layernorm_affine_fp32(x, p["norm3.w"], p["norm3.b"], eps)
    Lc = context.shape[1]
    cq = rmsnorm_fp32(lin(p["cross.q"], xn), p["cross.norm_q"], eps).view(B, L, n, d)
    ck = rmsnorm_fp32(lin(p["cross.k"], context), p["cross.norm_k"], eps).view(B, Lc, n, d)
    cv = lin(p["cross.v"], context).view(B, Lc, n, d)
    y = att(cq, ck, cv)
    x = x + lin(p["cross.o"], y.flatten(2))

    h = modulate(x, em[3], em[4], eps)
    y = lin(p["ffn.2"], gelu_tanh(lin(p["ffn.0"], h)))
    return gate_residual(x, y, em[5])


def make_wan_block_params(dim, ffn, heads, seed=0, dtype=torch.bfloat16, std=0.02):
    """Seeded random-init parameters in the style of the benchmark's configuration 1 (weights ~N(0, 0.02))."""
    g = torch.Generator().manual_seed(seed)

    def W(n, k):
        return (torch.randn(n, k, generator=g) * std).to(dtype)

    def Bv(n):
        return (torch.randn(n, generator=g) * std).to(dtype)

    p = {"num_heads": heads, "modulation": (torch.randn(1, 6, dim, generator=g) * 0.1).to(dtype)}
    for name, (n, k) in {
        "self.q": (dim, dim), "self.k": (dim, dim), "self.v": (dim, dim), "self.o": (dim, dim),
        "cross.q": (dim, dim), "cross.k": (dim, dim), "cross.v": (dim, dim), "cross.o": (dim, dim),
        "ffn.0": (ffn, dim), "ffn.2": (dim, ffn),
    }.items():
        p[name] = LinearParams(W(n, k), Bv(n))
    for name in ("self.norm_q", "self.norm_k", "cross.norm_q", "cross.norm_k", "norm3.w"):
        p[name] = 1.0 + 0.1 * torch.randn(dim, generator=g)
    p["norm3.b"] = 0.1 * torch.randn(dim, generator=g)
    return p


def make_activations(L, dim, seed=0, dtype=torch.bfloat16, outlier_frac=0.01, outlier_mul=20.0):
    """x ~ N(0,1) with 1% of channels scaled x20 (the benchmark's configurations 1 and 2)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(L, dim, generator=g)
    n_out = max(1, int(round(dim * outlier_frac)))
    idx = torch.randperm(dim, generator=g)[:n_out]
    x[:, idx] *= outlier_mul
    return x.to(dtype)


# --------------------------------------------------------------------------- Qwen-Image dual-stream block


def qwen_rope_angles(img_grid, txt_len, axes=(16, 56, 56), theta=10000.0, scale_rope=True):
    """Angles [L_txt + L_img, sum(axes)//2] restating QwenEmbedRope (qwen/attention.py:62-142).

    Image positions are centred when scale_rope (attention.py:100-104); text positions start at
    max(h, w) // 2 ... on every axis (attention.py:118-126).  Returned order: (img_angles, txt_angles).
    """
    Fr, Hh, Ww = img_grid
    inv = [1.0 / torch.pow(theta, torch.arange(0, d, 2).to(torch.float64).div(d)) for d in axes]
    fpos = torch.arange(Fr, dtype=torch.float64)
    if scale_rope:
        hpos = torch.cat([torch.arange(-(Hh - Hh // 2), 0), torch.arange(0, Hh // 2)]).to(torch.float64)
        wpos = torch.cat([torch.arange(-(Ww - Ww // 2), 0), torch.arange(0, Ww // 2)]).to(torch.float64)
        txt0 = max(Hh // 2, Ww // 2)
    else:
        hpos = torch.arange(Hh, dtype=torch.float64)
        wpos = torch.arange(Ww, dtype=torch.float64)
        txt0 = max(Hh, Ww)
    f = fpos.view(Fr, 1, 1, 1).expand(Fr, Hh, Ww, 1)
    h = hpos.view(1, Hh, 1, 1).expand(Fr, Hh, Ww, 1)
    w = wpos.view(1, 1, Ww, 1).expand(Fr, Hh, Ww, 1)
    img = torch.cat([f * inv[0], h * inv[1], w * inv[2]], dim=-1).reshape(Fr * Hh * Ww, -1)
    t = torch.arange(txt0, txt0 + txt_len, dtype=torch.float64).view(-1, 1)
    txt = torch.cat([t * inv[0], t * inv[1], t * inv[2]], dim=-1)
    return img, txt


def apply_rope_angles(x, ang):
    """apply_rotary_emb_qwen with complex freqs (qwen/attention.py:31-59): fp32 complex multiply.  x:[L,N,D]."""
    L, N, D = x.shape
    cis = torch.polar(torch.ones_like(ang), ang).to(torch.complex64)
    xc = torch.view_as_complex(x.float().reshape(L, N, D // 2, 2))
    return torch.view_as_real(xc * cis[:, None, :]).flatten(2).type_as(x)


def rmsnorm_heads(x, w, eps=1e-6):
    """Per-head RMSNorm over head_dim (qwen/attention.py:267-272,340-343).  x: [L,N,D], w: [D]."""
    return rmsnorm_fp32(x, w, eps)


def qwen_block_forward(p, img, txt, temb, img_ang, txt_ang, linear="fp8", attn="sage", eps=1e-6, modulate_index=None):
    """QwenImageTransformerBlock.forward (qwen/transformer.py:196-241), batch 1.

    img [Li,C], txt [Lt,C], temb [C] -- or [2,C] = [real timestep; zero timestep] together with
    ``modulate_index`` [Li] in {0,1} (the block's ``zero_cond_t`` mode, transformer.py:171-188,206-208:
    every image token picks its shift / scale / gate from the row its index names, the text stream uses
    row 0).  p holds LinearParams 'img_mod','txt_mod' (C -> 6C),
    'to_q','to_k','to_v','add_q_proj','add_k_proj','add_v_proj','to_out','to_add_out',
    'img_mlp.0','img_mlp.2','txt_mlp.0','txt_mlp.2' and fp32 [D] vectors 'norm_q','norm_k',
    'norm_added_q','norm_added_k'.  fp16 outputs are clamped to +-65504 (transformer.py:236-239).
    """
    lin = make_linear_fn(linear)
    att = make_attn_fn(attn)
    n = p["num_heads"]
    C = img.shape[-1]
    d = C // n
    st = F.silu(temb.reshape(-1, C))
    assert (st.shape[0] == 2) == (modulate_index is not None), "two temb rows go with a modulate_index"
    img_mod = lin(p["img_mod"], st).chunk(2, dim=-1)  # every ops.Linear of the block is the FP8 Linear
    txt_mod = lin(p["txt_mod"], st[:1]).chunk(2, dim=-1)

    def mod(x, m, index=None):  # transformer.py:171-194
        shift, scale, gate = m.chunk(3, dim=-1)
        if index is None:
            shift, scale, gate = shift[0], scale[0], gate[0]
        else:
            rows = index.long()
            shift, scale, gate = shift[rows], scale[rows], gate[rows]
        return layernorm_noaffine(x, eps) * (1 + scale) + shift, gate

    ih, ig1 = mod(img, img_mod[0], modulate_index)
    th, tg1 = mod(txt, txt_mod[0])
    Li, Lt = img.shape[0], txt.shape[0]
    iq = rmsnorm_heads(lin(p["to_q"], ih).view(Li, n, d), p["norm_q"], eps)
    ik = rmsnorm_heads(lin(p["to_k"], ih).view(Li, n, d), p["norm_k"], eps)
    iv = lin(p["to_v"], ih).view(Li, n, d)
    tq = rmsnorm_heads(lin(p["add_q_proj"], th).view(Lt, n, d), p["norm_added_q"], eps)
    tk = rmsnorm_heads(lin(p["add_k_proj"], th).view(Lt, n, d), p["norm_added_k"], eps)
    tv = lin(p["add_v_proj"], th).view(Lt, n, d)
    iq, ik = apply_rope_angles(iq, img_ang), apply_rope_angles(ik, img_ang)
    tq, tk = apply_rope_angles(tq, txt_ang), apply_rope_angles(tk, txt_ang)
    q = torch.cat([tq, iq])[None]  # text first (attention.py:355-357)
    k = torch.cat([tk, ik])[None]
    v = torch.cat([tv, iv])[None]
    o = att(q, k, v)[0].flatten(1)
    to, io = o[:Lt], o[Lt:]
    img = img + ig1 * lin(p["to_out"], io)
    txt = txt + tg1 * lin(p["to_add_out"], to)
    ih, ig2 = mod(img, img_mod[1], modulate_index)
    img = img + ig2 * lin(p["img_mlp.2"], gelu_tanh(lin(p["img_mlp.0"], ih)))
    th, tg2 = mod(txt, txt_mod[1])
    txt = txt + tg2 * lin(p["txt_mlp.2"], gelu_tanh(lin(p["txt_mlp.0"], th)))
    if img.dtype == torch.float16:
        img, txt = img.clamp(-65504, 65504), txt.clamp(-65504, 65504)
    return img, txt


def make_qwen_block_params(dim, ffn, heads, seed=0, dtype=torch.bfloat16, std=0.02):
    g = torch.Generator().manual_seed(seed)

    def W(n, k):
        return (torch.randn(n, k, generator=g) * std).to(dtype)

    def Bv(n):
        return (torch.randn(n, generator=g) * std).to(dtype)

    p = {"num_heads": heads}
    shapes = {"img_mod": (6 * dim, dim), "txt_mod": (6 * dim, dim)}
    for nm in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out", "to_add_out"):
        shapes[nm] = (dim, dim)
    for s in ("img_mlp", "txt_mlp"):
        shapes[s + ".0"] = (ffn, dim)
        shapes[s + ".2"] = (dim, ffn)
    for nm, (n, k) in shapes.items():
        p[nm] = LinearParams(W(n, k), Bv(n))
    for nm in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
        p[nm] = 1.0 + 0.1 * torch.randn(dim // heads, generator=g)
    return p
