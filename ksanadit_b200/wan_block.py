"""Wan DiT block on the B200 kernels: the fused form of ``WanAttentionBlock.forward``.

Takes the same inputs and holds the same parameters (same state-dict names) as KsanaDiT's
``WanAttentionBlock`` / ``WanSelfAttention`` / ``WanCrossAttention``
(ksana/models/wan/wan_model.py:61-393), but runs the block as the kernel sequence

  adaLN+quant -> QKV GEMM -> RMSNorm+RoPE (in place) -> [Ulysses all-to-all] -> Sage quantisers ->
  INT8/FP8 attention -> [all-to-all] -> quant -> o-proj GEMM (+gated residual) ->
  LayerNorm+quant -> cross-attention (q GEMM, cached context K/V, attention, o GEMM + residual) ->
  adaLN+quant -> FFN-up GEMM (+GELU) -> quant -> FFN-down GEMM (+gated residual)

so that every elementwise pass of the eager block is fused into a quantiser or a GEMM epilogue.
torch is used for buffers, views and the NCCL exchange only.
"""

from __future__ import annotations

import torch

from . import _lib, distribute, ops
from .linear import B200Fp8Linear, quantize_weight_per_channel

HEAD = 128


class B200WanBlock(torch.nn.Module):
    def __init__(self, dim, ffn_dim, num_heads, block_id=0, eps=1e-6, cross_attn_norm=True, device="cuda",
                 dtype=torch.bfloat16, tile_lists=None, cache_context=False):
        super().__init__()
        if dim != num_heads * HEAD:
            raise _lib.KsanaB200Error(f"head size {dim // num_heads} is not supported (only {HEAD})")
        self.dim, self.ffn_dim, self.num_heads, self.block_id, self.eps = dim, ffn_dim, num_heads, block_id, eps
        self.dtype = dtype
        kw = dict(device=device, dtype=dtype)
        self.self_attn = torch.nn.Module()
        self.self_attn.qkv = B200Fp8Linear(dim, 3 * dim, **kw)
        self.self_attn.o = B200Fp8Linear(dim, dim, **kw)
        self.self_attn.norm_q = torch.nn.Module()
        self.self_attn.norm_k = torch.nn.Module()
        self.cross_attn = torch.nn.Module()
        for n in "qkvo":
            setattr(self.cross_attn, n, B200Fp8Linear(dim, dim, **kw))
        self.cross_attn.norm_q = torch.nn.Module()
        self.cross_attn.norm_k = torch.nn.Module()
        for m in (self.self_attn.norm_q, self.self_attn.norm_k, self.cross_attn.norm_q, self.cross_attn.norm_k):
            m.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=torch.float32), requires_grad=False)
        self.norm3 = torch.nn.Module()
        self.norm3.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=torch.float32), requires_grad=False)
        self.norm3.bias = torch.nn.Parameter(torch.zeros(dim, device=device, dtype=torch.float32), requires_grad=False)
        self.cross_attn_norm = cross_attn_norm
        self.ffn = torch.nn.ModuleList([B200Fp8Linear(dim, ffn_dim, **kw), torch.nn.Identity(), B200Fp8Linear(ffn_dim, dim, **kw)])
        self.modulation = torch.nn.Parameter(torch.zeros(1, 6, dim, device=device, dtype=dtype), requires_grad=False)
        self.tile_lists = tile_lists  # (offsets, entries, order) for block-sparse self-attention, or None
        self.cache_context = cache_context  # keep the quantised context K/V across steps (off: recomputed every call)
        self.peer_exchange = None  # distribute.PeerExchange: exchange fused into the kernels instead of NCCL all-to-alls
        self._ones = None
        self._ctx_cache = None

    # ------------------------------------------------------------------ parameter loading
    @staticmethod
    def _set_linear(lin: B200Fp8Linear, w, b, scale=None):
        if w.dtype == torch.float8_e4m3fn:
            wq, s = w, (torch.ones((), dtype=torch.float32) if scale is None else scale.float())
        else:
            wq, s = quantize_weight_per_channel(w.to(lin.weight.device))
        lin.weight = torch.nn.Parameter(wq.to(lin.weight.device).contiguous(), requires_grad=False)
        lin.scale_weight = torch.nn.Parameter(s.to(lin.weight.device), requires_grad=False)
        lin._w_scale_vec = None
        if b is not None:
            lin.bias = torch.nn.Parameter(b.to(lin.weight.device, lin.compute_dtype), requires_grad=False)

    def load_block_state_dict(self, sd: dict):
        """Loads a state dict with WanAttentionBlock's names.  High-precision weights are quantised per output
        channel; fp8 weights are taken as they are with their ``scale_weight``.  Separate q/k/v are fused."""
        sd = dict(sd)
        from .fuse_qkv import MODEL_QKV_PATTERNS, remap_qkv_weights
        if "self_attn.q.weight" in sd and sd["self_attn.q.weight"].dtype != torch.float8_e4m3fn:
            for n in "qkv":  # quantise before fusing so that each projection keeps its own channel scales
                wq, s = quantize_weight_per_channel(sd["self_attn." + n + ".weight"].to(self.modulation.device))
                sd["self_attn." + n + ".weight"], sd["self_attn." + n + ".scale_weight"] = wq, s
        remap_qkv_weights(sd, [tuple(p.lstrip(".") for p in MODEL_QKV_PATTERNS["wan"][0])])
        for name, lin in (("self_attn.qkv", self.self_attn.qkv), ("self_attn.o", self.self_attn.o), ("cross_attn.q", self.cross_attn.q),
                          ("cross_attn.k", self.cross_attn.k), ("cross_attn.v", self.cross_attn.v), ("cross_attn.o", self.cross_attn.o),
                          ("ffn.0", self.ffn[0]), ("ffn.2", self.ffn[2])):
            self._set_linear(lin, sd[name + ".weight"], sd.get(name + ".bias"), sd.get(name + ".scale_weight"))
        dev = self.modulation.device
        for name, mod in (("self_attn.norm_q", self.self_attn.norm_q), ("self_attn.norm_k", self.self_attn.norm_k),
                          ("cross_attn.norm_q", self.cross_attn.norm_q), ("cross_attn.norm_k", self.cross_attn.norm_k)):
            mod.weight = torch.nn.Parameter(sd[name + ".weight"].float().to(dev).contiguous(), requires_grad=False)
        if "norm3.weight" in sd:
            self.norm3.weight = torch.nn.Parameter(sd["norm3.weight"].float().to(dev).contiguous(), requires_grad=False)
            self.norm3.bias = torch.nn.Parameter(sd["norm3.bias"].float().to(dev).contiguous(), requires_grad=False)
        self.modulation = torch.nn.Parameter(sd["modulation"].to(dev, self.dtype), requires_grad=False)
        self._ctx_cache = None
        return self

    def random_init(self, seed: int, std: float = 0.02, qk_offset: float = 0.5):
        """Random-init weights of this architecture, drawn on the device (weights ~ N(0, std)); the Q and K
        projections get a per-channel bias ~ N(0, qk_offset) so that K smoothing has a mean to remove."""
        g = torch.Generator(device=self.modulation.device).manual_seed(seed)
        dev = self.modulation.device

        def W(n, k):
            return (torch.randn(n, k, device=dev, generator=g) * std).to(self.dtype)

        def V(n, s=std):
            return (torch.randn(n, device=dev, generator=g) * s)

        for lin in (self.self_attn.qkv, self.self_attn.o, self.cross_attn.q, self.cross_attn.k, self.cross_attn.v, self.cross_attn.o,
                    self.ffn[0], self.ffn[2]):
            self._set_linear(lin, W(lin.out_features, lin.in_features), V(lin.out_features).to(self.dtype))
        if qk_offset:
            self.self_attn.qkv.bias.data[: 2 * self.dim] = V(2 * self.dim, qk_offset).to(self.dtype)
        for mod in (self.self_attn.norm_q, self.self_attn.norm_k, self.cross_attn.norm_q, self.cross_attn.norm_k, self.norm3):
            mod.weight = torch.nn.Parameter((1 + V(self.dim, 0.1)).float(), requires_grad=False)
        self.norm3.bias = torch.nn.Parameter(V(self.dim, 0.1).float(), requires_grad=False)
        self.modulation = torch.nn.Parameter((torch.randn(1, 6, self.dim, device=dev, generator=g) * 0.1).to(self.dtype), requires_grad=False)
        self._ctx_cache = None
        return self

    # ------------------------------------------------------------------ pieces
    def _context_kv(self, context, owner=None, slot=0):
        """Quantised cross-attention K / V of the text context [Lc, C].  They depend only on the block's weights and
        the prompt; with ``cache_context`` they are kept across denoise steps (the reference recomputes them every
        step, wan_model.py:237-238, and so does the default here).  A cached entry is reused only while the caller
        passes the very same tensor object ``owner`` (the batch the row ``slot`` was taken from), unmodified: the
        cache holds a reference to it, so a new prompt tensor can never be mistaken for the old one by its address.
        One entry per batch row."""
        if self.cache_context and owner is not None:
            if self._ctx_cache is None:
                self._ctx_cache = {}
            hit = self._ctx_cache.get(slot)
            if hit is not None and hit[0] is owner and hit[1] == owner._version:
                return hit[2]
        ca = self.cross_attn
        Lc = context.shape[0]
        k = ca.k(context)
        ops.rmsnorm_rope_inplace(k, ca.norm_k.weight, self.eps)
        v = ca.v(context)
        k3, v3 = k.view(Lc, self.num_heads, HEAD), v.view(Lc, self.num_heads, HEAD)
        km = ops.sage_kmean(k3)
        k8, ks = ops.sage_quant_int8(k3, ops.K_BLOCK, mean=km)
        vt, vs = ops.sage_quant_v(v3)
        val = (k8, ks, vt, vs, Lc)
        if self.cache_context and owner is not None:
            self._ctx_cache[slot] = (owner, owner._version, val)
        return val

    # The sequence-parallel self-attention with the exchange fused into the kernels' output stages, in three
    # phases separated by "all ranks are done storing" barriers (distribute.PeerExchange):
    #   a: QKV GEMM storing into the head owners' buffers + the norm factors of this rank's tokens to every rank
    #   b: norm / RoPE / quantisers on (all tokens, local heads), attention storing into the token owners' buffers
    #   c: this rank's [L, C] attention output
    def _fused_phase_a(self, ex, xq, sx):
        sa = self.self_attn
        ops.fp8_gemm_qkv_scatter(xq, sx, sa.qkv.weight.data, sa.qkv.weight_scale_vector(), sa.qkv.bias, self.num_heads,
                                 ex.qkv_ptrs, ex.rank, ex.tile_sumsq, self.dtype)
        ops.rowsumsq_to_rstd_scatter(ex.tile_sumsq, xq.shape[0], self.dim, self.eps, ex.rstd_ptrs, ex.rank)

    def _fused_phase_b(self, ex, grid, rope):
        sa = self.self_attn
        Hl = self.num_heads // ex.P
        Cl = Hl * HEAD
        La = ex.P * ex.L_loc
        w = slice(ex.rank * Cl, (ex.rank + 1) * Cl)
        q3, k3, v3 = ex.qkv[:, 0], ex.qkv[:, 1], ex.qkv[:, 2]  # [La, Hl, 128] each
        # norm + RoPE run inside the K mean and the quantisers, with the norm factors every rank stored in phase a
        wq, wk = sa.norm_q.weight[w], sa.norm_k.weight[w]
        km = ops.sage_kmean_normed(k3, wk, self.eps, rope, grid, row_rstd=ex.rstd[1])
        q8, qs = ops.sage_quant_int8_normed(q3, ops.Q_BLOCK, wq, premul=ops.q_premul(HEAD), eps=self.eps, rope=rope, grid=grid,
                                            row_rstd=ex.rstd[0])
        k8, ks = ops.sage_quant_int8_normed(k3, ops.K_BLOCK, wk, mean=km, eps=self.eps, rope=rope, grid=grid, row_rstd=ex.rstd[1])
        vt, vs = ops.sage_quant_v(v3)
        offs, ents, order = self.tile_lists if self.tile_lists is not None else (None, None, None)
        esz = ex.out.element_size()
        ptrs = [p + ex.rank * Cl * esz for p in ex.out_ptrs]  # this rank's head slot in every token owner's buffer
        ops.sage_attn_core(q8, qs, k8, ks, vt, vs, La, La, self.dtype, offs, ents, tile_order=order,
                           peer_out=(ptrs, ex.L_loc, self.dim, HEAD))

    def _self_attention(self, xq, sx, L, grid, rope):
        C, H = self.dim, self.num_heads
        ex = self.peer_exchange
        if ex is not None:
            if ex.L_loc != L or ex.heads != H or ex.dtype != self.dtype:
                raise _lib.KsanaB200Error(f"peer exchange was built for {ex.L_loc} tokens x {ex.heads} heads, got {L} x {H}")
            self._fused_phase_a(ex, xq, sx)
            ex.barrier()
            self._fused_phase_b(ex, grid, rope)
            ex.barrier()
            return ex.out.view(L, C)
        P, rank = distribute.get_world_size(), distribute.get_rank_id()
        sa = self.self_attn
        if P == 1 and C % 256 == 0:
            # one GPU: the norm factors come out of the projection's epilogue, and norm + RoPE run inside the K mean
            # and the quantisers, so the normalised Q and K are never written (Q is read once, K twice)
            qkv, sums = sa.qkv.forward_quantized_rowstats(xq, sx, self.dtype, 2 * C)
            rstd = ops.rowsumsq_to_rstd(sums, C, self.eps)
            t = qkv.view(L, 3, H, HEAD)
            km = ops.sage_kmean_normed(t[:, 1], sa.norm_k.weight, self.eps, rope, grid, row_rstd=rstd[1])
            q8, qs = ops.sage_quant_int8_normed(t[:, 0], ops.Q_BLOCK, sa.norm_q.weight, premul=ops.q_premul(HEAD), eps=self.eps,
                                                rope=rope, grid=grid, row_rstd=rstd[0])
            k8, ks = ops.sage_quant_int8_normed(t[:, 1], ops.K_BLOCK, sa.norm_k.weight, mean=km, eps=self.eps, rope=rope, grid=grid,
                                                row_rstd=rstd[1])
            vt, vs = ops.sage_quant_v(t[:, 2])
            offs, ents, order = self.tile_lists if self.tile_lists is not None else (None, None, None)
            return ops.sage_attn_core(q8, qs, k8, ks, vt, vs, L, L, self.dtype, offs, ents, tile_order=order).reshape(L, C)
        qkv = sa.qkv.forward_quantized(xq, sx, self.dtype)  # [L, 3C]
        km = ops.rmsnorm_rope_inplace(qkv[:, C:2 * C], sa.norm_k.weight, self.eps, rope, grid, pos0=rank * L, want_mean=(P == 1))
        ops.rmsnorm_rope_inplace(qkv[:, :C], sa.norm_q.weight, self.eps, rope, grid, pos0=rank * L)
        if P > 1:
            g = distribute.heads_to_sequence(qkv.view(L, 3, H, HEAD))  # [L*P, 3, H/P, D]
            q3, k3, v3 = g[:, 0], g[:, 1], g[:, 2]
            km = ops.sage_kmean(k3)
        else:
            t = qkv.view(L, 3, H, HEAD)
            q3, k3, v3 = t[:, 0], t[:, 1], t[:, 2]
            km = km.view(H, HEAD)
        Lf = q3.shape[0]
        q8, qs = ops.sage_quant_int8(q3, ops.Q_BLOCK, premul=ops.q_premul(HEAD))
        k8, ks = ops.sage_quant_int8(k3, ops.K_BLOCK, mean=km)
        vt, vs = ops.sage_quant_v(v3)
        offs, ents, order = self.tile_lists if self.tile_lists is not None else (None, None, None)
        o = ops.sage_attn_core(q8, qs, k8, ks, vt, vs, Lf, Lf, self.dtype, offs, ents, tile_order=order)  # [L*P, H/P, D]
        if P > 1:
            o = distribute.sequence_to_heads(o)  # [L, H, D]
        return o.reshape(L, C)

    def _block_one(self, x, e6, context, grid, rope, ctx_owner=None, slot=0):
        """x [L, C]; e6 six [1, C] or [L, C] tensors (modulation already added); context [Lc, C]."""
        L, C = x.shape
        if self._ones is None or self._ones.device != x.device:
            self._ones = torch.ones(1, C, dtype=self.dtype, device=x.device)
        # self-attention
        xq, sx = ops.adaln_quant_fp8(x, e6[0], e6[1], self.eps)
        a = self._self_attention(xq, sx, L, grid, rope)
        aq, sa = ops.quant_fp8_rowwise(a)
        x = self.self_attn.o.forward_quantized(aq, sa, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x, gate=e6[2])
        # cross-attention
        ca = self.cross_attn
        if self.cross_attn_norm:
            hq, hs = ops.layernorm_quant_fp8(x, self.norm3.weight, self.norm3.bias, self.eps)
        else:
            hq, hs = ops.quant_fp8_rowwise(x)
        k8, ks, vt, vs, Lc = self._context_kv(context, ctx_owner, slot)
        if C % 256 == 0:
            q, sums = ca.q.forward_quantized_rowstats(hq, hs, self.dtype, C)
            q8, qs = ops.sage_quant_int8_normed(q.view(L, self.num_heads, HEAD), ops.Q_BLOCK, ca.norm_q.weight, premul=ops.q_premul(HEAD),
                                                eps=self.eps, row_rstd=ops.rowsumsq_to_rstd(sums, C, self.eps)[0])
        else:
            q = ca.q.forward_quantized(hq, hs, self.dtype)
            ops.rmsnorm_rope_inplace(q, ca.norm_q.weight, self.eps)
            q8, qs = ops.sage_quant_int8(q.view(L, self.num_heads, HEAD), ops.Q_BLOCK, premul=ops.q_premul(HEAD))
        o = ops.sage_attn_core(q8, qs, k8, ks, vt, vs, L, Lc, self.dtype).view(L, C)
        oq, os_ = ops.quant_fp8_rowwise(o)
        x = ca.o.forward_quantized(oq, os_, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x, gate=self._ones, out=x)
        # FFN
        xq, sx = ops.adaln_quant_fp8(x, e6[3], e6[4], self.eps)
        h = self.ffn[0].forward_quantized(xq, sx, self.dtype, _lib.EPI_GELU_TANH)
        hq, hs = ops.quant_fp8_rowwise(h)
        x = self.ffn[2].forward_quantized(hq, hs, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x, gate=e6[5], out=x)
        return x

    def _per_sample_quant(self, B, L, K, fn):
        """Runs a row-wise quantiser once per sample, each writing its rows of one [B*L, K] activation buffer."""
        dev = self.modulation.device
        q = torch.empty(B * L, K, dtype=torch.float8_e4m3fn, device=dev)
        s = torch.empty(B * L, dtype=torch.float32, device=dev)
        for b in range(B):
            fn(b, (q[b * L:(b + 1) * L], s[b * L:(b + 1) * L]))
        return q, s

    def _block_batched(self, x, em, context, grid, rope):
        """The block on a batch of B equal-length sequences folded into the row dimension (cond / uncond batching,
        ksana/generators/generator.py:356-375,859-871): every Linear runs once at M = B * L, so its weights are streamed
        once and its tail is paid once; every attention runs once over B * H heads.  x [B, L, C]; em [B, 1, 6, C]
        (modulation per sample; the row-wise passes that take a modulation vector run once per sample on that sample's
        rows of the shared buffers, the GEMM epilogues take one gate row per sample); context [B, Lc, C]."""
        B, L, C = x.shape
        H, M = self.num_heads, B * L
        dev = x.device
        if self._ones is None or self._ones.device != dev:
            self._ones = torch.ones(1, C, dtype=self.dtype, device=dev)
        e6 = [em[:, 0, i].contiguous() for i in range(6)]  # six [B, C]
        x2 = x.reshape(M, C)
        sa, ca = self.self_attn, self.cross_attn
        Lp = ops.pad128(L)

        def heads_operands(Lk_pad):
            return (torch.empty(B * H, Lk_pad, HEAD, dtype=torch.int8, device=dev),
                    torch.empty(B * H, Lk_pad // ops.K_BLOCK, dtype=torch.float32, device=dev),
                    torch.empty(B * H, HEAD, Lk_pad, dtype=torch.float8_e4m3fn, device=dev),
                    torch.empty(B * H, HEAD, dtype=torch.float32, device=dev))

        def quant_q(q2):  # [M, C] -> INT8 Q of B * H heads
            q8 = torch.empty(B * H, Lp, HEAD, dtype=torch.int8, device=dev)
            qs = torch.empty(B * H, Lp // ops.Q_BLOCK, dtype=torch.float32, device=dev)
            for b in range(B):
                ops.sage_quant_int8(q2[b * L:(b + 1) * L].view(L, H, HEAD), ops.Q_BLOCK, premul=ops.q_premul(HEAD),
                                    out=(q8[b * H:(b + 1) * H], qs[b * H:(b + 1) * H]))
            return q8, qs

        def requant_attention_output(o):  # o [L, B, H, 128]: sample b's rows are a strided [L, C] view
            return self._per_sample_quant(B, L, C, lambda b, out: ops.quant_fp8_rowwise(o[:, b].reshape(L, C), out=out))

        # ---- self-attention
        xq, sx = self._per_sample_quant(B, L, C, lambda b, out: ops.adaln_quant_fp8(x[b], e6[0][b:b + 1], e6[1][b:b + 1], self.eps, out=out))
        k8, ks, vt, vs = heads_operands(Lp)
        folded = C % 256 == 0  # norm + RoPE inside the quantisers, as in _self_attention
        if folded:
            qkv, sums = sa.qkv.forward_quantized_rowstats(xq, sx, self.dtype, 2 * C)  # [M, 3C]
            rstd = ops.rowsumsq_to_rstd(sums, C, self.eps)  # [2, M]
            q8 = torch.empty(B * H, Lp, HEAD, dtype=torch.int8, device=dev)
            qs = torch.empty(B * H, Lp // ops.Q_BLOCK, dtype=torch.float32, device=dev)
        else:
            qkv = sa.qkv.forward_quantized(xq, sx, self.dtype)
        for b in range(B):
            rows = qkv[b * L:(b + 1) * L]
            t = rows.view(L, 3, H, HEAD)
            hb = slice(b * H, (b + 1) * H)
            if folded:
                rq, rk = rstd[0, b * L:(b + 1) * L], rstd[1, b * L:(b + 1) * L]
                km = ops.sage_kmean_normed(t[:, 1], sa.norm_k.weight, self.eps, rope, grid, row_rstd=rk)
                ops.sage_quant_int8_normed(t[:, 1], ops.K_BLOCK, sa.norm_k.weight, mean=km, eps=self.eps, rope=rope, grid=grid, row_rstd=rk,
                                           out=(k8[hb], ks[hb]))
                ops.sage_quant_int8_normed(t[:, 0], ops.Q_BLOCK, sa.norm_q.weight, premul=ops.q_premul(HEAD), eps=self.eps, rope=rope,
                                           grid=grid, row_rstd=rq, out=(q8[hb], qs[hb]))
            else:
                km = ops.rmsnorm_rope_inplace(rows[:, C:2 * C], sa.norm_k.weight, self.eps, rope, grid, want_mean=True)
                ops.rmsnorm_rope_inplace(rows[:, :C], sa.norm_q.weight, self.eps, rope, grid)
                ops.sage_quant_int8(t[:, 1], ops.K_BLOCK, mean=km.view(H, HEAD), out=(k8[hb], ks[hb]))
            ops.sage_quant_v(t[:, 2], out=(vt[hb], vs[hb]))
        if not folded:
            q8, qs = quant_q(qkv[:, :C])
        offs, ents, order = self.tile_lists if self.tile_lists is not None else (None, None, None)
        o = torch.empty(L, B, H, HEAD, dtype=self.dtype, device=dev)
        ops.sage_attn_core(q8, qs, k8, ks, vt, vs, L, L, self.dtype, offs, ents, out=o.view(L, B * H, HEAD), tile_order=order)
        aq, sq = requant_attention_output(o)
        x2 = sa.o.forward_quantized(aq, sq, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x2, gate=e6[2])
        # ---- cross-attention
        if self.cross_attn_norm:
            hq, hs = ops.layernorm_quant_fp8(x2, self.norm3.weight, self.norm3.bias, self.eps)
        else:
            hq, hs = ops.quant_fp8_rowwise(x2)
        if folded:
            q, sums = ca.q.forward_quantized_rowstats(hq, hs, self.dtype, C)
            rstd = ops.rowsumsq_to_rstd(sums, C, self.eps)  # [1, M]
        else:
            q = ca.q.forward_quantized(hq, hs, self.dtype)
            ops.rmsnorm_rope_inplace(q, ca.norm_q.weight, self.eps)
        Lc = context.shape[1]
        ck8, cks, cvt, cvs = heads_operands(ops.pad128(Lc))
        for b in range(B):
            kb, sb, vb, vsb, _ = self._context_kv(context[b], context, b)
            for dst, src in ((ck8, kb), (cks, sb), (cvt, vb), (cvs, vsb)):
                dst[b * H:(b + 1) * H].copy_(src)
        if folded:
            for b in range(B):
                ops.sage_quant_int8_normed(q[b * L:(b + 1) * L].view(L, H, HEAD), ops.Q_BLOCK, ca.norm_q.weight, premul=ops.q_premul(HEAD),
                                           eps=self.eps, row_rstd=rstd[0, b * L:(b + 1) * L], out=(q8[b * H:(b + 1) * H], qs[b * H:(b + 1) * H]))
        else:
            q8, qs = quant_q(q)
        ops.sage_attn_core(q8, qs, ck8, cks, cvt, cvs, L, Lc, self.dtype, out=o.view(L, B * H, HEAD))
        oq, os_ = requant_attention_output(o)
        x2 = ca.o.forward_quantized(oq, os_, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x2, gate=self._ones, out=x2)
        # ---- FFN
        xq, sx = self._per_sample_quant(B, L, C, lambda b, out: ops.adaln_quant_fp8(x2[b * L:(b + 1) * L], e6[3][b:b + 1], e6[4][b:b + 1],
                                                                                   self.eps, out=out))
        h = self.ffn[0].forward_quantized(xq, sx, self.dtype, _lib.EPI_GELU_TANH)
        hq, hs = ops.quant_fp8_rowwise(h)
        x2 = self.ffn[2].forward_quantized(hq, hs, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x2, gate=e6[5], out=x2)
        return x2.view(B, L, C)

    # ------------------------------------------------------------------ WanAttentionBlock.forward signature
    def forward(self, x, e, seq_lens=None, grid_sizes=None, freqs=None, context=None, context_lens=None, step_iter=None,
                latent_shape=None, rope_func="default", **_):
        """x [B, L, C]; e [B, 1, 6, C] (or [B, L, 6, C]); grid_sizes [B, 3] (F, H, W); context [B, Lc, C].
        ``freqs`` is accepted for signature compatibility; the rotation table is rebuilt from the same formula:
        the complex one for ``rope_func="default"``, the ComfyUI one (2x2 matrices held in the activation dtype,
        ksana/utils/rope.py:151-212) for a name containing "comfy", as WanModel selects it (wan_model.py:743-755)."""
        if x.dtype != self.dtype:
            raise TypeError(f"block built for {self.dtype}, got {x.dtype}")
        B = x.shape[0]
        if "comfy" in (rope_func or "default"):
            rope = ops.comfy_rope_table(HEAD, 1024, dtype=self.dtype, device=x.device)
        elif rope_func in (None, "default"):
            rope = ops.wan_rope_table(HEAD, 1024, device=x.device)
        else:
            raise _lib.KsanaB200Error(f"unknown rope_func {rope_func!r} (default or comfy)")
        em = (self.modulation.unsqueeze(0) + e) if e.dim() == 4 else (self.modulation + e).unsqueeze(1)  # [B, 1|L, 6, C]
        em = em.to(self.dtype)
        grids = [tuple(int(v) for v in (grid_sizes[b].tolist() if torch.is_tensor(grid_sizes) else grid_sizes[b])) for b in range(len(grid_sizes))]
        if len(grids) == 1 and B > 1:
            grids = grids * B
        if (B > 1 and em.shape[1] == 1 and all(g == grids[0] for g in grids) and self.peer_exchange is None
                and distribute.get_world_size() == 1):
            return self._block_batched(x, em, context, grids[0], rope)
        outs = []
        for b in range(B):  # sequence-parallel runs, per-token modulation and mixed grids: one sample at a time
            e6 = [em[b, :, i].contiguous() for i in range(6)]
            outs.append(self._block_one(x[b], e6, context[b], grids[b], rope, context, b))
        return torch.stack(outs) if B > 1 else outs[0].unsqueeze(0)


class B200WanDenoiseStep(torch.nn.Module):
    """The per-step hot loop of WanModel: ``for block in self.blocks: x = block(x, ...)`` (wan_model.py:785-793)
    over a token shard, for a Wan-shaped stack of blocks.  With a ``step_cache`` (``step_cache.B200DBCache``) the loop
    runs through the cache, which may skip all but the first blocks of a step (ksana/cache/dbcache.py:287-344)."""

    def __init__(self, num_layers, dim, ffn_dim, num_heads, device="cuda", dtype=torch.bfloat16, tile_lists=None, seed=0,
                 cache_context=False, step_cache=None):
        super().__init__()
        self.blocks = torch.nn.ModuleList(
            [B200WanBlock(dim, ffn_dim, num_heads, block_id=i, device=device, dtype=dtype, tile_lists=tile_lists,
                          cache_context=cache_context).random_init(seed + i)
             for i in range(num_layers)]
        )
        self.step_cache = step_cache

    def use_peer_exchange(self, ex):
        """Route every block's Ulysses exchange through ``ex`` (distribute.PeerExchange; None = NCCL all-to-alls)."""
        for blk in self.blocks:
            blk.peer_exchange = ex
        return self

    def forward(self, x, e, grid_sizes, context, phase="cond", step_iter=0, timestep=0):
        if self.step_cache is not None:
            return self.step_cache(phase, x, step_iter, timestep, list(self.blocks), e=e, grid_sizes=grid_sizes, context=context)
        for blk in self.blocks:
            x = blk(x, e, grid_sizes=grid_sizes, context=context)
        return x
