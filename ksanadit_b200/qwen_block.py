"""Qwen-Image dual-stream (MMDiT) block on the B200 kernels: the fused form of
``QwenImageTransformerBlock.forward`` + ``QwenDoubleStreamAttention.forward``.

Same parameters (state-dict names) and inputs as KsanaDiT's block
(ksana/models/qwen/transformer.py:122-241, ksana/models/qwen/attention.py:221-371), run as

  per stream: adaLN+quant -> fused QKV GEMM written straight into the joint [text; image] buffer ->
              per-head RMSNorm + RoPE in place
  joint:      K mean, INT8 Q/K, FP8 V quantisers -> one INT8/FP8 attention over text+image tokens
  per stream: quant -> out-projection GEMM (+ gated residual) -> adaLN+quant -> MLP up GEMM (+GELU-tanh) ->
              quant -> MLP down GEMM (+ gated residual)

Under Ulysses sequence parallelism (a process group is initialised) the image tokens are sharded over the ranks
and the text stream is replicated, as in the reference (qwen/attention.py:283-318, 352-368): the per-head norm and
RoPE run on the local image rows (global positions), one all-to-all brings this rank's heads of all image tokens
next to its slice of the text heads, attention runs over the joint sequence for the local heads, the image rows
go back by the reverse all-to-all and the text rows are all-gathered over heads.
"""

from __future__ import annotations

import torch

from . import _lib, distribute, ops
from .linear import B200Fp8Linear, quantize_weight_per_channel

HEAD = 128


class B200QwenBlock(torch.nn.Module):
    def __init__(self, dim, num_heads, ffn_dim=None, eps=1e-6, device="cuda", dtype=torch.bfloat16, zero_cond_t=False):
        super().__init__()
        self.zero_cond_t = bool(zero_cond_t)
        if dim != num_heads * HEAD:
            raise _lib.KsanaB200Error(f"head size {dim // num_heads} is not supported (only {HEAD})")
        self.dim, self.num_heads, self.eps, self.dtype = dim, num_heads, eps, dtype
        self.ffn_dim = ffn_dim or 4 * dim  # FeedForward(mult=4), qwen/attention.py:191-192
        kw = dict(device=device, dtype=dtype)
        self.img_mod = torch.nn.Sequential(torch.nn.SiLU(), B200Fp8Linear(dim, 6 * dim, **kw))
        self.txt_mod = torch.nn.Sequential(torch.nn.SiLU(), B200Fp8Linear(dim, 6 * dim, **kw))
        self.attn = torch.nn.Module()
        self.attn.to_qkv = B200Fp8Linear(dim, 3 * dim, **kw)
        self.attn.add_qkv_proj = B200Fp8Linear(dim, 3 * dim, **kw)
        self.attn.to_out = torch.nn.ModuleList([B200Fp8Linear(dim, dim, **kw), torch.nn.Identity()])
        self.attn.to_add_out = B200Fp8Linear(dim, dim, **kw)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            m = torch.nn.Module()
            m.weight = torch.nn.Parameter(torch.ones(HEAD, device=device, dtype=torch.float32), requires_grad=False)
            setattr(self.attn, n, m)
        self._mod_fused = None  # (key, weight [12 dim, dim] e4m3, scales, bias) of img_mod | txt_mod, built on first use
        for s in ("img_mlp", "txt_mlp"):
            mlp = torch.nn.Module()
            act = torch.nn.Module()
            act.proj = B200Fp8Linear(dim, self.ffn_dim, **kw)
            mlp.net = torch.nn.ModuleList([act, torch.nn.Identity(), B200Fp8Linear(self.ffn_dim, dim, **kw)])
            setattr(self, s, mlp)

    # ------------------------------------------------------------------ parameters
    def _linears(self):
        return {
            "img_mod.1": self.img_mod[1], "txt_mod.1": self.txt_mod[1], "attn.to_qkv": self.attn.to_qkv,
            "attn.add_qkv_proj": self.attn.add_qkv_proj, "attn.to_out.0": self.attn.to_out[0], "attn.to_add_out": self.attn.to_add_out,
            "img_mlp.net.0.proj": self.img_mlp.net[0].proj, "img_mlp.net.2": self.img_mlp.net[2],
            "txt_mlp.net.0.proj": self.txt_mlp.net[0].proj, "txt_mlp.net.2": self.txt_mlp.net[2],
        }

    @staticmethod
    def _set_linear(lin, w, b, scale=None):
        dev = lin.weight.device
        if w.dtype == torch.float8_e4m3fn:
            wq, s = w, (torch.ones((), dtype=torch.float32) if scale is None else scale.float())
        else:
            wq, s = quantize_weight_per_channel(w.to(dev))
        lin.weight = torch.nn.Parameter(wq.to(dev).contiguous(), requires_grad=False)
        lin.scale_weight = torch.nn.Parameter(s.to(dev), requires_grad=False)
        lin._w_scale_vec = None
        if b is not None:
            lin.bias = torch.nn.Parameter(b.to(dev, lin.compute_dtype), requires_grad=False)

    def load_block_state_dict(self, sd: dict):
        """State dict with QwenImageTransformerBlock's names; separate to_q/to_k/to_v (and add_*_proj) are fused,
        high-precision weights are quantised per output channel."""
        from .fuse_qkv import remap_qkv_weights
        sd = dict(sd)
        dev = self.attn.norm_q.weight.device
        for names in (("attn.to_q", "attn.to_k", "attn.to_v"), ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj")):
            if names[0] + ".weight" in sd and sd[names[0] + ".weight"].dtype != torch.float8_e4m3fn:
                for n in names:
                    wq, s = quantize_weight_per_channel(sd[n + ".weight"].to(dev))
                    sd[n + ".weight"], sd[n + ".scale_weight"] = wq, s
        remap_qkv_weights(sd, [("attn.to_q", "attn.to_k", "attn.to_v", "attn.to_qkv"),
                               ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj", "attn.add_qkv_proj")])
        for name, lin in self._linears().items():
            self._set_linear(lin, sd[name + ".weight"], sd.get(name + ".bias"), sd.get(name + ".scale_weight"))
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            getattr(self.attn, n).weight = torch.nn.Parameter(sd[f"attn.{n}.weight"].float().to(dev).contiguous(), requires_grad=False)
        return self

    def random_init(self, seed: int, std: float = 0.02):
        dev = self.attn.norm_q.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        for lin in self._linears().values():
            w = (torch.randn(lin.out_features, lin.in_features, device=dev, generator=g) * std).to(self.dtype)
            b = (torch.randn(lin.out_features, device=dev, generator=g) * std).to(self.dtype)
            self._set_linear(lin, w, b)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            getattr(self.attn, n).weight = torch.nn.Parameter((1 + 0.1 * torch.randn(HEAD, device=dev, generator=g)).float(), requires_grad=False)
        return self

    # ------------------------------------------------------------------ forward
    def _norm_weight(self, name):
        """fp32 [128] weight of one of the four per-head RMSNorms."""
        return getattr(self.attn, name).weight

    _rotary_tables = None  # (key, image table, text table) built from a caller's rotary embeddings

    def _tables_from_rotary(self, image_rotary_emb):
        """Rotation tables from the reference's own ``image_rotary_emb = (vid_freqs, txt_freqs)`` (complex [L, 64], one row
        per token: QwenEmbedRope.forward, qwen/attention.py:113-142): row t of a table is token t's (cos, sin) pairs, read
        with one position for all axes."""
        vf, tf = image_rotary_emb
        key = (vf.data_ptr(), tf.data_ptr(), tuple(vf.shape), tuple(tf.shape))
        if self._rotary_tables is None or self._rotary_tables[0] != key:
            tabs = []
            for f in (vf, tf):
                if not f.is_complex() or f.shape[-1] != HEAD // 2:
                    raise _lib.KsanaB200Error("image_rotary_emb must hold complex [L, 64] tensors")
                tabs.append(torch.view_as_real(f.reshape(-1, HEAD // 2)).to(torch.float32).contiguous())
            self._rotary_tables = (key, tabs[0], tabs[1])
        return (self._rotary_tables[1], 0, 0), (self._rotary_tables[2], 0, 0)

    def _modulation(self, st, quantized=None, out=None):
        """img_mod and txt_mod (transformer.py:204-211) as ONE GEMM: both are Linears of the same one-row input, and at
        one row a GEMM only streams its weight, so two launches cost twice the fixed part.  The two weights are
        concatenated once; the modules' own parameters become views of the concatenation (no second copy).
        ``quantized``: (xq, sx) of ``st`` when the caller has quantised it already (the same rows feed every block);
        ``out``: a [rows, 12 C] buffer to write."""
        im, tm = self.img_mod[1], self.txt_mod[1]
        key = (im.weight.data_ptr(), tm.weight.data_ptr(), im.scale_weight.data_ptr(), tm.scale_weight.data_ptr())
        if self._mod_fused is None or self._mod_fused[0] != key:
            w = torch.cat([im.weight.data, tm.weight.data], dim=0).contiguous()
            sc = torch.cat([im.weight_scale_vector(), tm.weight_scale_vector()]).contiguous()
            b = torch.cat([im.bias.data, tm.bias.data]).contiguous() if im.bias is not None else None
            n = im.out_features
            im.weight.data, tm.weight.data = w[:n], w[n:]
            key = (im.weight.data_ptr(), tm.weight.data_ptr(), im.scale_weight.data_ptr(), tm.scale_weight.data_ptr())
            self._mod_fused = (key, w, sc, b)
        _, w, sc, b = self._mod_fused
        xq, sx = quantized if quantized is not None else ops.quant_fp8_rowwise(st)
        return ops.fp8_gemm(xq, sx, w, sc, b, out_dtype=self.dtype, out=out)

    def _stream_tail(self, x, attn_out, gate1, mod2, out_lin, mlp):
        """x + gate1 * out(attn_out), then x + gate2 * mlp(modulate(LN(x)))  (transformer.py:225-234)."""
        aq, sa = ops.quant_fp8_rowwise(attn_out)
        x = out_lin.forward_quantized(aq, sa, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x, gate=gate1)
        shift2, scale2, gate2 = mod2
        xq, sx = ops.adaln_quant_fp8(x, shift2, scale2, self.eps, round_product=True)
        h = mlp.net[0].proj.forward_quantized(xq, sx, self.dtype, _lib.EPI_GELU_TANH)
        hq, hs = ops.quant_fp8_rowwise(h)
        return mlp.net[2].forward_quantized(hq, hs, self.dtype, _lib.EPI_GATE_RESIDUAL, resid=x, gate=gate2, out=x)

    def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None, img_grid=None, modulate_index=None, mods=None,
                side_stream=None, **_):
        """hidden_states [1, Li, C] (image; under sequence parallelism this rank's Li rows of the P * Li image
        tokens, rows past the grid being padding), encoder_hidden_states [1, Lt, C] (text, replicated),
        temb [1, C]; img_grid (F, H, W) of all image tokens.  Returns (text, image) like the reference block.
        ``image_rotary_emb`` is accepted for signature compatibility; the rotation tables are rebuilt from the
        same formula (QwenEmbedRope) for ``img_grid`` and the text length.

        ``zero_cond_t`` blocks (transformer.py:171-188,206-208) take temb [2, C] = [real timestep; zero timestep]
        and ``modulate_index`` [1, Li] in {0, 1}: every image token reads its shift / scale / gate from the row
        its index names (the kernels take one modulation row per token), the text stream uses row 0.

        ``mods``: this block's modulation rows [rows, 12 C] when the caller has computed them ahead (``B200QwenDenoiseStep``).
        ``side_stream``: a CUDA stream for the text stream's kernels: its few-tile GEMMs and row passes then fill the
        idle SMs at the ends of the image stream's launches instead of running alone (under sequence parallelism the
        text stream is replicated and as large as a rank's share of the image stream; the collectives stay on the
        caller's stream)."""
        if hidden_states.shape[0] != 1:
            raise _lib.KsanaB200Error("batch 1 only")
        if img_grid is None and image_rotary_emb is None:
            raise ValueError("img_grid=(F, H, W) or image_rotary_emb is required")
        img, txt = hidden_states[0], encoder_hidden_states[0]
        Li, C = img.shape  # local image rows
        Lt = txt.shape[0]
        H = self.num_heads
        P, rank = distribute.get_world_size(), distribute.get_rank_id()
        if H % P != 0:
            raise _lib.KsanaB200Error(f"{H} heads cannot be split over {P} ranks")
        Hl = H // P
        if img_grid is not None:
            img_tab, txt_tab = ops.qwen_rope_tables(img_grid, Lt, device=img.device)
            img_rope = (img_grid, False)
        else:  # per-token rows taken from the caller's embeddings: one running position, rank r starts at its first row
            img_tab, txt_tab = self._tables_from_rotary(image_rotary_emb)
            if img_tab[0].shape[0] < P * Li or txt_tab[0].shape[0] < Lt:
                raise _lib.KsanaB200Error("image_rotary_emb is shorter than the token sequences")
            img_rope = ((img_tab[0].shape[0], 1, 1), True)
        if temb.shape[0] != (2 if self.zero_cond_t else 1) or (modulate_index is not None) != self.zero_cond_t:
            raise _lib.KsanaB200Error("a zero_cond_t block takes temb [2, C] and a modulate_index; any other block temb [1, C] and none")
        if mods is None:
            mods = self._modulation(torch.nn.functional.silu(temb))  # [rows, 12 C]: image then text, each [mod1|mod2] x [shift|scale|gate]
        elif mods.shape != (temb.shape[0], 12 * C):
            raise _lib.KsanaB200Error(f"mods must be [{temb.shape[0]}, {12 * C}]")
        if self.zero_cond_t:
            index = modulate_index.reshape(-1).to(img.device, torch.int64)
            if index.numel() != Li:
                raise _lib.KsanaB200Error(f"modulate_index must name a row for each of the {Li} image tokens")
            imod = mods[:, :6 * C].reshape(2, 2, 3, C).permute(1, 2, 0, 3).index_select(2, index)  # [2, 3, Li, C]
        else:
            imod = mods[0, :6 * C].view(2, 3, 1, C)
        tmod = mods[0, 6 * C:].view(2, 3, 1, C)

        # local projections: text rows first (attention.py:355-357), then this rank's image rows
        qkv = torch.empty(Lt + Li, 3 * C, dtype=self.dtype, device=img.device)
        a = self.attn
        main = torch.cuda.current_stream()
        side = side_stream  # the text stream's own kernels only: every collective stays on the main stream

        def on_text_stream(fn, after):
            """Runs fn on the text stream once ``after`` (an event of the main stream) has passed; returns its result and
            the event that marks its end.  Without a text stream fn simply runs here."""
            if side is None:
                return fn(), None
            with torch.cuda.stream(side):
                side.wait_event(after)
                r = fn()
                done = torch.cuda.Event()
                done.record(side)
            return r, done

        def project(x, mod, lin, nq, nk, rows, tab, grid, diag, pos0):
            xq, sx = ops.adaln_quant_fp8(x, mod[0, 0], mod[0, 1], self.eps, round_product=True)
            lin.forward_quantized(xq, sx, self.dtype, out=qkv[rows])
            ops.rmsnorm_rope_inplace(qkv[rows, :C], self._norm_weight(nq), self.eps, tab, grid, per_head=True, diag=diag, pos0=pos0)
            ops.rmsnorm_rope_inplace(qkv[rows, C:2 * C], self._norm_weight(nk), self.eps, tab, grid, per_head=True, diag=diag, pos0=pos0)

        start = None
        if side is not None:
            start = torch.cuda.Event()
            start.record(main)  # qkv, mods and both inputs are ready (in stream order) from here on
        _, txt_projected = on_text_stream(lambda: project(txt, tmod, a.add_qkv_proj, "norm_added_q", "norm_added_k", slice(0, Lt), txt_tab,
                                                          (txt_tab[0].shape[0] if img_grid is None else Lt, 1, 1), True, 0), start)
        project(img, imod, a.to_qkv, "norm_q", "norm_k", slice(Lt, Lt + Li), img_tab, img_rope[0], img_rope[1], rank * Li)
        if txt_projected is not None:
            main.wait_event(txt_projected)
        if P == 1:
            t = qkv.view(Lt + Li, 3, H, HEAD)
            o = ops.sage_attention(t[:, 0], t[:, 1], t[:, 2]).view(Lt + Li, C)
            o_txt, o_img = o[:Lt], o[Lt:]
        else:
            # joint [text; all image tokens] x this rank's heads
            joint = torch.empty(Lt + P * Li, 3, Hl, HEAD, dtype=self.dtype, device=img.device)
            joint[:Lt] = qkv[:Lt].view(Lt, 3, H, HEAD)[:, :, rank * Hl:(rank + 1) * Hl]
            distribute.heads_to_sequence(qkv[Lt:].view(Li, 3, H, HEAD), out=joint[Lt:])
            o = ops.sage_attention(joint[:, 0], joint[:, 1], joint[:, 2])  # [Lt + P*Li, Hl, D]
            o_txt = distribute.gather_heads(o[:Lt]).reshape(Lt, C)
            o_img = distribute.sequence_to_heads(o[Lt:]).reshape(Li, C)
        attended = None
        if side is not None:
            attended = torch.cuda.Event()
            attended.record(main)
        txt, txt_done = on_text_stream(lambda: self._stream_tail(txt, o_txt, tmod[0, 2], tmod[1], a.to_add_out, self.txt_mlp), attended)
        img = self._stream_tail(img, o_img, imod[0, 2], imod[1], a.to_out[0], self.img_mlp)
        if txt_done is not None:
            main.wait_event(txt_done)  # everything this block launched is ordered before whatever follows on this stream
        if self.dtype == torch.float16:  # transformer.py:236-239: an overflow to inf comes back as the largest fp16
            txt, img = txt.clamp_(-65504, 65504), img.clamp_(-65504, 65504)
        return txt.unsqueeze(0), img.unsqueeze(0)


class B200QwenDenoiseStep(torch.nn.Module):
    """The per-step loop over the dual-stream blocks (``for block in self.transformer_blocks``,
    ksana/models/qwen/transformer.py:196-241 called once per block) with the two things a block cannot do on its own:

    * every block's modulation rows depend on the timestep embedding only, and computing them streams 12 C x C weights
      per block through a one-row GEMM: they are all launched at the start of the step on a stream of their own, so
      the weight streaming hides under the first blocks' tensor-core work;
    * ``text_stream=True`` (used on one or two ranks): the text stream's kernels of every block run on a second stream
      beside the image stream's (see ``B200QwenBlock.forward``).

    The caller's stream waits for both before this returns, and the step can be captured into a CUDA graph."""

    def __init__(self, blocks, text_stream=True):
        super().__init__()
        self.blocks = torch.nn.ModuleList(blocks)
        self.text_stream = text_stream
        self._streams = None

    def _side_streams(self, device):
        if self._streams is None or self._streams[0].device != device:
            self._streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        return self._streams

    def forward(self, hidden_states, encoder_hidden_states, temb, img_grid=None, image_rotary_emb=None, modulate_index=None):
        img, txt = hidden_states, encoder_hidden_states
        main = torch.cuda.current_stream()
        mod_stream, txt_stream = self._side_streams(img.device)
        b0 = self.blocks[0]
        C = b0.dim
        st = torch.nn.functional.silu(temb)
        quantized = ops.quant_fp8_rowwise(st)
        mods = torch.empty(len(self.blocks), temb.shape[0], 12 * C, dtype=b0.dtype, device=img.device)
        ready = torch.cuda.Event()
        ready.record(main)
        events = []
        with torch.cuda.stream(mod_stream):
            mod_stream.wait_event(ready)
            for i, blk in enumerate(self.blocks):
                blk._modulation(st, quantized=quantized, out=mods[i])
                ev = torch.cuda.Event()
                ev.record(mod_stream)
                events.append(ev)
        # with four or more ranks a rank's kernels are so short (862 - 1723 image rows) that the step is bound by the
        # host's launch rate, and the extra events and stream switches cost more than the overlap gives
        # (8 ranks: 68.4 against 65.3 ms; 2 ranks: 71.4 against 77.0 ms; 1 rank: 96.7 against 102.4 ms)
        side = txt_stream if (self.text_stream and distribute.get_world_size() <= 2) else None
        for i, blk in enumerate(self.blocks):
            main.wait_event(events[i])
            txt, img = blk(img, txt, temb, image_rotary_emb=image_rotary_emb, img_grid=img_grid, modulate_index=modulate_index,
                           mods=mods[i], side_stream=side)
        if side is not None:
            txt.record_stream(main)  # allocated on the text stream, handed to the caller's stream
        return txt, img
