"""Functional wrappers: torch CUDA tensors in, torch CUDA tensors out, every kernel through the C ABI.

torch is used for device memory and streams only.  Nothing here computes on the CPU or falls back to
a PyTorch implementation.
"""

from __future__ import annotations

import torch

from . import _lib

Q_BLOCK, K_BLOCK, KV_TILE = 128, 64, 128
LOG2E = 1.4426950408889634


class LaunchStats:
    """Counts the CUDA kernels this library launches and, when ``timing`` is on, brackets every call of a
    chosen entry point with CUDA events on the launching stream (used by the benchmark's roofline)."""

    def __init__(self):
        self.kernels = 0
        self.timing = False
        self.events: dict = {}

    def reset(self):
        self.kernels = 0
        self.events = {}

    def count(self, n):
        self.kernels += n

    def timed(self, tag, fn):
        if not self.timing:
            return fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        self.events.setdefault(tag, []).append((a, b))
        return r

    def summary(self):
        """tag -> (launches, total ms); call after a synchronize."""
        return {t: (len(ev), sum(a.elapsed_time(b) for a, b in ev)) for t, ev in self.events.items()}


STATS = LaunchStats()


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    if t.dtype == torch.float16:
        return _lib.FP16
    raise TypeError(f"expected bfloat16 or float16, got {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.KsanaB200Error("ksanadit_b200 kernels need CUDA tensors (no CPU path exists)")


def pad128(n: int) -> int:
    return (n + 127) // 128 * 128


# ----------------------------------------------------------------------------- FP8 Linear pieces


def _quant_out(out, M, K, device):
    """(q [M,K] e4m3, s [M] fp32): fresh tensors, or the caller's (row slices of a larger batch buffer) after a shape check."""
    if out is None:
        return torch.empty(M, K, dtype=torch.float8_e4m3fn, device=device), torch.empty(M, dtype=torch.float32, device=device)
    q, s = out
    if q.shape != (M, K) or s.shape != (M,) or q.dtype != torch.float8_e4m3fn or s.dtype != torch.float32 or not q.is_contiguous() or not s.is_contiguous():
        raise _lib.KsanaB200Error(f"out must be a contiguous ([{M}, {K}] float8_e4m3fn, [{M}] float32) pair")
    _cuda(q, s)
    return q, s


def quant_fp8_rowwise(x: torch.Tensor, out=None):
    """x [M,K] half (row stride allowed) -> (q [M,K] float8_e4m3fn, scale [M] fp32)."""
    _cuda(x)
    assert x.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    q, s = _quant_out(out, M, K, x.device)
    _lib.check(_lib.load().ksb_quant_fp8_rowwise(_p(x), _dt(x), M, K, x.stride(0) if M > 1 else K, _p(q), _p(s), _stream()),
               "ksb_quant_fp8_rowwise")
    STATS.count(1)
    return q, s


def quant_fp8_static(x: torch.Tensor, scale_input: torch.Tensor | None):
    _cuda(x, scale_input)
    assert x.dim() == 2 and x.stride(1) == 1
    M, K = x.shape
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(M, dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().ksb_quant_fp8_static(_p(x), _dt(x), M, K, x.stride(0) if M > 1 else K, _p(scale_input), _p(q), _p(s),
                                                _stream()), "ksb_quant_fp8_static")
    STATS.count(1)
    return q, s


def adaln_quant_fp8(x, shift, scale, eps=1e-6, want_h=False, round_product=False, out=None):
    """h = shift + LN(x)*(1+scale) -> per-token FP8.  x [M,K]; shift/scale [1,K] or [M,K].
    round_product: round LN(x)*(1+scale) to half before adding shift (the Qwen-Image block's eager order)."""
    _cuda(x, shift, scale)
    M, K = x.shape
    shift = shift.reshape(-1, K).contiguous()
    scale = scale.reshape(-1, K).contiguous()
    assert shift.shape == scale.shape and shift.dtype == x.dtype == scale.dtype
    q, s = _quant_out(out, M, K, x.device)
    h = torch.empty(M, K, dtype=x.dtype, device=x.device) if want_h else None
    _lib.check(_lib.load().ksb_adaln_quant_fp8(_p(x), _dt(x), M, K, x.stride(0) if M > 1 else K, _p(shift), _p(scale),
                                               shift.shape[0], int(round_product), float(eps), _p(h), _p(q), _p(s), _stream()),
               "ksb_adaln_quant_fp8")
    STATS.count(1)
    return (q, s, h) if want_h else (q, s)


def layernorm_quant_fp8(x, w, b, eps=1e-6, want_h=False):
    _cuda(x, w, b)
    M, K = x.shape
    w = w.float().contiguous()
    b = None if b is None else b.float().contiguous()
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(M, dtype=torch.float32, device=x.device)
    h = torch.empty(M, K, dtype=x.dtype, device=x.device) if want_h else None
    _lib.check(_lib.load().ksb_layernorm_quant_fp8(_p(x), _dt(x), M, K, x.stride(0) if M > 1 else K, _p(w), _p(b), float(eps),
                                                   _p(h), _p(q), _p(s), _stream()), "ksb_layernorm_quant_fp8")
    STATS.count(1)
    return (q, s, h) if want_h else (q, s)


def fp8_gemm(a_q, a_scale, w_q, w_scale, bias=None, out_dtype=torch.bfloat16, epilogue=_lib.EPI_NONE, resid=None, gate=None,
             out=None):
    """out[M,N] = epi((a_q @ w_q.T) * a_scale[:,None] * w_scale[None,:] + bias)."""
    _cuda(a_q, a_scale, w_q, w_scale, bias, resid, gate, out)
    M, K = a_q.shape
    N = w_q.shape[0]
    assert w_q.shape[1] == K and a_q.is_contiguous() and w_q.is_contiguous()
    assert a_scale.dtype == torch.float32 and w_scale.dtype == torch.float32 and a_scale.numel() == M and w_scale.numel() == N
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    dt = _lib.BF16 if out.dtype == torch.bfloat16 else _lib.FP16
    if bias is not None:
        bias = bias.to(out.dtype).contiguous()
    ldr, gate_rows = 0, 0
    if epilogue == _lib.EPI_GATE_RESIDUAL:
        assert resid is not None and gate is not None and resid.dtype == out.dtype
        gate = gate.reshape(-1, N).to(out.dtype).contiguous()
        gate_rows = gate.shape[0]
        ldr = resid.stride(0) if M > 1 else N
    STATS.timed(("gemm", M, N, K), lambda: _lib.check(
        _lib.load().ksb_fp8_gemm(_p(a_q), _p(a_scale), _p(w_q), _p(w_scale), _p(bias), M, N, K, _p(out), dt,
                                 out.stride(0) if M > 1 else N, epilogue, _p(resid), ldr, _p(gate), gate_rows, _stream()),
        "ksb_fp8_gemm"))
    STATS.count(1)
    return out


def _ptr_array(ptrs):
    """Host array of device pointers for the C ABI (kept alive by the caller for the duration of the call)."""
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*[int(v) for v in ptrs])


def fp8_gemm_qkv_scatter(a_q, a_scale, w_q, w_scale, bias, heads, peer_ptrs, rank, tile_sumsq, dtype=torch.bfloat16):
    """Fused QKV projection whose epilogue stores every element into the [P*M, 3, heads/P, 128] buffer of the GPU
    that owns its head (``peer_ptrs``: device addresses of those buffers, own one included) and leaves per-tile
    row sums of squares of the Q and K thirds in ``tile_sumsq`` ([2*C/256, M] fp32)."""
    _cuda(a_q, a_scale, w_q, w_scale, bias, tile_sumsq)
    M, K = a_q.shape
    C = w_q.shape[0] // 3
    assert w_q.shape == (3 * C, K) and a_q.is_contiguous() and w_q.is_contiguous() and C == heads * 128
    assert tile_sumsq.dtype == torch.float32 and tile_sumsq.numel() >= 2 * (C // 256) * M and tile_sumsq.is_contiguous()
    dt = _lib.BF16 if dtype == torch.bfloat16 else _lib.FP16
    if bias is not None:
        bias = bias.to(dtype).contiguous()
    arr = _ptr_array(peer_ptrs)
    STATS.timed(("gemm", M, 3 * C, K), lambda: _lib.check(
        _lib.load().ksb_fp8_gemm_qkv_scatter(_p(a_q), _p(a_scale), _p(w_q), _p(w_scale), _p(bias), M, C, K, dt, arr, len(peer_ptrs),
                                             int(rank), heads, _p(tile_sumsq), _stream()),
        "ksb_fp8_gemm_qkv_scatter"))
    STATS.count(1)


def rowsumsq_to_rstd_scatter(tile_sumsq, M, C, eps, peer_ptrs, rank):
    """rstd of the full-width RMSNorm of Q and K from the tile sums above, stored into every peer's [2, P*M] table."""
    _cuda(tile_sumsq)
    arr = _ptr_array(peer_ptrs)
    _lib.check(_lib.load().ksb_rowsumsq_to_rstd_scatter(_p(tile_sumsq), M, C, float(eps), arr, len(peer_ptrs), int(rank), _stream()),
               "ksb_rowsumsq_to_rstd_scatter")
    STATS.count(1)


def gate_residual(x, y, gate):
    _cuda(x, y, gate)
    M, N = x.shape
    gate = gate.reshape(-1, N).to(x.dtype).contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.load().ksb_gate_residual(_p(x.contiguous()), _p(y.contiguous()), _p(gate), gate.shape[0], _p(out), _dt(x), M, N,
                                             _stream()), "ksb_gate_residual")
    STATS.count(1)
    return out


def residual_diff(x_new, x_old, prev=None, want_residual=True):
    """r = x_new - x_old (rounded to the activation dtype) and the fp32 sums [sum |r - prev|, sum |r|, sum |prev|]
    (a device tensor of 3 floats) in one pass -- the reductions the block-level step cache decides on."""
    _cuda(x_new, x_old, prev)
    assert x_new.shape == x_old.shape and x_new.dtype == x_old.dtype and x_new.is_contiguous() and x_old.is_contiguous()
    assert prev is None or (prev.shape == x_new.shape and prev.dtype == x_new.dtype and prev.is_contiguous())
    res = torch.empty_like(x_new) if want_residual else None
    sums = torch.empty(3, dtype=torch.float32, device=x_new.device)
    _lib.check(_lib.load().ksb_residual_diff(_p(x_new), _p(x_old), _p(prev), _p(res), _p(sums), _dt(x_new), x_new.numel(), _stream()),
               "ksb_residual_diff")
    STATS.count(1)
    return res, sums


# ----------------------------------------------------------------------------- Sage attention pieces


def _lhd(x):
    """[L,H,D] view with D contiguous -> (L,H,D, token_stride, head_stride)."""
    assert x.dim() == 3 and x.stride(2) == 1
    return x.shape[0], x.shape[1], x.shape[2], x.stride(0), x.stride(1)


def sage_kmean(k):
    _cuda(k)
    L, H, D, ts, hs = _lhd(k)
    lib = _lib.load()
    partial = torch.empty(lib.ksb_sage_kmean_scratch_floats(L, H, D), dtype=torch.float32, device=k.device)
    km = torch.empty(H, D, dtype=torch.float32, device=k.device)
    _lib.check(lib.ksb_sage_kmean(_p(k), _dt(k), L, H, D, ts, hs, _p(partial), _p(km), _stream()), "ksb_sage_kmean")
    STATS.count(2)
    return km


def sage_quant_int8(x, block, premul=0.0, mean=None, out=None):
    """x [L,H,128] -> (int8 [H,Lpad,128], scale [H, Lpad/block]).  out: that pair, preallocated (e.g. the head slots of
    one sample inside the operands of a batched attention launch)."""
    _cuda(x, mean)
    L, H, D, ts, hs = _lhd(x)
    Lp = pad128(L)
    if out is None:
        out = torch.empty(H, Lp, D, dtype=torch.int8, device=x.device)
        sc = torch.empty(H, Lp // block, dtype=torch.float32, device=x.device)
    else:
        out, sc = out
        if out.shape != (H, Lp, D) or sc.shape != (H, Lp // block) or out.dtype != torch.int8 or sc.dtype != torch.float32 \
                or not out.is_contiguous() or not sc.is_contiguous():
            raise _lib.KsanaB200Error(f"out must be a contiguous ([{H}, {Lp}, {D}] int8, [{H}, {Lp // block}] float32) pair")
        _cuda(out, sc)
    _lib.check(_lib.load().ksb_sage_quant_int8(_p(x), _dt(x), L, H, D, ts, hs, block, float(premul), _p(mean), _p(out), _p(sc),
                                               _stream()), "ksb_sage_quant_int8")
    STATS.count(1)
    return out, sc


def fp8_gemm_rowstats(a_q, a_scale, w_q, w_scale, bias, sumsq_cols, out_dtype=torch.bfloat16, out=None):
    """fp8_gemm without epilogue that also returns tile_sumsq [sumsq_cols / 256, M] fp32: per 256-column tile and row, the
    sum of squares of the rounded outputs (the row statistics an RMSNorm over those columns needs)."""
    _cuda(a_q, a_scale, w_q, w_scale, bias, out)
    M, K = a_q.shape
    N = w_q.shape[0]
    assert w_q.shape[1] == K and a_q.is_contiguous() and w_q.is_contiguous()
    assert a_scale.dtype == torch.float32 and w_scale.dtype == torch.float32 and a_scale.numel() == M and w_scale.numel() == N
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    dt = _lib.BF16 if out.dtype == torch.bfloat16 else _lib.FP16
    if bias is not None:
        bias = bias.to(out.dtype).contiguous()
    sums = torch.empty(sumsq_cols // 256, M, dtype=torch.float32, device=a_q.device)
    STATS.timed(("gemm", M, N, K), lambda: _lib.check(
        _lib.load().ksb_fp8_gemm_rowstats(_p(a_q), _p(a_scale), _p(w_q), _p(w_scale), _p(bias), M, N, K, _p(out), dt,
                                          out.stride(0) if M > 1 else N, _p(sums), int(sumsq_cols), _stream()),
        "ksb_fp8_gemm_rowstats"))
    STATS.count(1)
    return out, sums


def rowsumsq_to_rstd(tile_sumsq, C, eps=1e-6):
    """tile_sumsq [groups * C / 256, M] -> rstd [groups, M] = rsqrt(mean of squares over the C channels of a group + eps)."""
    _cuda(tile_sumsq)
    tiles, M = tile_sumsq.shape
    assert tile_sumsq.dtype == torch.float32 and tile_sumsq.is_contiguous() and C % 256 == 0 and tiles % (C // 256) == 0
    groups = tiles // (C // 256)
    rstd = torch.empty(groups, M, dtype=torch.float32, device=tile_sumsq.device)
    _lib.check(_lib.load().ksb_rowsumsq_to_rstd(_p(tile_sumsq), M, C, groups, float(eps), _p(rstd), _stream()), "ksb_rowsumsq_to_rstd")
    STATS.count(1)
    return rstd


def _norm_args(x, w, eps, rope, grid, pos0, per_head, diag, row_rstd):
    L, H = x.shape[0], x.shape[1]
    _cuda(w, row_rstd)
    assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == (128 if per_head else H * 128)
    if not per_head:
        assert row_rstd is not None and row_rstd.dtype == torch.float32 and row_rstd.is_contiguous() and row_rstd.numel() == L
    tab, tlen, nf, nh, F, Hh, Ww = None, 0, 0, 0, 1, 1, 1
    if rope is not None:
        tab, nf, nh = rope
        tlen = tab.shape[0]
        F, Hh, Ww = (int(v) for v in grid)
    return (_p(w), int(per_head), None if per_head else _p(row_rstd), float(eps), _p(tab), tlen, nf, nh, F, Hh, Ww, int(pos0), int(diag))


def sage_kmean_normed(k, w, eps=1e-6, rope=None, grid=None, pos0=0, per_head=False, diag=False, row_rstd=None):
    """Column means [H,128] of rope(rmsnorm(k)) for k [L,H,128], without writing the normalised tensor (the arguments
    are those of rmsnorm_rope_inplace; row_rstd [L] is required unless per_head)."""
    _cuda(k)
    L, H, D, ts, hs = _lhd(k)
    lib = _lib.load()
    partial = torch.empty(lib.ksb_sage_kmean_scratch_floats(L, H, D), dtype=torch.float32, device=k.device)
    km = torch.empty(H, D, dtype=torch.float32, device=k.device)
    _lib.check(lib.ksb_sage_kmean_normed(_p(k), _dt(k), L, H, D, ts, hs, *_norm_args(k, w, eps, rope, grid, pos0, per_head, diag, row_rstd),
                                         _p(partial), _p(km), _stream()), "ksb_sage_kmean_normed")
    STATS.count(2)
    return km


def sage_quant_int8_normed(x, block, w, premul=0.0, mean=None, eps=1e-6, rope=None, grid=None, pos0=0, per_head=False, diag=False,
                           row_rstd=None, out=None):
    """sage_quant_int8 of rope(rmsnorm(x)) for x [L,H,128], reading x once and never writing the normalised tensor."""
    _cuda(x, mean)
    L, H, D, ts, hs = _lhd(x)
    Lp = pad128(L)
    if out is None:
        out = torch.empty(H, Lp, D, dtype=torch.int8, device=x.device)
        sc = torch.empty(H, Lp // block, dtype=torch.float32, device=x.device)
    else:
        out, sc = out
        if out.shape != (H, Lp, D) or sc.shape != (H, Lp // block) or out.dtype != torch.int8 or sc.dtype != torch.float32 \
                or not out.is_contiguous() or not sc.is_contiguous():
            raise _lib.KsanaB200Error(f"out must be a contiguous ([{H}, {Lp}, {D}] int8, [{H}, {Lp // block}] float32) pair")
        _cuda(out, sc)
    _lib.check(_lib.load().ksb_sage_quant_int8_normed(_p(x), _dt(x), L, H, D, ts, hs, block, float(premul), _p(mean),
                                                      *_norm_args(x, w, eps, rope, grid, pos0, per_head, diag, row_rstd),
                                                      _p(out), _p(sc), _stream()), "ksb_sage_quant_int8_normed")
    STATS.count(1)
    return out, sc


def sage_quant_v(v, out=None):
    """v [L,H,128] -> (vt [H,128,Lpad] float8_e4m3fn, vs [H,128]).  out: that pair, preallocated."""
    _cuda(v)
    L, H, D, ts, hs = _lhd(v)
    Lp = pad128(L)
    amax = torch.empty(H * D, dtype=torch.float32, device=v.device)
    if out is None:
        vt = torch.empty(H, D, Lp, dtype=torch.float8_e4m3fn, device=v.device)
        vs = torch.empty(H, D, dtype=torch.float32, device=v.device)
    else:
        vt, vs = out
        if vt.shape != (H, D, Lp) or vs.shape != (H, D) or vt.dtype != torch.float8_e4m3fn or vs.dtype != torch.float32 \
                or not vt.is_contiguous() or not vs.is_contiguous():
            raise _lib.KsanaB200Error(f"out must be a contiguous ([{H}, {D}, {Lp}] float8_e4m3fn, [{H}, {D}] float32) pair")
        _cuda(vt, vs)
    _lib.check(_lib.load().ksb_sage_quant_v_fp8(_p(v), _dt(v), L, H, D, ts, hs, _p(amax), _p(vt), _p(vs), _stream()),
               "ksb_sage_quant_v_fp8")
    STATS.count(2)
    return vt, vs


def q_premul(head_dim: int, sm_scale: float | None = None) -> float:
    sc = head_dim ** -0.5 if sm_scale is None else sm_scale
    return float(torch.tensor(sc * LOG2E, dtype=torch.float64).to(torch.float32))


_PAIR_LISTS: dict = {}
# A pair of Q blocks walks the union of its two lists, so pairing only pays while the union is barely longer than the
# lists themselves: sharing the K / V tiles is worth ~8 %.  Measured at 75 600 tokens: the radial mask's unions are
# 11 % longer and a mask with independent random tiles per block 43 % (18.8 ms against 11.4 ms): both stay on the
# one-block kernel.
PAIR_LIST_MAX_OVERHEAD = 1.03


def _pair_lists(tile_offsets, tile_entries, want_order):
    """Per-pair tile lists (radial_mask.pair_tile_lists) of the given per-block lists, or None when walking the unions
    would cost more than sharing the tiles saves.  Built once per list object on the host (one device -> host copy)
    and kept on the device: masks are built once per shape and reused every step.  The cache holds the source
    tensors, so their addresses cannot be handed to other tensors while the entry lives."""
    from . import radial_mask
    key = (tile_offsets.data_ptr(), tile_entries.data_ptr(), tile_offsets._version, tile_entries._version, tile_offsets.numel(),
           tile_entries.numel())
    hit = _PAIR_LISTS.get(key)
    if hit is None:
        if len(_PAIR_LISTS) >= 64:
            _PAIR_LISTS.clear()
        offs, ents = tile_offsets.cpu().numpy(), tile_entries.cpu().numpy()
        n_real = int(offs[-1])
        po, pe = radial_mask.pair_tile_lists(offs, ents[:n_real])
        if n_real == 0 or 2 * pe.size > PAIR_LIST_MAX_OVERHEAD * n_real:
            hit = (tile_offsets, tile_entries, None, None, None)
        else:
            order = radial_mask.longest_first_order(po)
            dev = tile_offsets.device
            hit = (tile_offsets, tile_entries, torch.from_numpy(po).to(dev), torch.from_numpy(pe).to(dev), torch.from_numpy(order).to(dev))
        _PAIR_LISTS[key] = hit
    if hit[2] is None:
        return None
    return hit[2], hit[3], (hit[4] if want_order else None)


def sage_attn_core(q8, qs, k8, ks, vt, vs, Lq, Lk, out_dtype=torch.bfloat16, tile_offsets=None, tile_entries=None, out=None,
                   tile_order=None, peer_out=None):
    """Quantised operands -> out [Lq, H, 128].

    peer_out = (ptrs, rows_per_peer, token_stride, head_stride): instead of ``out``, row l is stored at row
    l % rows_per_peer of the buffer at ptrs[l // rows_per_peer] (device addresses, already offset to this rank's
    head slot).  Returns None then."""
    _cuda(q8, qs, k8, ks, vt, vs, tile_offsets, tile_entries, tile_order, out)
    H = q8.shape[0]
    nq = (Lq + 127) // 128
    if q8.shape[1] != nq * 128 or k8.shape[1] != pad128(Lk) or vt.shape[2] != pad128(Lk):
        raise _lib.KsanaB200Error("quantised operands do not match Lq / Lk (token axis must be padded to 128)")
    if tile_offsets is not None and (tile_offsets.numel() != nq + 1 or tile_offsets.dtype != torch.int32 or tile_entries.dtype != torch.int32):
        raise _lib.KsanaB200Error(f"tile_offsets must hold ceil(Lq/128)+1 = {nq + 1} int32 values, got {tile_offsets.numel()}")
    if tile_order is not None and (tile_order.numel() != nq or tile_order.dtype != torch.int32):
        raise _lib.KsanaB200Error(f"tile_order must hold ceil(Lq/128) = {nq} int32 values, got {tile_order.numel()}")
    entry = _lib.load().ksb_sage_attn
    if tile_offsets is not None and _lib.load().ksb_attn_dual_mode(-1) == 1:
        # block-sparse on the two-blocks-per-CTA kernel where adjacent Q blocks share their lists: the lists are merged
        # per pair (longest pairs first when the caller asked for an order); otherwise the one-block kernel
        paired = _pair_lists(tile_offsets, tile_entries, tile_order is not None)
        if paired is not None:
            tile_offsets, tile_entries, tile_order = paired
            entry = _lib.load().ksb_sage_attn_pairs
    if peer_out is not None:
        ptrs, rows, ts, hs = peer_out
        arr = _ptr_array(ptrs)
        dt = _lib.BF16 if out_dtype == torch.bfloat16 else _lib.FP16
        STATS.timed(("attn", H, Lq, Lk, tile_offsets is not None), lambda: _lib.check(
            entry(_p(q8), _p(qs), _p(k8), _p(ks), _p(vt), _p(vs), H, Lq, Lk, _p(tile_offsets),
                                      _p(tile_entries), _p(tile_order), None, dt, ts, hs, arr, len(ptrs), rows, _stream()),
            "ksb_sage_attn"))
        STATS.count(1)
        return None
    if out is None:
        out = torch.empty(Lq, H, 128, dtype=out_dtype, device=q8.device)
    assert out.stride(2) == 1
    dt = _lib.BF16 if out.dtype == torch.bfloat16 else _lib.FP16
    STATS.timed(("attn", H, Lq, Lk, tile_offsets is not None), lambda: _lib.check(
        entry(_p(q8), _p(qs), _p(k8), _p(ks), _p(vt), _p(vs), H, Lq, Lk, _p(tile_offsets),
              _p(tile_entries), _p(tile_order), _p(out), dt, out.stride(0), out.stride(1), None, 0, 0,
              _stream()),
        "ksb_sage_attn"))
    STATS.count(1)
    return out


def sage_attention(q, k, v, sm_scale=None, tile_offsets=None, tile_entries=None, out=None, tile_order=None):
    """q [Lq,H,128], k,v [Lk,H,128] half -> [Lq,H,128]: K smoothing, INT8 Q/K, FP8 V, attention core."""
    km = sage_kmean(k)
    q8, qs = sage_quant_int8(q, Q_BLOCK, premul=q_premul(q.shape[-1], sm_scale))
    k8, ks = sage_quant_int8(k, K_BLOCK, mean=km)
    vt, vs = sage_quant_v(v)
    return sage_attn_core(q8, qs, k8, ks, vt, vs, q.shape[0], k.shape[0], q.dtype, tile_offsets, tile_entries, out, tile_order)


# ----------------------------------------------------------------------------- RMSNorm + RoPE (in place)

_ROPE_TABLES: dict = {}


def wan_rope_table(head_dim: int = 128, max_len: int = 1024, theta: float = 10000.0, device="cuda"):
    """(cos, sin) table fp32 [max_len, head_dim//2, 2] of Wan's concatenated axis tables, plus (n_f, n_h).

    Same construction as KsanaDiT's ``rope_params`` x3 (ksana/models/wan/wan_model.py:51-58,676-684):
    computed in fp64, stored in fp32.  Host-side set-up, cached per (head_dim, max_len, theta, device).
    """
    key = (head_dim, max_len, theta, str(device))
    if key not in _ROPE_TABLES:
        d = head_dim
        dims = [d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)]
        pos = torch.arange(max_len, dtype=torch.float64)
        cols = []
        for dd in dims:
            inv = 1.0 / torch.pow(theta, torch.arange(0, dd, 2, dtype=torch.float64) / dd)
            cols.append(torch.outer(pos, inv))
        ang = torch.cat(cols, dim=1)
        tab = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()
        _ROPE_TABLES[key] = (tab.to(device), dims[0] // 2, dims[1] // 2)
    return _ROPE_TABLES[key]


def comfy_rope_table(head_dim: int = 128, max_len: int = 1024, theta: float = 10000.0, dtype=torch.bfloat16, device="cuda"):
    """(cos, sin) table of the ComfyUI RoPE formulation (``EmbedND`` / ``_comfy_rope``, ksana/utils/rope.py:151-180,
    selected by ``rope_func="comfy"``, wan_model.py:724-741), in the same [max_len, head_dim//2, 2] layout as
    ``wan_rope_table``.

    The rotation is the same pairwise one; what differs is the arithmetic: frequencies 1 / theta**linspace(0, (d-2)/d, d/2)
    per axis in fp64, angle = position * frequency in fp64, cos / sin rounded to fp32 and then to the model's
    ``dtype`` -- the reference builds its 2x2 matrices in the activation dtype, so with a bf16 model the table holds
    bf16-rounded entries.  They are stored here as fp32 values that are exactly representable in ``dtype``.
    Positions are exact for grids up to 256 per axis in bf16 (the reference's position ids are made in ``dtype`` too).
    """
    key = ("comfy", head_dim, max_len, theta, dtype, str(device))
    if key not in _ROPE_TABLES:
        d = head_dim
        dims = [d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)]
        pos = torch.arange(max_len, dtype=torch.float64)
        cols = []
        for dd in dims:
            expo = torch.linspace(0, (dd - 2) / dd, steps=dd // 2, dtype=torch.float64)
            cols.append(torch.outer(pos, 1.0 / (theta ** expo)))
        ang = torch.cat(cols, dim=1)
        tab = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).to(dtype).to(torch.float32).contiguous()
        _ROPE_TABLES[key] = (tab.to(device), dims[0] // 2, dims[1] // 2)
    return _ROPE_TABLES[key]


def rmsnorm_rope_inplace(x, w, eps=1e-6, rope=None, grid=None, pos0=0, want_mean=False, per_head=False, diag=False,
                         row_rstd=None):
    """x: [L, C] half view (row stride allowed), normalised (and rotated) in place.

    w: fp32 [C] (norm over all channels) or [128] with per_head (norm over each head's 128 channels).
    rope: (table [len,64,2] fp32, n_f, n_h) or None; grid: (F, H, W); diag: one position for all axes.
    row_rstd: fp32 [L] factors to use instead of rsqrt(mean(x^2) + eps) over the C channels present.
    Returns the fp32 column mean [C] of the written values when want_mean.
    """
    _cuda(x, w, row_rstd)
    assert row_rstd is None or (row_rstd.dtype == torch.float32 and row_rstd.is_contiguous() and row_rstd.numel() == x.shape[0])
    assert x.dim() == 2 and x.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous()
    L, C = x.shape
    assert w.numel() == (128 if per_head else C)
    lib = _lib.load()
    partial = mean = None
    if want_mean:
        partial = torch.empty(lib.ksb_rmsnorm_rope_scratch_floats(L, C), dtype=torch.float32, device=x.device)
        mean = torch.empty(C, dtype=torch.float32, device=x.device)
    tab, tlen, nf, nh, F, Hh, Ww = None, 0, 0, 0, 1, 1, 1
    if rope is not None:
        tab, nf, nh = rope
        tlen = tab.shape[0]
        F, Hh, Ww = (int(v) for v in grid)
    _lib.check(lib.ksb_rmsnorm_rope_inplace(_p(x), _dt(x), L, C, x.stride(0) if L > 1 else C, _p(w), int(per_head), _p(row_rstd),
                                            float(eps), _p(tab),
                                            tlen, nf, nh, F, Hh, Ww, int(pos0), int(diag), _p(partial), _p(mean), _stream()),
               "ksb_rmsnorm_rope_inplace")
    STATS.count(3 if want_mean else 1)
    return mean


def qwen_rope_tables(img_grid, txt_len, axes=(16, 56, 56), theta=10000.0, scale_rope=True, device="cuda"):
    """Rotation tables of the Qwen-Image block (QwenEmbedRope, ksana/models/qwen/attention.py:62-142), in the
    row-per-coordinate-index form rmsnorm_rope_inplace reads: (img_table, txt_table), each (tab, n_f, n_h).

    Image rows: row r holds the frame angle of frame r, the angle of the r-th (centred when scale_rope) image
    row and of the r-th image column.  Text rows: row t holds the angles of position t0 + t on all three axes.
    """
    Fr, Hh, Ww = (int(v) for v in img_grid)
    key = ("qwen", Fr, Hh, Ww, int(txt_len), tuple(axes), theta, scale_rope, str(device))
    if key in _ROPE_TABLES:  # host-side set-up, cached per shape (also keeps the forward free of host->device copies)
        return _ROPE_TABLES[key]
    inv = [1.0 / torch.pow(theta, torch.arange(0, d, 2, dtype=torch.float64) / d) for d in axes]
    n = max(Fr, Hh, Ww)

    def centred(m):
        return torch.cat([torch.arange(-(m - m // 2), 0), torch.arange(0, m // 2)]).to(torch.float64)

    fpos = torch.arange(n, dtype=torch.float64)
    hpos = torch.zeros(n, dtype=torch.float64)
    wpos = torch.zeros(n, dtype=torch.float64)
    hpos[:Hh] = centred(Hh) if scale_rope else torch.arange(Hh, dtype=torch.float64)
    wpos[:Ww] = centred(Ww) if scale_rope else torch.arange(Ww, dtype=torch.float64)
    ang = torch.cat([torch.outer(fpos, inv[0]), torch.outer(hpos, inv[1]), torch.outer(wpos, inv[2])], dim=1)
    img = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous().to(device)
    t0 = max(Hh // 2, Ww // 2) if scale_rope else max(Hh, Ww)
    tpos = torch.arange(t0, t0 + txt_len, dtype=torch.float64)
    tang = torch.cat([torch.outer(tpos, i) for i in inv], dim=1)
    txt = torch.stack([torch.cos(tang), torch.sin(tang)], dim=-1).to(torch.float32).contiguous().to(device)
    _ROPE_TABLES[key] = ((img, axes[0] // 2, axes[1] // 2), (txt, axes[0] // 2, axes[1] // 2))
    return _ROPE_TABLES[key]
