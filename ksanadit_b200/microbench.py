"""Single-kernel micro-benchmarks (CUDA-event timing) for the kernels of this package.

  python -m ksanadit_b200.microbench gemm  --M 75600 --N 15360 --K 5120
  python -m ksanadit_b200.microbench attn  --L 75600 --H 40 [--density 0.25]
  python -m ksanadit_b200.microbench quant --M 75600 --K 5120
  python -m ksanadit_b200.microbench prepass --L 75600 --H 40
  python -m ksanadit_b200.microbench qwen [--layers 60]

Each line reports the median device time of `--iters` launches after `--warmup` and the achieved
TFLOP/s (contractions) or GB/s of algorithmic bytes (HBM-bound passes).  Used for profiler captures of
one kernel on a small case as well.
"""

from __future__ import annotations

import argparse

import numpy as np
import torch

from . import _lib, ops, radial_mask


def timeit(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in ev)
    return ts[len(ts) // 2]


def fp8_rand(*shape, scale=50.0):
    return (torch.randn(*shape, device="cuda") * scale).clamp(-448, 448).to(torch.float8_e4m3fn)


def run_gemm(a):
    M, N, K = a.M, a.N, a.K
    xq, wq = fp8_rand(M, K), fp8_rand(N, K)
    sx, sw = torch.rand(M, device="cuda") + 0.5, (torch.rand(N, device="cuda") + 0.5) * 5e-6  # outputs of O(1)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    epi = {"none": _lib.EPI_NONE, "gelu": _lib.EPI_GELU_TANH, "gate": _lib.EPI_GATE_RESIDUAL}[a.epilogue]
    resid = torch.randn(M, N, device="cuda").to(torch.bfloat16) if epi == _lib.EPI_GATE_RESIDUAL else None
    gate = torch.randn(1, N, device="cuda").to(torch.bfloat16) if epi == _lib.EPI_GATE_RESIDUAL else None
    t = timeit(lambda: ops.fp8_gemm(xq, sx, wq, sw, bias, epilogue=epi, resid=resid, gate=gate, out=out), a.iters, a.warmup)
    fl = 2.0 * M * N * K
    print(f"fp8_gemm M={M} N={N} K={K} epilogue={a.epilogue}: {t:.3f} ms  {fl / t / 1e9:.1f} TFLOP/s")
    if a.compare:
        t2 = timeit(lambda: torch._scaled_mm(xq, wq.t(), scale_a=sx[:, None], scale_b=sw[None, :], bias=bias, out_dtype=torch.bfloat16),
                    a.iters, a.warmup)
        print(f"  torch._scaled_mm (row-wise scales, cuBLASLt): {t2:.3f} ms  {fl / t2 / 1e9:.1f} TFLOP/s")


def run_attn(a):
    L, H = a.L, a.H
    q, k, v = (torch.randn(L, H, 128, device="cuda").to(torch.bfloat16) for _ in range(3))
    km = ops.sage_kmean(k)
    q8, qs = ops.sage_quant_int8(q, 128, premul=ops.q_premul(128))
    k8, ks = ops.sage_quant_int8(k, 64, mean=km)
    vt, vs = ops.sage_quant_v(v)
    out = torch.empty(L, H, 128, dtype=torch.bfloat16, device="cuda")
    offs = ents = order = None
    pairs = ((L + 127) // 128) ** 2
    if a.density < 1.0:
        tpf = max(128, L // 21)
        m = radial_mask.bernoulli_frame_tile_mask(L, tpf, seed=0)
        o, e = radial_mask.compact_tile_lists(radial_mask.expand_to_kernel_granularity(m, 128))
        offs, ents = torch.from_numpy(o).cuda(), torch.from_numpy(e).cuda()
        if a.sorted:
            order = torch.from_numpy(radial_mask.longest_first_order(o)).cuda()
        pairs = int(e.size)
        print(f"  tile mask density {m.mean():.3f}")
    t = timeit(lambda: ops.sage_attn_core(q8, qs, k8, ks, vt, vs, L, L, tile_offsets=offs, tile_entries=ents, out=out, tile_order=order), a.iters, a.warmup)
    fl = 4.0 * H * 128 * 128 * 128 * pairs
    print(f"sage_attn L={L} H={H} tiles/head={pairs}: {t:.3f} ms  {fl / t / 1e9:.1f} TFLOP/s (visited tiles)")
    if a.compare and L <= 16384:
        qq, kk, vv = (x.permute(1, 0, 2)[None] for x in (q, k, v))
        t2 = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv), a.iters, a.warmup)
        print(f"  torch SDPA bf16: {t2:.3f} ms  {4.0 * H * L * L * 128 / t2 / 1e9:.1f} TFLOP/s")


def run_quant(a):
    M, K = a.M, a.K
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    sh = torch.randn(1, K, device="cuda").to(torch.bfloat16)
    w = torch.randn(K, device="cuda")
    by = M * K * 3 + M * 4
    for name, fn in (("quant_fp8_rowwise", lambda: ops.quant_fp8_rowwise(x)), ("adaln_quant_fp8", lambda: ops.adaln_quant_fp8(x, sh, sh)),
                     ("layernorm_quant_fp8", lambda: ops.layernorm_quant_fp8(x, w, w))):
        t = timeit(fn, a.iters, a.warmup)
        print(f"{name} M={M} K={K}: {t:.3f} ms  {by / t / 1e6:.0f} GB/s")


def run_prepass(a):
    L, H = a.L, a.H
    C = H * 128
    qkv = torch.randn(L, 3 * C, device="cuda").to(torch.bfloat16)
    w = torch.ones(C, device="cuda")
    rope = ops.wan_rope_table(128, 1024)
    grid = (21, max(1, L // 21 // 80), 80)
    t3 = qkv.view(L, 3, H, 128)
    km = torch.zeros(H, 128, device="cuda")
    sums = qkv[:, :2 * C].float().view(L, 2 * C // 256, 256).pow(2).sum(-1).t().contiguous() if C % 256 == 0 else None
    rstd = torch.rsqrt(qkv[:, :2 * C].float().view(L, 2, C).pow(2).mean(-1) + 1e-6).t().contiguous()
    for name, fn, by in (
        ("rmsnorm_rope_inplace(k, +mean)", lambda: ops.rmsnorm_rope_inplace(qkv[:, C:2 * C], w, 1e-6, rope, grid, want_mean=True), L * C * 4),
        ("sage_quant_int8(q)", lambda: ops.sage_quant_int8(t3[:, 0], 128, premul=0.1), L * C * 3),
        ("sage_quant_int8(k)", lambda: ops.sage_quant_int8(t3[:, 1], 64, mean=km), L * C * 3),
        ("sage_quant_v", lambda: ops.sage_quant_v(t3[:, 2]), L * C * 5),
        ("sage_kmean", lambda: ops.sage_kmean(t3[:, 1]), L * C * 2),
        ("sage_kmean_normed(k)", lambda: ops.sage_kmean_normed(t3[:, 1], w, 1e-6, rope, grid, row_rstd=rstd[1]), L * C * 2),
        ("sage_quant_int8_normed(q)", lambda: ops.sage_quant_int8_normed(t3[:, 0], 128, w, premul=0.1, rope=rope, grid=grid, row_rstd=rstd[0]), L * C * 3),
        ("sage_quant_int8_normed(k)", lambda: ops.sage_quant_int8_normed(t3[:, 1], 64, w, mean=km, rope=rope, grid=grid, row_rstd=rstd[1]), L * C * 3),
    ):
        t = timeit(fn, a.iters, a.warmup)
        print(f"{name} L={L} H={H}: {t:.3f} ms  {by / t / 1e6:.0f} GB/s")

    # the whole pre-pass of one self-attention, both ways (algorithmic bytes: Q, K, V read once, 8-bit copies written)
    def in_place():
        m = ops.rmsnorm_rope_inplace(qkv[:, C:2 * C], w, 1e-6, rope, grid, want_mean=True)
        ops.rmsnorm_rope_inplace(qkv[:, :C], w, 1e-6, rope, grid)
        ops.sage_quant_int8(t3[:, 0], 128, premul=0.1)
        ops.sage_quant_int8(t3[:, 1], 64, mean=m.view(H, 128))
        ops.sage_quant_v(t3[:, 2])

    def folded():
        r = ops.rowsumsq_to_rstd(sums, C)
        m = ops.sage_kmean_normed(t3[:, 1], w, 1e-6, rope, grid, row_rstd=r[1])
        ops.sage_quant_int8_normed(t3[:, 0], 128, w, premul=0.1, rope=rope, grid=grid, row_rstd=r[0])
        ops.sage_quant_int8_normed(t3[:, 1], 64, w, mean=m, rope=rope, grid=grid, row_rstd=r[1])
        ops.sage_quant_v(t3[:, 2])

    by = L * C * 9
    for name, fn in (("pre-pass, norm + RoPE in place then quantise", in_place), ("pre-pass, norm + RoPE inside the quantisers", folded)):
        t = timeit(fn, a.iters, a.warmup)
        print(f"{name} L={L} H={H}: {t:.3f} ms  {by / t / 1e6:.0f} GB/s of algorithmic bytes")


def run_qwen(a):
    """Qwen-Image-20B-shaped MMDiT step: 60 dual-stream blocks, dim 3072, 24 heads, 6889 image + 256 text tokens."""
    import os

    import torch.distributed as dist

    from .qwen_block import B200QwenBlock
    dim, heads, ffn, grid, Lt = 3072, 24, 12288, (1, 83, 83), 256
    layers = a.layers
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:  # launched by torch.distributed.run: image tokens sharded (padded to a multiple of the ranks)
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    blocks = [B200QwenBlock(dim, heads, ffn).random_init(100 + i) for i in range(layers)]
    Li_all = grid[1] * grid[2]
    Li = (Li_all + world - 1) // world
    img = torch.randn(1, Li, dim, device="cuda").to(torch.bfloat16)
    txt = torch.randn(1, Lt, dim, device="cuda").to(torch.bfloat16)
    temb = torch.randn(1, dim, device="cuda").to(torch.bfloat16)

    def step():
        t, i = txt, img
        with torch.no_grad():
            for b in blocks:
                t, i = b(i, t, temb, img_grid=grid)
        return i

    L = Li_all + Lt
    if world > 1:
        fl = layers * (2.0 * L * (3 * dim * dim + dim * dim + 2 * dim * ffn) + 2.0 * 2 * dim * 6 * dim + 4.0 * heads * L * L * 128)

        def report(tag, t):
            tt = torch.tensor([t], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            if rank == 0:
                print(f"qwen-image step on {world} GPUs (Ulysses, NCCL), {tag}: {layers} blocks, {Li_all}+{Lt} tokens, {Li} image rows per rank: "
                      f"{tt.item():.2f} ms  {fl / tt.item() / 1e9:.1f} TFLOP/s", flush=True)

        report("eager launches, block after block", timeit(step, a.iters, a.warmup))
        from .qwen_block import B200QwenDenoiseStep
        drv = B200QwenDenoiseStep(blocks)

        def driven():
            with torch.no_grad():
                return drv(img, txt, temb, img_grid=grid)[1]

        same = bool((step().float() == driven().float()).all())
        report(f"step driver (modulations ahead + text stream; equals the plain loop: {same})", timeit(driven, a.iters, a.warmup))
        dist.barrier()
        dist.destroy_process_group()
        return
    fl = layers * (2.0 * L * (3 * dim * dim + dim * dim + 2 * dim * ffn) + 2.0 * 2 * dim * 6 * dim + 4.0 * heads * L * L * 128)
    t = timeit(step, a.iters, a.warmup)
    print(f"qwen-image step, block after block: {layers} blocks, {Li}+{Lt} tokens: {t:.2f} ms  {fl / t / 1e9:.1f} TFLOP/s ({fl / 1e15:.4f} PFLOP)")
    from .graph import StepGraph
    from .qwen_block import B200QwenDenoiseStep
    ref = step().float()
    for text_stream in (False, True):
        drv = B200QwenDenoiseStep(blocks, text_stream=text_stream)

        def run(i=img, t_=txt, e=temb):
            with torch.no_grad():
                return drv(i, t_, e, img_grid=grid)[1]

        tag = "modulations ahead" + (" + text stream" if text_stream else "")
        got = run().float()
        t = timeit(run, a.iters, a.warmup)
        print(f"qwen-image step driver ({tag}): {t:.2f} ms  {fl / t / 1e9:.1f} TFLOP/s  equals the plain loop: {bool((ref == got).all())}")
        g = StepGraph(lambda i, t_, e: drv(i, t_, e, img_grid=grid)[1], (img, txt, temb))
        got = g(img, txt, temb).float()
        t = timeit(lambda: g(img, txt, temb), a.iters, a.warmup)
        print(f"  as one CUDA graph ({g.kernels_per_replay} kernels per replay): {t:.2f} ms  {fl / t / 1e9:.1f} TFLOP/s  equals: {bool((ref == got).all())}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemm", "attn", "quant", "prepass", "qwen"])
    ap.add_argument("--layers", type=int, default=60)
    ap.add_argument("--sorted", action="store_true", help="block-sparse: walk the Q blocks longest list first")
    ap.add_argument("--M", type=int, default=75600)
    ap.add_argument("--N", type=int, default=5120)
    ap.add_argument("--K", type=int, default=5120)
    ap.add_argument("--L", type=int, default=75600)
    ap.add_argument("--H", type=int, default=40)
    ap.add_argument("--density", type=float, default=1.0)
    ap.add_argument("--epilogue", default="none", choices=["none", "gelu", "gate"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--compare", action="store_true", help="also time the library kernel for the same shape")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    {"gemm": run_gemm, "attn": run_attn, "quant": run_quant, "prepass": run_prepass, "qwen": run_qwen}[a.kind](a)
    _lib.assert_device_ok()


if __name__ == "__main__":
    main()
_ = np
