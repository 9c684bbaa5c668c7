"""Benchmark of the DiT-block hot path: one Wan2.2-14B-shaped 40-block denoise step at 75 600 tokens.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Prints ONE JSON line (rank 0).  ``value`` is whole-job TFLOP/s (algorithmic flop of the step / device time,
inputs resident in HBM); ``e2e`` is the same metric through the public call with host buffers (pinned
host -> device copies of the step's inputs and a device -> host read of the result inside the timed
region).  Ulysses shards the 75 600 tokens across ranks: total work is fixed, so scaling is "strong".

``--impl reference`` times the CPU restatement of the reference's torch path (fp32 Linear with emulated
FP8 quantisation + SDPA) on this host's cores, rank 0 only, on a bounded sample of the same block shape.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Wan2.2-T2V-14B block stack (ksana/settings/wan/modules/14b.yaml:16-26) at 720p x 81 frames
W14 = dict(layers=40, dim=5120, ffn=13824, heads=40, grid=(21, 45, 80), text_len=512)
# DRAM bytes (read + write) of one self-attention launch per head at 75 600 tokens, from the one-pass ncu capture of
# the full-size launch summarised in profiles/sage_attn_kernel_L16384_H16_and_full.md (3.26 GB for 40 heads)
ATTN_DRAM_BYTES_PER_HEAD = 3.262e9 / 40
METRIC = "wan14b_dit_step_tflops"
UNIT = "TFLOP/s"


def step_flops(cfg, L):
    """Algorithmic flop of one denoise step: Linears 2*M*N*K, attention 4*H*Lq*Lk*D (embeddings/head excluded)."""
    d, f, h, lc = cfg["dim"], cfg["ffn"], cfg["heads"], cfg["text_len"]
    lin = 2.0 * L * (d * 3 * d + d * d + d * f + f * d + 2 * d * d) + 2.0 * lc * 2 * d * d
    att = 4.0 * h * L * L * 128 + 4.0 * h * L * lc * 128
    return cfg["layers"] * (lin + att)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measure_fp8_peak(device):
    """Dense FP8 tensor peak measured the way MEASURED_PEAKS.json measures bf16: torch._scaled_mm e4m3 8192^3, best of 10."""
    n = 8192
    a = torch.randn(n, n, device=device).clamp(-2, 2).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=device).clamp(-2, 2).to(torch.float8_e4m3fn)
    one = torch.ones((), device=device)
    best = float("inf")
    for _ in range(3):
        torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2.0 * n ** 3 / best / 1e9


def cpu_reference_sample(tokens, reps):
    """Times the CPU restatement of the reference path (emulated FP8 Linear + SDPA) on one Wan-14B-shaped block
    over `tokens` tokens; returns (TFLOP/s, seconds per block, description)."""
    from oracle import dit_ops as D
    cfg = W14
    torch.set_num_threads(os.cpu_count() or 1)
    grid = (1, 16, tokens // 16)
    p = D.make_wan_block_params(cfg["dim"], cfg["ffn"], cfg["heads"], seed=0)
    x = D.make_activations(tokens, cfg["dim"], seed=0)[None]
    g = torch.Generator().manual_seed(0)
    e = (torch.randn(1, 1, 6, cfg["dim"], generator=g) * 0.1).to(torch.bfloat16)
    ctx = torch.randn(1, cfg["text_len"], cfg["dim"], generator=g).to(torch.bfloat16)
    one = dict(cfg, layers=1)
    fl = step_flops(one, tokens)
    ts = []
    with torch.no_grad():
        for _ in range(reps):
            t0 = time.perf_counter()
            D.wan_block_forward(p, x, e, ctx, grid, linear="fp8", attn="sdpa")
            ts.append(time.perf_counter() - t0)
    t = statistics.median(ts)
    desc = (f"one Wan2.2-14B-shaped block (dim {cfg['dim']}, ffn {cfg['ffn']}, {cfg['heads']} heads) on {tokens} tokens + "
            f"{cfg['text_len']} text tokens, torch CPU, emulated per-token/per-channel FP8 Linear + SDPA, median of {reps}")
    return fl / t / 1e12, t, desc


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_reference_sample(args.cpu_tokens, 1)
    vals = [cpu_reference_sample(args.cpu_tokens, 1) for _ in range(max(1, args.steps))]
    v = statistics.median(x[0] for x in vals)
    t = statistics.median(x[1] for x in vals)
    cores = torch.get_num_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3+int8 (emulated in fp32)", "data": "synthetic",
        "config": {"workload": f"wan2.2-14b denoise step: {W14['layers']} blocks, dim {W14['dim']}, {W14['heads']} heads x 128, "
                               f"ffn {W14['ffn']}, 75600 tokens (grid {W14['grid']}), {W14['text_len']} text tokens, batch 1",
                   "parallelism": "host cores", "sample": f"one block of that shape on {args.cpu_tokens} tokens per step"},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": vals[0][2]},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import torch.distributed as dist
    from ksanadit_b200 import _lib, ops
    from ksanadit_b200.wan_block import B200WanDenoiseStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    cfg = dict(W14)
    if args.layers:
        cfg["layers"] = args.layers
    if args.grid:
        cfg["grid"] = tuple(int(v) for v in args.grid.split("x"))
    L = cfg["grid"][0] * cfg["grid"][1] * cfg["grid"][2]
    if L % world != 0 or cfg["heads"] % world != 0:
        raise SystemExit(f"tokens {L} and heads {cfg['heads']} must be divisible by the world size {world}")
    Ll = L // world
    flops = step_flops(cfg, L)

    model = B200WanDenoiseStep(cfg["layers"], cfg["dim"], cfg["ffn"], cfg["heads"], device=dev, seed=1000)
    exchange = "none" if world == 1 else args.exchange
    if exchange in ("auto", "fused"):
        # peer stores fused into the GEMM / attention output stages; "auto" keeps the NCCL all-to-alls when the
        # peer-mapped buffers cannot be set up on this box (every rank takes the same branch)
        from ksanadit_b200.distribute import PeerExchange
        try:
            model.use_peer_exchange(PeerExchange.symmetric(Ll, cfg["heads"], torch.bfloat16, dev))
            exchange = "fused"
        except _lib.KsanaB200Error as err:
            if exchange == "fused":
                raise
            exchange = f"nccl (peer buffers unavailable: {err})"
    gh = torch.Generator().manual_seed(rank)
    # host-side inputs of a step (pinned): this rank's token shard, modulation, projected text context
    x_host = torch.empty(1, Ll, cfg["dim"], dtype=torch.bfloat16).pin_memory()
    chunk = 4096
    for i in range(0, Ll, chunk):  # N(0,1) with 1% outlier channels x20, generated in slices to bound host memory
        n = min(chunk, Ll - i)
        x_host[0, i:i + n] = torch.randn(n, cfg["dim"], generator=gh).to(torch.bfloat16)
    gsh = torch.Generator().manual_seed(12345)
    out_idx = torch.randperm(cfg["dim"], generator=gsh)[: cfg["dim"] // 100]
    x_host[0][:, out_idx] *= 20
    e_host = (torch.randn(1, 1, 6, cfg["dim"], generator=gsh) * 0.1).to(torch.bfloat16).pin_memory()
    c_host = torch.randn(1, cfg["text_len"], cfg["dim"], generator=gsh).to(torch.bfloat16).pin_memory()
    y_host = torch.empty(1, Ll, cfg["dim"], dtype=torch.bfloat16).pin_memory()
    grid_sizes = [cfg["grid"]]
    x_dev, e_dev, c_dev = x_host.to(dev), e_host.to(dev), c_host.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        return model(x_dev, e_dev, grid_sizes, c_dev)

    def step_e2e():
        xd = x_host.to(dev, non_blocking=True)
        ed = e_host.to(dev, non_blocking=True)
        cd = c_host.to(dev, non_blocking=True)
        y = model(xd, ed, grid_sizes, cd)
        y_host.copy_(y, non_blocking=True)

    def timed(fn, k):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    with torch.no_grad():
        for _ in range(args.warmup):
            step_resident()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ops.STATS.reset()
        ops.STATS.timing = True
        torch.cuda.cudart().cudaProfilerStart()  # lets a profiler started with --profile-from-start off see only the timed region
        ms = timed(step_resident, args.steps)
        torch.cuda.cudart().cudaProfilerStop()
        ops.STATS.timing = False
        launches = ops.STATS.kernels
        per_kernel = ops.STATS.summary()
        clocks = sampler.stop() if rank == 0 else None
        step_e2e()  # one untimed pass so that the context-K/V cache state matches the resident loop
        ms_e2e = timed(step_e2e, args.steps)
    _lib.assert_device_ok()

    # roofline of the dominant kernel: the self-attention launches (tensor bound)
    Hl = cfg["heads"] // world
    att_key = ("attn", Hl, L, L, False)
    n_att, ms_att = per_kernel.get(att_key, (0, 0.0))
    att_flop = 4.0 * Hl * L * L * 128
    achieved = att_flop * n_att / ms_att / 1e9 if ms_att > 0 else None
    gemm_ms = sum(v[1] for k, v in per_kernel.items() if k[0] == "gemm")
    gemm_fl = sum(2.0 * k[1] * k[2] * k[3] * v[0] for k, v in per_kernel.items() if k[0] == "gemm")

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        fp8_peak = measure_fp8_peak(dev)
        cpu_v, cpu_t, cpu_desc = cpu_reference_sample(args.cpu_tokens, 2)
        out = {
            "metric": METRIC, "value": flops * args.steps / ms / 1e9, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3+int8 (f32/s32 accumulate)", "data": "synthetic",
            "config": {"workload": f"wan2.2-14b denoise step: {cfg['layers']} blocks, dim {cfg['dim']}, {cfg['heads']} heads x 128, "
                                   f"ffn {cfg['ffn']}, {L} tokens (grid {cfg['grid']}), {cfg['text_len']} text tokens, batch 1",
                       "parallelism": f"ulysses{world}", "tokens_per_rank": Ll, "exchange": exchange,
                       "l2": "inputs larger than L2: every kernel streams >= 387 MB per launch, no flush needed",
                       "step_pflop": flops / 1e15},
            "clocks": clocks,
            "e2e": {"value": flops * args.steps / ms_e2e / 1e9, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 2 + e_host.numel() * 2 + c_host.numel() * 2,
                    "d2h_bytes_per_step": y_host.numel() * 2},
            "gpu_launches": launches,
            "roofline": {"kernel": "sage_attn_kernel (self-attention)", "bound": "tensor", "achieved": achieved, "peak": fp8_peak,
                         "unit": "TFLOP/s", "frac": (achieved / fp8_peak) if achieved else None,
                         "traffic": ATTN_DRAM_BYTES_PER_HEAD * Hl if L == 75600 else None,
                         "algorithmic_flop_per_launch": att_flop,
                         "peak_source": "of measured: torch._scaled_mm e4m3 8192^3 best of 10 in this run (MEASURED_PEAKS.json holds "
                                        f"bf16 only: {peaks.get('bf16_tflops')} TF/s burst)",
                         "launches": n_att, "ms_per_launch": (ms_att / n_att) if n_att else None,
                         "share_of_step": (ms_att / ms) if ms else None,
                         "gemm": {"tflops": gemm_fl / gemm_ms / 1e9 if gemm_ms else None, "share_of_step": gemm_ms / ms if ms else None}},
            "cpu_baseline": {"value": cpu_v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": cpu_desc,
                             "sec_per_block_sample": cpu_t},
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="(profiling only) fewer blocks than the 40 of the headline workload")
    ap.add_argument("--grid", default="", help="(profiling only) FxHxW token grid instead of 21x45x80")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "fused"],
                    help="Ulysses exchange at N > 1: NCCL all-to-alls, or peer stores fused into the GEMM / attention output stages")
    ap.add_argument("--cpu-tokens", type=int, default=1024, help="tokens of the bounded CPU sample")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
