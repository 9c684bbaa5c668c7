"""CUDA-graph replay of a fixed-shape step (one block, or the whole per-step loop over the blocks).

The fused block paths launch 45-70 small kernels per block through ctypes; at Qwen-Image sizes (7 k tokens)
the host needs longer to issue them than the GPU needs to run them.  Every kernel of this library takes its
stream from ``torch.cuda.current_stream()``, allocates only through torch's caching allocator and never
synchronises, so a whole step can be captured once and replayed with one launch.

    step = StepGraph(lambda img, txt, temb: run_blocks(img, txt, temb), (img, txt, temb))
    out = step(img_new, txt_new, temb_new)      # copies into the static inputs, replays, returns static outputs

Constraints (checked where they can be): fixed shapes and dtypes; tensors only; the callable must be pure device
work (no ``.item()``, no host-side tables built per call -- the RoPE tables are cached per shape for this reason).
The outputs are views of graph-owned memory and are overwritten by the next replay.

Single-process steps only: a step that contains collectives (a process group is initialised with more than one
rank) is refused -- a capture with NCCL all-to-alls inside did not complete when it was tried on two GPUs.
"""

from __future__ import annotations

import torch

from . import _lib, ops


class StepGraph:
    def __init__(self, fn, example_inputs, warmup: int = 2):
        if not all(torch.is_tensor(t) and t.is_cuda for t in example_inputs):
            raise _lib.KsanaB200Error("StepGraph needs CUDA tensors as inputs")
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            raise _lib.KsanaB200Error("StepGraph captures single-process steps only (no collectives inside a graph)")
        if ops.STATS.timing:
            raise _lib.KsanaB200Error("switch per-call event timing off before capturing (events cannot be recorded into a graph)")
        self._fn = fn
        self._static_in = [t.clone() for t in example_inputs]
        # warm-up on a side stream: first calls set function attributes and look up the status words, the
        # allocator reaches its steady state
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                fn(*self._static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        _lib.assert_device_ok()
        kernels0 = ops.STATS.kernels
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph), torch.no_grad():
            out = fn(*self._static_in)
        self.kernels_per_replay = ops.STATS.kernels - kernels0  # kernels of this library inside the graph
        self._static_out = out

    def __call__(self, *inputs):
        if len(inputs) != len(self._static_in):
            raise _lib.KsanaB200Error(f"expected {len(self._static_in)} inputs, got {len(inputs)}")
        for dst, src in zip(self._static_in, inputs):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise _lib.KsanaB200Error(f"graph was captured for {tuple(dst.shape)} {dst.dtype}, got {tuple(src.shape)} {src.dtype}")
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self._graph.replay()
        ops.STATS.count(self.kernels_per_replay)
        return self._static_out
