"""CPU oracle for the DiT-block hot path. TEST INFRASTRUCTURE ONLY.

This package restates, in plain torch on the CPU, the arithmetic of KsanaDiT's
DiT-block path (FP8 quantized Linear, Sage-style quantized attention, adaLN /
RMSNorm / RoPE passes, Ulysses exchange, radial tile mask).  It is the checker
for the CUDA kernels in ``ksanadit_b200`` and the timed CPU baseline of the
benchmark.  Nothing in the product package imports it; only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py`` do.

Parity status
-------------
* Linear / norm / modulate / RoPE / block wiring / radial mask / all-to-all
  layout: pinned against the reference's own torch code imported on CPU (the
  generating script and the vectors live under ``tests/golden/``).
* Sage arithmetic (K smoothing, per-block INT8 Q/K, FP8 P.V): the reference
  calls un-vendored, un-pinned third-party packages (``sageattention``,
  ``spas_sage_attn``; call sites ``ksana/operations/attention/backends/
  sage_attn.py:75-81`` and ``.../radial_sage_attn/radial_sage_attn.py:170-176``)
  -> PARITY UNPINNED for the quantised INT8/FP8 attention tensors.  The oracle
  defines them; the only reference-held pin is the bound the reference's own
  test applies to Sage vs SDPA (``tests/ksana/attention_op_test.py:183-186``).
* Per-token x per-output-channel FP8 scales are a superset of the reference's
  per-tensor scales (``ksana/operations/linear/fp8_linear.py:41-63``); the
  per-tensor special case is pinned against the reference's ``fp8_linear``.
"""

from . import quantizers, sage, dit_ops, radial_mask, ulysses  # noqa: F401
