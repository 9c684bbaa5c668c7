"""GPU: the time-out path of the kernels' bounded waits, exercised without faulting the GPU.

A self-test kernel waits (for 2 ms at most) on a barrier nothing completes.  It must return by itself, the status
words must name the wait, the Python layer must turn them into an exception, reading them must clear them, and the
next launches on the same context must work."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported_then_cleared():
    from ksanadit_b200 import _lib, ops
    lib = _lib.load()
    assert _lib.device_status() == (0, 0)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(lib.ksb_selftest_bounded_wait(2_000_000, flag.data_ptr(), torch.cuda.current_stream().cuda_stream), "selftest")
    torch.cuda.synchronize()  # the kernel came back by itself
    assert int(flag.item()) == 2, "the wait must report failure, not success"
    with pytest.raises(_lib.KsanaB200Error, match="kernel=15 site=1"):
        _lib.assert_device_ok()
    assert _lib.device_status() == (0, 0)  # reading cleared the words
    # the context is intact: a real kernel runs and is bit-exact afterwards
    x = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    q, s = ops.quant_fp8_rowwise(x)
    from oracle import quantizers as Qz
    q_ref, s_ref = Qz.act_quant_fp8_rowwise(x.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s.cpu(), s_ref)
    _lib.assert_device_ok()
