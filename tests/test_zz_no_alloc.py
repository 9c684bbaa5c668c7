"""GPU test of the allocation-free V quantiser (collected last on purpose: every other test has already run
if a stop-at-first-failure run gets here).

Some callers hand this library raw device pointers out of an arena they sized in advance and have no
allocator to lend it, or sit in a loop that must never reach cudaMalloc.  For them
``ksb_sage_quant_v_fp8_noalloc`` keeps its absmax scratch in a fixed array inside the library.  The test
drives it through the C ABI and requires the same bytes as the entry point that takes caller scratch, on
two calls in a row whose inputs differ (the second is much smaller in magnitude, so scratch left over from
the first call would show up as wrong scales).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, v, vt, vs):
    from ksanadit_b200 import _lib
    L, H, D = v.shape
    rc = lib.ksb_sage_quant_v_fp8_noalloc(v.data_ptr(), _lib.BF16, L, H, D, v.stride(0), v.stride(1), vt.data_ptr(), vs.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "ksb_sage_quant_v_fp8_noalloc")


def test_noalloc_v_quantiser_matches_existing_entry_point_twice():
    from ksanadit_b200 import _lib, ops
    lib = _lib.load()
    g = torch.Generator().manual_seed(21)
    L, H, D = 300, 3, 128
    Lp = ops.pad128(L)
    for scale in (8.0, 0.05):  # second call: far smaller values than the first
        v = (torch.randn(L, H, D, generator=g) * scale).to(torch.bfloat16).cuda()
        vt_ref, vs_ref = ops.sage_quant_v(v)  # existing entry point, scratch passed by the caller
        vt = torch.empty(H, D, Lp, dtype=torch.float8_e4m3fn, device="cuda")
        vs = torch.empty(H, D, dtype=torch.float32, device="cuda")
        before = torch.cuda.memory_allocated()
        _call_noalloc(lib, v, vt, vs)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # nothing came from torch's allocator
        assert torch.equal(vs, vs_ref)
        assert torch.equal(vt.view(torch.uint8), vt_ref.view(torch.uint8))
    _lib.assert_device_ok()


def test_noalloc_rejects_shapes_beyond_the_builtin_scratch():
    from ksanadit_b200 import _lib
    lib = _lib.load()
    H = 513  # 513 * 128 words > 65536
    v = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device="cuda")
    rc = lib.ksb_sage_quant_v_fp8_noalloc(v.data_ptr(), _lib.BF16, 1, H, 128, H * 128, 128, v.data_ptr(), v.data_ptr(), None)
    assert rc == -1 and b"exceeds the built-in scratch" in lib.ksb_last_error()
