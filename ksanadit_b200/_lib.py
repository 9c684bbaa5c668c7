"""ctypes binding of libksana_b200.so (the C ABI declared in include/ksana_b200.h).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("KSANA_B200_LIB", os.path.join(_HERE, "lib", "libksana_b200.so"))

BF16, FP16 = 0, 1
EPI_NONE, EPI_GELU_TANH, EPI_GATE_RESIDUAL = 0, 1, 2

# name -> (restype, argtypes); mirrors include/ksana_b200.h one to one
SIGNATURES = {
    "ksb_version": (c_int, []),
    "ksb_last_error": (c_char_p, []),
    "ksb_device_status": (c_int, [POINTER(c_int), POINTER(c_int)]),
    "ksb_sm_count": (c_int, []),
    "ksb_selftest_bounded_wait": (c_int, [c_int64, c_void_p, c_void_p]),
    "ksb_quant_fp8_rowwise": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "ksb_quant_fp8_static": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ksb_adaln_quant_fp8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int, c_float,
                                    c_void_p, c_void_p, c_void_p, c_void_p]),
    "ksb_layernorm_quant_fp8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_float,
                                        c_void_p, c_void_p, c_void_p, c_void_p]),
    "ksb_fp8_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int,
                             c_int64, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "ksb_gate_residual": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int64, c_int64, c_void_p]),
    "ksb_residual_diff": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "ksb_sage_kmean_scratch_floats": (c_int64, [c_int64, c_int64, c_int64]),
    "ksb_sage_kmean": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "ksb_rmsnorm_rope_scratch_floats": (c_int64, [c_int64, c_int64]),
    "ksb_rmsnorm_rope_inplace": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_float, c_void_p, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "ksb_sage_quant_int8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_void_p,
                                    c_void_p, c_void_p, c_void_p]),
    "ksb_sage_quant_v_fp8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_void_p]),
    "ksb_sage_quant_v_fp8_noalloc": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                             c_void_p]),
    "ksb_sage_attn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p]),
    "ksb_sage_attn_pairs": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p]),
    "ksb_fp8_gemm_qkv_scatter": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int,
                                         c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p]),
    "ksb_rowsumsq_to_rstd_scatter": (c_int, [c_void_p, c_int64, c_int64, c_float, c_void_p, c_int, c_int, c_void_p]),
    "ksb_gemm_pair_mode": (c_int, [c_int]),
    "ksb_attn_dual_mode": (c_int, [c_int]),
    "ksb_fp8_gemm_rowstats": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int,
                                      c_int64, c_void_p, c_int64, c_void_p]),
    "ksb_rowsumsq_to_rstd": (c_int, [c_void_p, c_int64, c_int64, c_int, c_float, c_void_p, c_void_p]),
    "ksb_sage_kmean_normed": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_float,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "ksb_sage_quant_int8_normed": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int, c_float, c_void_p,
                                           c_void_p, c_int, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int64,
                                           c_int, c_void_p, c_void_p, c_void_p]),
}

_lib = None


class KsanaB200Error(RuntimeError):
    pass


def load():
    """Loads the shared library (once) and declares every entry point.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise KsanaB200Error(
            f"{LIB_PATH} is missing: build it with `python -m ksanadit_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback for these kernels"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library out of step
        fn.restype = res
        fn.argtypes = args
    # KSANA_B200_GEMM_PAIR=0 selects the single-CTA GEMM form for the whole process (default: CTA pairs)
    mode = os.environ.get("KSANA_B200_GEMM_PAIR")
    if mode in ("0", "1"):
        lib.ksb_gemm_pair_mode(int(mode))
    # KSANA_B200_ATTN_DUAL=0 keeps dense attention on the one-block-per-CTA kernel (default: two blocks per CTA)
    mode = os.environ.get("KSANA_B200_ATTN_DUAL")
    if mode in ("0", "1"):
        lib.ksb_attn_dual_mode(int(mode))
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().ksb_last_error()
        raise KsanaB200Error(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def device_status():
    """Synchronises and returns (code, detail) of the kernels' bounded-wait status words, clearing them.

    The words are sticky: after one wait has run out, later kernels give up their waits at once (and leave their
    outputs unwritten) until this call has read the words -- check once per step where results are consumed."""
    code, detail = c_int(0), c_int(0)
    check(load().ksb_device_status(ctypes.byref(code), ctypes.byref(detail)), "ksb_device_status")
    return code.value, detail.value


def assert_device_ok():
    code, detail = device_status()
    if code != 0:
        raise KsanaB200Error(f"a kernel wait ran out: code={code} kernel={detail >> 16} site={detail & 0xffff}")


_ = (c_int32,)
