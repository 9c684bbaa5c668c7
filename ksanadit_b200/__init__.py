"""ksanadit_b200: B200 (sm_100a) kernels for KsanaDiT's DiT-block hot path behind its operator API.

Layout: ``csrc/`` CUDA kernels + C ABI, ``_lib`` ctypes binding, ``ops`` functional wrappers,
``linear`` / ``attention`` / ``fuse_qkv`` / ``distribute`` mirrors of the KsanaDiT operator contracts,
``install`` to register them into a KsanaDiT process.
"""

from . import _lib  # noqa: F401

__all__ = ["_lib"]
__version__ = "0.1.0"
