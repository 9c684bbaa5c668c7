"""Configuration types of the operator boundary, mirroring KsanaDiT's so callers can switch unchanged.

Mirrors ``KsanaAttentionBackend`` / ``KsanaAttentionConfig`` / ``KsanaRadialSageAttentionConfig``
(ksana/config/attention_config.py:23-104) and ``KsanaLinearBackend`` (ksana/config/linear_config.py:20-37).
When KsanaDiT itself is importable, ``ksanadit_b200.install`` registers the implementations under
KsanaDiT's own enum members; these classes serve standalone use and carry the same names, values and
validation.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum


class KsanaAttentionBackend(Enum):
    SAGE_ATTN = "sage_attention"
    RADIAL_SAGE_ATTN = "radial_sage_attention"

    @staticmethod
    def get_supported_list() -> list[str]:
        return [b.value for b in KsanaAttentionBackend]

    @staticmethod
    def support(type) -> bool:  # noqa: A002  (argument name kept from the mirrored interface)
        if isinstance(type, str):
            return type in KsanaAttentionBackend.get_supported_list()
        return isinstance(type, KsanaAttentionBackend)


@dataclass(frozen=True)
class KsanaAttentionConfig:
    backend: KsanaAttentionBackend | None = field(default=KsanaAttentionBackend.SAGE_ATTN)

    def __post_init__(self):
        if not KsanaAttentionBackend.support(self.backend):
            raise ValueError(f"attention_config {self.backend} not supported in {KsanaAttentionBackend.get_supported_list()}")


@dataclass(frozen=True)
class KsanaRadialSageAttentionConfig(KsanaAttentionConfig):
    backend: KsanaAttentionBackend = field(init=False, default=KsanaAttentionBackend.RADIAL_SAGE_ATTN)
    dense_blocks_num: int = field(default=0)
    dense_attn_steps: int = field(default=0)
    decay_factor: float = field(default=0.02)
    block_size: int = field(default=128)
    dense_attention_config: KsanaAttentionConfig = field(default=KsanaAttentionConfig(backend=KsanaAttentionBackend.SAGE_ATTN))

    def __post_init__(self):
        if self.block_size not in [64, 128]:
            raise ValueError(f"block_size must be 64 or 128, got {self.block_size}")
        if not (0 < self.decay_factor < 1):
            raise ValueError(f"decay_factor must be in range (0, 1), got {self.decay_factor}")


class KsanaLinearBackend(Enum):
    DEFAULT = "default"
    FP8_GEMM = "fp8_gemm"
    FP8_GEMM_DYNAMIC = "fp8_gemm_dynamic"
    FP16_GEMM = "fp16_gemm"

    @staticmethod
    def get_supported_list() -> list[str]:
        return [b.value for b in KsanaLinearBackend]

    @staticmethod
    def support(type) -> bool:  # noqa: A002
        if isinstance(type, str):
            return type in KsanaLinearBackend.get_supported_list()
        return isinstance(type, KsanaLinearBackend)


def backend_value(b) -> str:
    """Enum member (ours or KsanaDiT's) or string -> its string value."""
    return b.value if isinstance(b, Enum) else str(b)
