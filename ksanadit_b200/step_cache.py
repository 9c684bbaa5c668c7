"""Block-level step cache (DBCache) around a stack of B200 blocks.

Mirrors ``DBCacheConfig`` (ksana/config/cache_config/dbcache.py:21-34), ``DBCacheContext`` / ``CacheBuffer`` /
``DBCache`` (ksana/cache/dbcache.py:60-450): the first ``fn_compute_blocks`` blocks always run; the residual they add
is compared with the one kept from the last computed step (relative L1 distance, dbcache.py:228-239); below the
threshold the remaining blocks are skipped and the residual those blocks added last time is applied instead; warm-up
steps, a cap on consecutive and on total cached steps, separate state for the cond / uncond / combine phases.

What is done differently: the residual ``x - x_ori`` and the three reductions the decision needs are one kernel pass
over the activations (``ksb_residual_diff``) instead of a subtraction, an ``abs`` and three ``mean`` launches, and the
host reads back three floats.  The means are rounded to the activation dtype before they are combined, as eager
torch does, so that decisions agree with the reference's except on exact ties of the fp32 summation order.
TaylorSeer extrapolation (first order, dbcache.py:271-283) is supported.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from . import _lib, ops

PHASES = ("cond", "uncond", "combine")


@dataclass
class DBCacheConfig:
    name: str = "DBCache"
    fn_compute_blocks: int = 1
    bn_compute_blocks: int = 0
    residual_diff_threshold: float = 0.08
    max_warmup_steps: int = 4
    warmup_interval: int = 1
    max_cached_steps: int = 8
    max_continuous_cached_steps: int = 2
    enable_separate_cfg: bool = True
    cfg_compute_first: bool = False
    enable_taylorseer: bool = False
    taylorseer_order: int = 1
    num_blocks: int = 40  # the recommended Wan2.2-T2V-14B settings (dbcache.py:45-57) are the defaults


@dataclass
class _PhaseState:
    first_residual: torch.Tensor | None = None   # what the first blocks added at the last computed step
    rest_residual: torch.Tensor | None = None    # what all later blocks added at the last computed step
    older_rest: list = field(default_factory=list)
    total: int = 0
    cached: int = 0


def relative_l1(sums: torch.Tensor, n: int, dtype: torch.dtype) -> float:
    """dbcache.py:228-239 from the kernel's sums: mean |cur - prev| / ((mean |cur| + mean |prev|) / 2), every mean and
    every intermediate rounded to ``dtype`` as the eager expression on half tensors rounds them."""
    d, c, p = (sums.detach().float().cpu() / n).to(dtype)
    eps = torch.tensor(1e-8, dtype=dtype)
    avg = ((c + eps) + (p + eps)) / 2
    return float(d / avg)


class B200DBCache:
    """``cache(phase, x, step_iter, timestep, blocks, **kwargs) -> x`` with every block called as ``block(x, **kwargs)``."""

    def __init__(self, config: DBCacheConfig | None = None, diff_fn=None):
        self.config = config or DBCacheConfig()
        c = self.config
        if c.fn_compute_blocks < 0 or c.bn_compute_blocks < 0 or c.fn_compute_blocks + c.bn_compute_blocks > c.num_blocks:
            raise ValueError(f"fn_compute_blocks({c.fn_compute_blocks}) + bn_compute_blocks({c.bn_compute_blocks}) must be within "
                             f"num_blocks({c.num_blocks})")
        self._diff_fn = diff_fn or self._device_diff
        self.diff_history: list[float] = []
        self.reset()

    # ------------------------------------------------------------------ state
    def reset(self):
        self.step = 0
        self.cached_steps = 0
        self.consecutive_cached = 0
        self.last_timestep = None
        self.state = {p: _PhaseState() for p in PHASES}

    def _is_warmup(self) -> bool:
        c = self.config
        if self.step >= c.max_warmup_steps:
            return False
        return c.warmup_interval <= 1 or self.step % c.warmup_interval == 0

    def valid_for(self, phase: str, **_) -> bool:
        """May this step try the cache at all (dbcache.py:187-211)?"""
        st = self.state[phase]
        st.total += 1
        if self._is_warmup() or st.first_residual is None:
            return False
        c = self.config
        if c.max_continuous_cached_steps > 0 and self.consecutive_cached >= c.max_continuous_cached_steps:
            self.consecutive_cached = 0
            return False
        if c.max_cached_steps > 0 and self.cached_steps >= c.max_cached_steps:
            return False
        return True

    # ------------------------------------------------------------------ the reductions
    @staticmethod
    def _device_diff(x_new, x_old, prev):
        """(residual, relative L1 distance to prev or None) through the CUDA kernel; no CPU path."""
        if not x_new.is_cuda:
            raise _lib.KsanaB200Error("the step cache's residual statistics run on the GPU (no CPU path exists)")
        same = prev is not None and prev.shape == x_new.shape and prev.device == x_new.device
        res, sums = ops.residual_diff(x_new.contiguous(), x_old.contiguous(), prev.contiguous() if same else None)
        return res, (relative_l1(sums, x_new.numel(), x_new.dtype) if same else None)

    def _advance(self, timestep):
        """One step per distinct timestep: cond and uncond of the same timestep share the step counter (dbcache.py:373-387)."""
        try:
            ts = int(timestep) if isinstance(timestep, (int, float)) else int(timestep.item())
        except (ValueError, TypeError, RuntimeError):
            ts = None
        if ts is not None:
            if self.last_timestep == ts:
                return
            self.last_timestep = ts
        self.step += 1

    def _remember(self, st, first, rest):
        if self.config.enable_taylorseer and st.rest_residual is not None:
            st.older_rest.append(st.rest_residual)
            del st.older_rest[: max(0, len(st.older_rest) - (self.config.taylorseer_order + 1))]
        st.first_residual, st.rest_residual = first, rest
        self.consecutive_cached = 0

    def _cached_rest(self, st):
        st.cached += 1
        self.cached_steps += 1
        self.consecutive_cached += 1
        r = st.rest_residual
        if self.config.enable_taylorseer and st.older_rest and min(self.config.taylorseer_order, len(st.older_rest)) >= 1:
            r = r + (r - st.older_rest[-1])
        return r

    # ------------------------------------------------------------------ the wrapped block loop
    def __call__(self, phase, x, step_iter, timestep, blocks, **kwargs):
        if blocks is None:
            return x
        c = self.config
        nb = c.num_blocks
        f_end = c.fn_compute_blocks
        rest = list(range(f_end, nb))  # the middle blocks, then the last bn_compute_blocks: both run only on a miss
        st = self.state[phase]
        if self.valid_for(phase, x=x, step_iter=step_iter, timestep=timestep):
            x0 = x
            for i in range(0, min(f_end, len(blocks))):
                x = blocks[i](x, **kwargs)
            first, rel = self._diff_fn(x, x0, st.first_residual)
            hit = False
            if rel is not None:
                self.diff_history.append(rel)
                if rel < c.residual_diff_threshold and st.rest_residual is not None:
                    x = x + self._cached_rest(st).to(x.device)
                    hit = True
            if not hit:
                x1 = x
                for i in rest:
                    if i < len(blocks):
                        x = blocks[i](x, **kwargs)
                rest_res, _ = self._diff_fn(x, x1, None)
                self._remember(st, first, rest_res)
        else:
            x0 = x
            for blk in blocks:
                x = blk(x, **kwargs)
            full, _ = self._diff_fn(x, x0, None)
            self._remember(st, full, full)
        self._advance(timestep)
        return x

    # ------------------------------------------------------------------ reporting / housekeeping
    def get_stats_summary(self) -> dict:
        s = self.state
        return {"name": self.config.name, "config": str(self.config),
                "cond_total_steps": s["cond"].total, "cond_cached_steps": s["cond"].cached,
                "cond_cache_rate": s["cond"].cached / max(s["cond"].total, 1),
                "uncond_total_steps": s["uncond"].total, "uncond_cached_steps": s["uncond"].cached,
                "uncond_cache_rate": s["uncond"].cached / max(s["uncond"].total, 1)}

    def show_cache_rate(self) -> str:
        t = self.get_stats_summary()
        return (f"[DBCache] fn={self.config.fn_compute_blocks} bn={self.config.bn_compute_blocks} threshold={self.config.residual_diff_threshold} "
                f"cond {t['cond_cached_steps']}/{t['cond_total_steps']} uncond {t['uncond_cached_steps']}/{t['uncond_total_steps']}")

    def offload_to_cpu(self):
        for st in self.state.values():
            st.first_residual = None if st.first_residual is None else st.first_residual.cpu()
            st.rest_residual = None if st.rest_residual is None else st.rest_residual.cpu()
            st.older_rest = [t.cpu() for t in st.older_rest]
