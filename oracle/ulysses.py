"""Oracle for the Ulysses exchange layout (plain torch, CPU).  Test infrastructure only.

Restates ``all_to_all(x, scatter_dim, gather_dim)`` of ksana/utils/distribute.py:112-122
as a pure function over the list of every rank's tensor, so the multi-rank layout
can be checked without a process group:

  rank r sends chunk p of its tensor along ``scatter_dim`` to rank p and
  concatenates what it receives, in rank order, along ``gather_dim``.

Used around attention as in wan_model.py:134-146: q/k/v scatter heads (dim 2) and
gather sequence (dim 1); the attention output does the inverse.
"""

from __future__ import annotations

import torch


def all_to_all_emulated(xs, scatter_dim, gather_dim):
    """xs: list (one per rank) of equally shaped tensors -> list of outputs per rank."""
    P = len(xs)
    chunks = [list(x.chunk(P, dim=scatter_dim)) for x in xs]
    return [torch.cat([chunks[src][dst] for src in range(P)], dim=gather_dim).contiguous() for dst in range(P)]


def shard_sequence(x, P, dim=1):
    """Sequence sharding of the block input: contiguous chunks (wan_model.py:919-920 uses torch.chunk)."""
    return list(x.chunk(P, dim=dim))
