"""Ulysses sequence-parallel exchange over NCCL (NVLink 5 / NVSwitch), one process per GPU.

Mirrors ``get_rank_id`` / ``get_world_size`` / ``all_to_all`` / ``all_gather`` / ``gather_forward``
(ksana/utils/distribute.py:88-142).  The reference issues a list all-to-all wrapped in
chunk -> contiguous -> all_to_all -> cat -> contiguous; here one ``all_to_all_single`` moves a buffer whose
leading dimension is already the peer index, so the only copies are one pack and one unpack, and the
fused block path writes / reads those layouts directly.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def get_rank_id() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def all_to_all(x: torch.Tensor, scatter_dim: int, gather_dim: int, group=None, **kwargs) -> torch.Tensor:
    """Scatter ``x`` along ``scatter_dim`` and gather along ``gather_dim`` (same result as the reference's)."""
    P = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
    if P == 1:
        return x
    if x.shape[scatter_dim] % P != 0:
        raise ValueError(f"dimension {scatter_dim} of size {x.shape[scatter_dim]} is not divisible by the world size {P}")
    # [.., P*c, ..] -> [P, .., c, ..] : chunk p goes to rank p
    send = torch.stack(x.chunk(P, dim=scatter_dim), dim=0).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[p] came from rank p; concatenate along gather_dim in rank order
    return torch.cat(list(recv.unbind(0)), dim=gather_dim).contiguous()


def heads_to_sequence(qkv: torch.Tensor, group=None) -> torch.Tensor:
    """[L_loc, n, H, D] (n stacked tensors, all heads, local tokens) -> [L, n, H/P, D] (local heads, all tokens).

    One all-to-all for q, k and v together (the reference does three, wan_model.py:138-140)."""
    P = get_world_size()
    if P == 1:
        return qkv
    Ll, n, H, D = qkv.shape
    send = qkv.view(Ll, n, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P, L_loc, n, H/P, D]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(P * Ll, n, H // P, D)


def sequence_to_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """[L, H/P, D] (local heads, all tokens) -> [L_loc, H, D] (all heads, local tokens); wan_model.py:146."""
    P = get_world_size()
    if P == 1:
        return x
    L, Hl, D = x.shape
    send = x.view(P, L // P, Hl, D).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3).reshape(L // P, P * Hl, D)


def all_gather(tensor: torch.Tensor):
    P = get_world_size()
    if P == 1:
        return [tensor]
    out = [torch.empty_like(tensor) for _ in range(P)]
    dist.all_gather(out, tensor)
    return out


def gather_forward(input: torch.Tensor, dim: int) -> torch.Tensor:  # noqa: A002
    if get_world_size() == 1:
        return input
    return torch.cat(all_gather(input), dim=dim).contiguous()
