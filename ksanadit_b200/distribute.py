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


def heads_to_sequence(qkv: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """[L_loc, n, H, D] (n stacked tensors, all heads, local tokens) -> [L, n, H/P, D] (local heads, all tokens).

    One all-to-all for q, k and v together (the reference does three, wan_model.py:138-140).  ``out``: a
    contiguous [L, n, H/P, D] buffer to receive into (e.g. the image rows of a joint text+image buffer)."""
    P = get_world_size()
    if P == 1:
        return qkv
    Ll, n, H, D = qkv.shape
    send = qkv.view(Ll, n, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P, L_loc, n, H/P, D]
    if out is None:
        out = torch.empty(P * Ll, n, H // P, D, dtype=qkv.dtype, device=qkv.device)
    if out.shape != (P * Ll, n, H // P, D) or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {(P * Ll, n, H // P, D)} tensor")
    dist.all_to_all_single(out.view(P, Ll, n, H // P, D), send, group=group)
    return out


def gather_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """[L, H/P, D] (this rank's heads of a replicated sequence) -> [L, H, D]: the all_gather + cat over heads of
    the replicated text stream (ksana/models/qwen/attention.py:298-307)."""
    P = get_world_size()
    if P == 1:
        return x
    L, Hl, D = x.shape
    buf = torch.empty(P * L, Hl, D, dtype=x.dtype, device=x.device)  # rank-major concatenation
    dist.all_gather_into_tensor(buf, x.contiguous(), group=group)
    return buf.view(P, L, Hl, D).permute(1, 0, 2, 3).reshape(L, P * Hl, D)


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


# ----------------------------------------------------------------------------- fused exchange over peer memory

class PeerExchange:
    """Buffers of one rank for the exchange fused into the GEMM / attention epilogues (plain peer stores over
    NVLink instead of the two all-to-alls of wan_model.py:134-146).

      qkv  [P*L_loc, 3, H/P, 128]  every rank's QKV GEMM stores its token rows of this rank's heads here
      rstd [2, P*L_loc] fp32       norm_q / norm_k factors of all tokens (every rank stores its own columns)
      out  [L_loc, H, 128]         every rank's attention kernel stores this rank's token rows of its heads here

    ``*_ptrs`` hold the device addresses of the same buffer on every rank, indexed by rank.  ``barrier()`` must
    order "all ranks have finished storing" before "any rank reads" on the current stream.
    """

    def __init__(self, P, rank, L_loc, heads, dtype, device, qkv, rstd, out, qkv_ptrs, rstd_ptrs, out_ptrs, barrier):
        self.P, self.rank, self.L_loc, self.heads, self.dtype, self.device = P, rank, L_loc, heads, dtype, device
        self.qkv, self.rstd, self.out = qkv, rstd, out
        self.qkv_ptrs, self.rstd_ptrs, self.out_ptrs = list(qkv_ptrs), list(rstd_ptrs), list(out_ptrs)
        self.barrier = barrier
        C = heads * 128
        self.tile_sumsq = torch.empty(2 * (C // 256), L_loc, dtype=torch.float32, device=device)

    @staticmethod
    def shapes(P, L_loc, heads):
        return (P * L_loc, 3, heads // P, 128), (2, P * L_loc), (L_loc, heads, 128)

    @classmethod
    def local_group(cls, P, L_loc, heads, dtype, device):
        """P contexts whose "peers" all live on one GPU: the layouts and kernels of the fused path without a second
        GPU (the caller runs each phase for every virtual rank in turn; barrier is a no-op)."""
        s_qkv, s_rstd, s_out = cls.shapes(P, L_loc, heads)
        qkv = [torch.empty(s_qkv, dtype=dtype, device=device) for _ in range(P)]
        rstd = [torch.empty(s_rstd, dtype=torch.float32, device=device) for _ in range(P)]
        out = [torch.empty(s_out, dtype=dtype, device=device) for _ in range(P)]
        return [cls(P, r, L_loc, heads, dtype, device, qkv[r], rstd[r], out[r], [t.data_ptr() for t in qkv],
                    [t.data_ptr() for t in rstd], [t.data_ptr() for t in out], lambda: None) for r in range(P)]

    @classmethod
    def symmetric(cls, L_loc, heads, dtype, device, group=None):
        """Buffers in torch's symmetric memory (one allocation per rank, mapped into every peer of the box).

        Raises KsanaB200Error when symmetric memory cannot be set up; the NCCL all-to-all path stays available."""
        import os

        from . import _lib
        # torch's switch for NVSwitch reduction objects: plain peer stores do not need them, and buffers that were
        # never bound to one cannot raise NVLink faults on the other ranks if a rank dies.  It only keeps the
        # allocation unbound; no kernel of this library issues a cluster-shared load.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        P, rank = dist.get_world_size(group), dist.get_rank(group)
        if P > 8:
            raise _lib.KsanaB200Error("the fused exchange spans at most the 8 GPUs of one box")

        def agree(err, what):
            """Every rank learns whether any rank failed `what`, so that all raise together and none is left alone
            in the next collective."""
            ok = torch.tensor([0 if err else 1], dtype=torch.int32, device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) != 1:
                raise _lib.KsanaB200Error(f"fused exchange: {what} failed ({err or 'on another rank'})")

        # the kernels address row l of rank r at r * L_loc + l: every rank must hold the same number of rows
        rows = torch.tensor([L_loc, -L_loc], dtype=torch.int64, device=device)
        dist.all_reduce(rows, op=dist.ReduceOp.MIN, group=group)
        if int(rows[0].item()) != -int(rows[1].item()):
            raise _lib.KsanaB200Error("fused exchange: every rank must hold the same number of token rows")
        # import and allocate first (local), agree that every rank could, and only then enter the collective rendezvous
        bufs, err, symm = [], None, None
        try:
            import torch.distributed._symmetric_memory as symm
            for shape, dt in zip(cls.shapes(P, L_loc, heads), (dtype, torch.float32, dtype)):
                bufs.append(symm.empty(shape, dtype=dt, device=device))
        except Exception as e:  # noqa: BLE001  (reported through agree())
            err = e
        agree(err, "symmetric-memory allocation")
        gname = (group or dist.group.WORLD).group_name
        ptrs, err = [], None
        try:
            for t in bufs:
                h = symm.rendezvous(t, gname)
                ptrs.append([int(v) for v in h.buffer_ptrs])
        except Exception as e:  # noqa: BLE001
            err = e
        agree(err, "symmetric-memory rendezvous")
        flag = torch.zeros(1, dtype=torch.float32, device=device)

        def barrier():
            # stream-ordered: the stores of earlier kernels on this stream are complete before the collective runs
            dist.all_reduce(flag, group=group)

        return cls(P, rank, L_loc, heads, dtype, device, bufs[0], bufs[1], bufs[2], ptrs[0], ptrs[1], ptrs[2], barrier)
