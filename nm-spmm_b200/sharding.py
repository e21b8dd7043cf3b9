"""Column-vector-group sharding of the sparse operand across the GPUs of one box.

The column vectors of B are independent, so C = A.B splits by columns with no
exchange: rank r owns a contiguous group of whole index blocks (``layout_ns``
columns each), the matching slab of compressed values and indices, and produces
the column slab ``C[:, c0:c1]``.  A is replicated.  The only collective is the
optional all-gather of C.  (The reference has no multi-GPU path; this is the
partition BASELINE's sharded configuration asks for.)
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np


def partition_columns(N: int, world: int, layout_ns: int = 128) -> List[Tuple[int, int]]:
    """[c0, c1) per rank: whole ``layout_ns`` blocks, sizes differing by at most one block."""
    if N % layout_ns != 0:
        raise ValueError("N must be a multiple of layout_ns")
    blocks = N // layout_ns
    if world < 1 or blocks < world:
        raise ValueError(f"cannot give {world} ranks at least one {layout_ns}-column block of N={N}")
    base, rem = divmod(blocks, world)
    out, b = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((b * layout_ns, (b + n) * layout_ns))
        b += n
    return out


def shard_operands(BT: np.ndarray, DT: np.ndarray, rank: int, world: int, layout_ns: int = 128):
    """This rank's slab of the compressed values (W, n_local) and raw indices (W, n_local/32)."""
    c0, c1 = partition_columns(BT.shape[1], world, layout_ns)[rank]
    return (np.ascontiguousarray(BT[:, c0:c1]), np.ascontiguousarray(DT[:, c0 // 32:c1 // 32]), (c0, c1))


def all_gather_columns(C_local, N: int, world: int, layout_ns: int = 128, group=None):
    """All-gather of the column slabs into the full row-major C (M, N) on every rank.

    Slabs are strided in row-major C and may differ by one block, so each rank
    contributes its slab padded to the widest one; the pieces are placed after the
    collective.  Works on any torch.distributed backend (NCCL on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist

    parts = partition_columns(N, world, layout_ns)
    widest = max(c1 - c0 for c0, c1 in parts)
    M = C_local.shape[0]
    send = C_local if C_local.shape[1] == widest else torch.nn.functional.pad(C_local, (0, widest - C_local.shape[1]))
    send = send.contiguous()
    flat = torch.empty((world * M, widest), dtype=C_local.dtype, device=C_local.device)
    dist.all_gather_into_tensor(flat, send, group=group)     # rank r's slab lands in rows [r*M, (r+1)*M)
    recv = flat.view(world, M, widest)
    C = torch.empty((M, N), dtype=C_local.dtype, device=C_local.device)
    for r, (c0, c1) in enumerate(parts):
        C[:, c0:c1] = recv[r, :, :c1 - c0]
    return C


class ShardedNMSpMM:
    """The rank-local part of a column-sharded sparse operand (one process per GPU)."""

    def __init__(self, pkg, BT: np.ndarray, DT: np.ndarray, K: int, n_keep: int, rank: int, world: int,
                 layout_ns: int = 128, device=None):
        self.N, self.world, self.rank, self.layout_ns = BT.shape[1], world, rank, layout_ns
        bt, dt, self.columns = shard_operands(BT, DT, rank, world, layout_ns)
        self.local = pkg.NMSpMM(bt, dt, K, n_keep, layout_ns, device=device)

    def matmul(self, A, gather: bool = False, **kw):
        """Local slab C[:, c0:c1]; with ``gather`` the full C on every rank."""
        C_local = self.local.matmul(A, **kw)
        return all_gather_columns(C_local, self.N, self.world, self.layout_ns) if gather else C_local
