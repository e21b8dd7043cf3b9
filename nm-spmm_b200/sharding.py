"""Column-vector-group sharding of the sparse operand across the GPUs of one box.

The column vectors of B are independent, so C = A.B splits by columns with no
exchange: rank r owns a contiguous group of whole index blocks (``layout_ns``
columns each), the matching slab of compressed values and indices, and produces
the column slab ``C[:, c0:c1]``.  A is replicated.  The only collective is the
optional all-gather of C.  (The reference has no multi-GPU path.)
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
                 layout_ns: int = 128, device=None, vec_len: int = 32):
        self.N, self.world, self.rank, self.layout_ns = BT.shape[1], world, rank, layout_ns
        bt, dt, self.columns = shard_operands(BT, DT, rank, world, layout_ns)
        self.local = pkg.NMSpMM(bt, dt, K, n_keep, layout_ns, device=device, vec_len=vec_len)
        self._symm = None

    def matmul(self, A, gather=False, **kw):
        """Local slab C[:, c0:c1]; with ``gather`` the full C on every rank.

        ``gather=True`` runs the multiply and then an NCCL all-gather of the slabs.
        ``gather="fused"`` lets the multiply kernel itself store every finished tile into the
        full-width C of all ranks (peer-mapped symmetric memory, plain stores over NVLink),
        so the transfer overlaps the arithmetic; the returned tensor is this rank's
        symmetric buffer, valid until the next fused call with the same row count."""
        if gather == "fused":
            return self._matmul_fused(A, **kw)
        C_local = self.local.matmul(A, **kw)
        return all_gather_columns(C_local, self.N, self.world, self.layout_ns) if gather else C_local

    def _symmetric_c(self, M: int, device):
        """Full-width C in symmetric memory and every rank's mapping of it (made once per M)."""
        import os

        import torch
        import torch.distributed as dist
        # plain peer mappings are all this path uses: no NVLink multicast object is bound
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        if self._symm is None or self._symm[0] != M:
            buf = symm_mem.empty((M, self.N), dtype=torch.float32, device=device)
            hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            # this rank's buffer first, then the peers in ring order (spreads the NVLink
            # traffic: at any moment different ranks write to different peers)
            order = [(self.rank + i) % self.world for i in range(self.world)]
            self._symm = (M, buf, hdl, [ptrs[r] for r in order], torch.zeros(1, device=device))
        return self._symm

    def _matmul_fused(self, A, **kw):
        import torch.distributed as dist

        _, buf, _, ptrs, flag = self._symmetric_c(A.shape[1], A.device)
        # Two stream-ordered barriers (a one-element NCCL all-reduce each): before the launch
        # every rank has finished reading the previous result out of its buffer; after it
        # every rank's stores have landed everywhere.
        dist.all_reduce(flag)
        self.local.matmul_into(A, ptrs, self.N, self.columns[0], **kw)
        dist.all_reduce(flag)
        return buf
