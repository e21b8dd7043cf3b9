"""A linear layer over the vector-wise N:M sparse multiply: ``y = x @ W.T + b`` with the
weight pruned to ``n_keep``:32 (per-vector L2 magnitude), compressed and packed on the GPU
once, and every forward one call of the multiply.  Inference only (no autograd)."""
from __future__ import annotations

from typing import Optional


def _torch():
    import torch
    return torch


class NMSparseLinear:
    """``weight`` is the usual (out_features, in_features) dense float32 CUDA tensor;
    in_features must be a multiple of 32 (64 for the 75 % / 87.5 % formats) and
    out_features a multiple of 128.  ``vec_len`` is the number of adjacent outputs that
    share their kept inputs (32 or 64)."""

    def __init__(self, pkg, weight, n_keep: int, bias=None, vec_len: int = 32, path: Optional[int] = None):
        torch = _torch()
        self.out_features, self.in_features = weight.shape
        self.n_keep = n_keep
        self.path = pkg.PATH_FP32 if path is None else path
        dense = weight.detach().to(torch.float32).t().contiguous()        # (K, N) row-major, as the pruning kernel reads it
        BT, self.raw_indices = pkg.prune_device(dense, n_keep, vec_len)   # (W, N) values, (W, N/32) window-local k
        self.op = pkg.NMSpMM(BT, self.raw_indices, self.in_features, n_keep, device=weight.device)
        self.bias = None if bias is None else bias.detach().to(torch.float32)

    def __call__(self, x):
        torch = _torch()
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features).to(torch.float32)
        rows = x2.shape[0]
        pad = (-rows) % 4                                                 # the multiply takes M in multiples of 4
        A = torch.zeros((self.in_features, rows + pad), dtype=torch.float32, device=x.device)
        A[:, :rows] = x2.t()                                              # col-major M x K, the reference's A
        y = self.op.matmul(A, path=self.path)[:rows]
        if self.bias is not None:
            y = y + self.bias
        return y.reshape(*lead, self.out_features)

    def dense_weight(self):
        """The pruned weight as a dense (out_features, in_features) tensor (zeros where pruned),
        rebuilt from the compressed operand: what the layer multiplies by."""
        torch = _torch()
        BT = self.op.B                                                    # (W, N)
        win = torch.arange(BT.shape[0], device=BT.device) // self.n_keep  # window of every compressed row
        rows = (self.raw_indices.to(torch.int64) + (win * 32)[:, None]).repeat_interleave(32, dim=1)   # (W, N) global k
        dense = torch.zeros((self.in_features, self.out_features), dtype=torch.float32, device=BT.device)
        dense.scatter_(0, rows, BT)
        return dense.t().contiguous()
