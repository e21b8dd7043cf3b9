"""A linear layer over the vector-wise N:M sparse multiply: ``y = x @ W.T + b`` with the
weight pruned to ``n_keep``:32 (per-vector L2 magnitude), compressed and packed on the GPU
once, and every forward one call of the multiply.

The forward is registered with ``torch.library`` as the custom operator
``nmspmm_b200::sparse_linear`` (with a fake kernel for tracing and an autograd formula), so
the layer can be traced, compiled around and differentiated.  Activations are taken
row-major as they come (``nmspmm_gemm_row_major`` transposes on the GPU ahead of the
multiply); nothing is padded or transposed in eager PyTorch.  float16 / bfloat16 activations
give a result of the same dtype (``nmspmm_gemm_row_major_16``: widened exactly inside the
transposition, summed in FP32, rounded once at the end); the compressed weights are FP32.

The reference has no framework binding (its only caller is its test driver,
tests/test_nmspmm.cu:8-160).  The backward pass is a convenience, not a tuned path: it
expands the compressed weight to dense and uses torch's own products.
"""
import ctypes
from typing import Optional

_registered = None
_workspaces = {}        # per device: the operator's scratch (zero when made: the multiply wants its counter block zero)


def _torch():
    import torch
    return torch


def _dense_rows(raw_indices, n_keep: int):
    """(W, N) global k of every compressed value, from the raw window-local indices (W, N/32)."""
    torch = _torch()
    win = torch.arange(raw_indices.shape[0], device=raw_indices.device) // n_keep
    return (raw_indices.to(torch.int64) + (win * 32)[:, None]).repeat_interleave(32, dim=1)


def register_ops(pkg):
    """Defines ``torch.ops.nmspmm_b200.sparse_linear`` once per process and returns it."""
    global _registered
    if _registered is not None:
        return _registered
    torch = _torch()

    @torch.library.custom_op("nmspmm_b200::sparse_linear", mutates_args=())
    def sparse_linear(x: torch.Tensor, values: torch.Tensor, packed: torch.Tensor, column_info: Optional[torch.Tensor],
                      raw_indices: torch.Tensor, n_keep: int, fmt: int, layout_ns: int, vec_len: int, path: int) -> torch.Tensor:
        """x (M, K) row-major float32 / float16 / bfloat16 . B (K, N) in N:M form -> (M, N) of x's dtype.  ``values`` (W, N) are the
        compressed weights, ``packed`` / ``column_info`` the packed indices the kernels read,
        ``raw_indices`` (W, N/32) the unpacked ones (used by the backward formula only)."""
        lib = pkg.load_library()
        x = x.contiguous()
        M, K = x.shape
        N = values.shape[1]
        dtype = pkg.dtype_id(x.dtype)
        d = pkg.make_desc(M, N, K, n_keep, fmt, layout_ns, path, 0, 0, vec_len)
        wide = dtype == pkg.DTYPE_F32
        need = int((lib.nmspmm_gemm_row_major_workspace_bytes if wide else lib.nmspmm_gemm_row_major_16_workspace_bytes)(ctypes.byref(d)))
        if need == 0:
            raise pkg.NMSpMMError("nmspmm_gemm_row_major_workspace_bytes", pkg.UNSUPPORTED)
        ws = _workspaces.get(x.device)
        if ws is None or ws.numel() < need:
            ws = _workspaces[x.device] = torch.zeros(need, dtype=torch.uint8, device=x.device)
        y = torch.empty((M, N), dtype=x.dtype, device=x.device)
        ci = ctypes.c_void_p(column_info.data_ptr()) if column_info is not None else ctypes.c_void_p(0)
        ptrs = (ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(values.data_ptr()), ctypes.c_void_p(packed.data_ptr()), ci,
                ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ws.numel(),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if wide:
            rc, where = lib.nmspmm_gemm_row_major(ctypes.byref(d), *ptrs), "nmspmm_gemm_row_major"
        else:
            rc, where = lib.nmspmm_gemm_row_major_16(ctypes.byref(d), dtype, *ptrs), "nmspmm_gemm_row_major_16"
        if rc != pkg.OK:
            raise pkg.NMSpMMError(where, rc)
        return y

    @sparse_linear.register_fake
    def _(x, values, packed, column_info, raw_indices, n_keep, fmt, layout_ns, vec_len, path):
        return x.new_empty((x.shape[0], values.shape[1]))

    def setup_context(ctx, inputs, output):
        x, values, _packed, _ci, raw_indices, n_keep = inputs[:6]
        ctx.n_keep = n_keep
        ctx.save_for_backward(x, values, raw_indices)

    def backward(ctx, grad_y):
        x, values, raw_indices = ctx.saved_tensors
        rows = _dense_rows(raw_indices, ctx.n_keep)                       # (W, N) global k of every kept value
        grad_x = grad_values = None
        g32 = grad_y.to(torch.float32)
        if ctx.needs_input_grad[0]:
            dense = torch.zeros((x.shape[1], values.shape[1]), dtype=torch.float32, device=values.device)
            dense.scatter_(0, rows, values)                               # B with explicit zeros, (K, N)
            grad_x = (g32 @ dense.t()).to(x.dtype)
        if ctx.needs_input_grad[1]:
            grad_values = (x.to(torch.float32).t() @ g32).gather(0, rows)  # d/dB restricted to the kept positions
        return grad_x, grad_values, None, None, None, None, None, None, None, None

    sparse_linear.register_autograd(backward, setup_context=setup_context)
    _registered = sparse_linear
    return sparse_linear


class NMSparseLinear:
    """``weight`` is the usual (out_features, in_features) dense float32 CUDA tensor;
    in_features must be a multiple of 32 (64 for the 75 % / 87.5 % formats) and
    out_features a multiple of 128.  ``vec_len`` is the number of adjacent outputs that
    share their kept inputs (32 or 64).  ``values`` (the kept weights, a leaf tensor) and
    ``bias`` may be given ``requires_grad_()``; the sparsity pattern is fixed at construction."""

    def __init__(self, pkg, weight, n_keep: int, bias=None, vec_len: int = 32, path: Optional[int] = None):
        torch = _torch()
        self._pkg = pkg
        self._op = register_ops(pkg)
        self.out_features, self.in_features = weight.shape
        self.n_keep, self.vec_len = n_keep, vec_len
        self.path = pkg.PATH_FP32 if path is None else path
        w = weight.detach()
        if w.dtype in (torch.float16, torch.bfloat16) and w.is_cuda and w.numel() % 4 == 0:
            w = pkg.widen_device(w.contiguous())                          # exact; the compressed weights stay FP32
        dense = w.to(torch.float32).t().contiguous()                      # (K, N) row-major, as the pruning kernel reads it
        BT, self.raw_indices = pkg.prune_device(dense, n_keep, vec_len)   # (W, N) values, (W, N/32) window-local k
        self.op = pkg.NMSpMM(BT, self.raw_indices, self.in_features, n_keep, device=weight.device, vec_len=vec_len)
        self.values = self.op.B                                           # the layer's trainable tensor
        self.bias = None if bias is None else bias.detach().to(torch.float32)

    def __call__(self, x):
        torch = _torch()
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            x2 = x2.to(torch.float32)
        y = self._op(x2, self.values, self.op.D, self.op.column_info, self.raw_indices, self.n_keep, self.op.format,
                     self.op.layout_ns, self.vec_len, self.path)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features)

    def dense_weight(self):
        """The pruned weight as a dense (out_features, in_features) tensor (zeros where pruned),
        rebuilt from the compressed operand: what the layer multiplies by."""
        torch = _torch()
        dense = torch.zeros((self.in_features, self.out_features), dtype=torch.float32, device=self.values.device)
        dense.scatter_(0, _dense_rows(self.raw_indices, self.n_keep), self.values.detach())
        return dense.t().contiguous()
