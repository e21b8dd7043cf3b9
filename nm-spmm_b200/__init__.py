"""nm_spmm_b200 -- host-side mirror of the NM-SpMM operator interface over the
sm_100a C-ABI library (``libnmspmm_b200.so``, built in-tree by ``build.py``).

The functions named like the reference's API (``PreProcessing_low_sparsity``,
``PreProcessing_high_sparsity``, ``transIndex``, ``nmGEMM_*_matrices_*_sparsity``;
include/NM-SpMM.h:10-24 of the reference) take the same arguments with the same
meaning; device buffers are torch CUDA tensors, host buffers numpy arrays.
``NMSpMM`` bundles a packed sparse operand that stays resident on the GPU.

There is no CPU fallback: every operation calls the CUDA library and raises if it
is missing or reports an error.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

from . import build, formats, linear, sharding, tuner  # noqa: F401  (in-tree nvcc build; seeded operands; layer; multi-GPU partition; plan tuner)

_HERE = os.path.dirname(os.path.abspath(__file__))
# NMSPMM_LIBRARY selects another build of the same library (A/B comparisons of kernels).
LIB_PATH = os.environ.get("NMSPMM_LIBRARY") or os.path.join(_HERE, "libnmspmm_b200.so")

OK, INVALID_ARGUMENT, UNSUPPORTED, CUDA_ERROR, WORKSPACE_TOO_SMALL, DEVICE_TIMEOUT = range(6)
PATH_FP32, PATH_TF32 = 0, 1
(TILE_AUTO, TILE_128x128, TILE_64x128, TILE_32x128, TILE_16x128, TILE_128x256, TILE_16x256, TILE_32x256,
 TILE_128x256_GATHER, TILE_128x256_EXPAND) = range(10)   # nmspmm_tile_id
FORMAT_LOW, FORMAT_HIGH = 0, 1
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2               # nmspmm_dtype
VEC_LEN = 32

# Every symbol include/nmspmm_b200.h declares.
C_ABI_SYMBOLS = (
    "nmspmm_status_string", "nmspmm_last_cuda_error", "nmspmm_version",
    "nmspmm_trans_index_device", "nmspmm_preprocess_low_device", "nmspmm_preprocess_high_device",
    "nmspmm_trans_index_host", "nmspmm_preprocess_low_host", "nmspmm_preprocess_high_host",
    "nmspmm_test_short_fill", "nmspmm_set_tile_band", "nmspmm_tuned_plan_set", "nmspmm_tuned_plan_load", "nmspmm_tuned_plan_clear",
    "nmspmm_tuned_plan_count", "nmspmm_gemm_workspace_bytes", "nmspmm_gemm", "nmspmm_gemm_row_major",
    "nmspmm_gemm_row_major_workspace_bytes", "nmspmm_gemm_row_major_16", "nmspmm_gemm_row_major_16_workspace_bytes",
    "nmspmm_widen_device", "nmspmm_gemm_with_cached_workspace", "nmspmm_device_status",
    "nmspmm_gemm_plan", "nmspmm_gemm_host", "nmspmm_release_cached", "nmspmm_measure_ffma_peak",
    "nmspmm_gemm_static_scratch", "nmspmm_gemm_gather", "nmspmm_prune_device",
)
STATIC_SCRATCH_BYTES = 16 << 20     # NMSPMM_STATIC_SCRATCH_BYTES of include/nmspmm_b200.h


class GemmDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("M", "N", "K", "n_keep", "format", "layout_ns", "path", "split_k", "tile", "vec_len")]


class PlanInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("tile", "tile_m", "tile_n", "split_k", "tiles_x", "tiles_y", "n_virtual", "grid", "stream_k",
                 "n_dp", "threads", "smem_bytes", "stages")]


class NMSpMMError(RuntimeError):
    def __init__(self, where: str, status: int):
        self.status = status
        msg = _lib.nmspmm_status_string(status).decode() if _lib is not None else str(status)
        cuda = _lib.nmspmm_last_cuda_error() if _lib is not None else 0
        super().__init__(f"{where}: {msg} (status {status}, cuda error {cuda})")


_lib = None


def load_library():
    """dlopen the CUDA library and declare its C-ABI.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc). "
            "There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name in C_ABI_SYMBOLS:
        getattr(lib, name)                      # AttributeError if the build lost a symbol
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.nmspmm_status_string.restype = ctypes.c_char_p
    lib.nmspmm_status_string.argtypes = [ci]
    lib.nmspmm_trans_index_device.argtypes = [vp, ci, ci, ci, ci, vp]
    lib.nmspmm_preprocess_low_device.argtypes = [vp, vp, ci, ci, ci, vp]
    lib.nmspmm_preprocess_high_device.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.nmspmm_trans_index_host.argtypes = [vp, ci, ci, ci, ctypes.POINTER(ci), ctypes.POINTER(ci)]
    lib.nmspmm_preprocess_low_host.argtypes = [vp, ci, ci, ci]
    lib.nmspmm_preprocess_high_host.argtypes = [vp, ci, ci, vp, ci, ci, ci, ci]
    lib.nmspmm_gemm_workspace_bytes.restype = sz
    lib.nmspmm_gemm_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc)]
    lib.nmspmm_gemm.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp, sz, vp]
    lib.nmspmm_tuned_plan_set.argtypes = [ctypes.POINTER(GemmDesc), ci, ci]
    lib.nmspmm_tuned_plan_load.argtypes = [ctypes.c_char_p]
    lib.nmspmm_gemm_row_major_workspace_bytes.restype = sz
    lib.nmspmm_gemm_row_major_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc)]
    lib.nmspmm_gemm_row_major.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp, sz, vp]
    lib.nmspmm_gemm_row_major_16_workspace_bytes.restype = sz
    lib.nmspmm_gemm_row_major_16_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc)]
    lib.nmspmm_gemm_row_major_16.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_int, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.nmspmm_widen_device.argtypes = [ctypes.c_int, vp, vp, sz, vp]
    lib.nmspmm_gemm_with_cached_workspace.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp]
    lib.nmspmm_gemm_static_scratch.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp, vp]
    lib.nmspmm_prune_device.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
    lib.nmspmm_gemm_gather.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, ctypes.POINTER(vp), ci, ctypes.c_longlong, ci,
                                       vp, sz, vp]
    lib.nmspmm_device_status.argtypes = [ctypes.POINTER(ci), ci]
    lib.nmspmm_gemm_plan.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(PlanInfo)]
    lib.nmspmm_gemm_host.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp, vp]
    lib.nmspmm_measure_ffma_peak.argtypes = [ctypes.POINTER(ctypes.c_double), ci, vp]
    _lib = lib
    return lib


def _check(where: str, status: int) -> None:
    if status != OK:
        raise NMSpMMError(where, status)


def _torch():
    import torch
    return torch


def _stream_ptr(stream=None):
    torch = _torch()
    s = torch.cuda.current_stream() if stream is None else stream
    return ctypes.c_void_p(s.cuda_stream)


def _dev_ptr(t, dtype, name: str):
    torch = _torch()
    if not (isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == dtype and t.is_contiguous()):
        raise TypeError(f"{name}: expected a contiguous CUDA tensor of {dtype}")
    return ctypes.c_void_p(t.data_ptr())


def n_keep_of(sparsity: float, pruning_M: int = 32) -> int:
    """Kept rows per window for the reference's float ``sparsity`` argument."""
    n = pruning_M * (1.0 - sparsity)
    if abs(n - round(n)) > 1e-4:
        raise ValueError(f"sparsity {sparsity} is not a multiple of 1/{pruning_M}")
    return int(round(n))


def format_of(n_keep: int) -> int:
    """The reference sends 75 % and 87.5 % to the high-sparsity family (tests/test_nmspmm.cu:13)."""
    return FORMAT_HIGH if n_keep in (8, 4) else FORMAT_LOW


# ----------------------------------------------------------------------------------
# Index packing.  Host arrays (numpy int32) are processed in place like the
# reference's functions; CUDA tensors go straight to the device kernels.
# ----------------------------------------------------------------------------------

def PreProcessing_low_sparsity(DT, W: int, Q: int, Ns: int):
    """In place on a host int32 array of W*Q elements (src/preprocessing.cu:80-100)."""
    lib = load_library()
    assert isinstance(DT, np.ndarray) and DT.dtype == np.int32 and DT.flags.c_contiguous and DT.size == W * Q
    _check("PreProcessing_low_sparsity", lib.nmspmm_preprocess_low_host(DT.ctypes.data, W, Q, Ns))


def PreProcessing_high_sparsity(column_info, pruning_M: int, pruning_N: int, DT, W: int, Q: int, N: int, Ns: int):
    """In place on host int32 arrays (src/preprocessing.cu:17-78)."""
    lib = load_library()
    assert isinstance(DT, np.ndarray) and DT.dtype == np.int32 and DT.flags.c_contiguous and DT.size == W * Q
    assert isinstance(column_info, np.ndarray) and column_info.dtype == np.int32 and column_info.flags.c_contiguous
    assert column_info.size >= (W // pruning_N) * (N // Ns) * pruning_M
    _check("PreProcessing_high_sparsity",
           lib.nmspmm_preprocess_high_host(column_info.ctypes.data, pruning_M, pruning_N, DT.ctypes.data, W, Q, N, Ns))


def transIndex(DT, W: int, N: int, Q: int, pruning_N: int, pruning_M: int):
    """In place on a host int32 array; returns the doubled (pruning_N, pruning_M)
    (the reference updates them through ``int&``, src/preprocessing.cu:3-15)."""
    lib = load_library()
    assert isinstance(DT, np.ndarray) and DT.dtype == np.int32 and DT.flags.c_contiguous and DT.size == W * Q
    pn, pm = ctypes.c_int(pruning_N), ctypes.c_int(pruning_M)
    _check("transIndex", lib.nmspmm_trans_index_host(DT.ctypes.data, W, N, Q, ctypes.byref(pn), ctypes.byref(pm)))
    return pn.value, pm.value


def trans_index_device(DT, pruning_N: int, pruning_M: int, stream=None) -> None:
    torch = _torch()
    W, Q = DT.shape
    _check("nmspmm_trans_index_device",
           load_library().nmspmm_trans_index_device(_dev_ptr(DT, torch.int32, "DT"), W, Q, pruning_N, pruning_M,
                                                    _stream_ptr(stream)))


def preprocess_low_device(DT, Ns: int, out=None, stream=None):
    """(W, Q) int32 CUDA tensor -> packed flat tensor of W*Q ints."""
    torch = _torch()
    W, Q = DT.shape
    D = torch.empty(W * Q, dtype=torch.int32, device=DT.device) if out is None else out
    _check("nmspmm_preprocess_low_device",
           load_library().nmspmm_preprocess_low_device(_dev_ptr(DT, torch.int32, "DT"), _dev_ptr(D, torch.int32, "D"),
                                                       W, Q, Ns, _stream_ptr(stream)))
    return D


def preprocess_high_device(DT, pruning_M: int, pruning_N: int, Ns: int, fuse_trans_index: bool = False,
                           out=None, column_info=None, stream=None):
    """(W, Q) int32 CUDA tensor -> (packed D flat, column_info flat incl. one extra -1 window).

    With ``fuse_trans_index`` the input holds raw 0..31 indices and ``pruning_M`` /
    ``pruning_N`` are the un-doubled values."""
    torch = _torch()
    W, Q = DT.shape
    pm = pruning_M * (2 if fuse_trans_index else 1)
    pn = pruning_N * (2 if fuse_trans_index else 1)
    n_ci = formats.column_info_ints(W, Q * VEC_LEN, pn, pm, Ns)
    D = torch.empty(W * Q, dtype=torch.int32, device=DT.device) if out is None else out
    ci = torch.empty(n_ci, dtype=torch.int32, device=DT.device) if column_info is None else column_info
    _check("nmspmm_preprocess_high_device",
           load_library().nmspmm_preprocess_high_device(
               _dev_ptr(DT, torch.int32, "DT"), _dev_ptr(D, torch.int32, "D"), _dev_ptr(ci, torch.int32, "column_info"),
               pruning_M, pruning_N, W, Q, Ns, 1 if fuse_trans_index else 0, pm, _stream_ptr(stream)))
    return D, ci


# ----------------------------------------------------------------------------------
# The multiply.
# ----------------------------------------------------------------------------------

def make_desc(M, N, K, n_keep, fmt, layout_ns, path=PATH_FP32, split_k=0, tile=0, vec_len=0) -> GemmDesc:
    return GemmDesc(M, N, K, n_keep, fmt, layout_ns, path, split_k, tile, vec_len)


def plan(desc: GemmDesc) -> PlanInfo:
    info = PlanInfo()
    _check("nmspmm_gemm_plan", load_library().nmspmm_gemm_plan(ctypes.byref(desc), ctypes.byref(info)))
    return info


def workspace_bytes(desc: GemmDesc) -> int:
    return int(load_library().nmspmm_gemm_workspace_bytes(ctypes.byref(desc)))


def gemm(desc: GemmDesc, A, B, D, column_info, C, workspace=None, stream=None) -> None:
    """nmspmm_gemm on CUDA tensors.  ``A`` is (K, M) (col-major M x K), ``B`` (W, N),
    ``C`` (M, N); ``workspace`` a uint8 tensor of at least workspace_bytes(desc)
    whose first bytes (the counters) are zero."""
    torch = _torch()
    ws_ptr, ws_bytes = ctypes.c_void_p(0), 0
    if workspace is not None:
        ws_ptr, ws_bytes = ctypes.c_void_p(workspace.data_ptr()), workspace.numel() * workspace.element_size()
    ci = ctypes.c_void_p(0) if column_info is None else _dev_ptr(column_info, torch.int32, "column_info")
    _check("nmspmm_gemm",
           load_library().nmspmm_gemm(ctypes.byref(desc), _dev_ptr(A, torch.float32, "A"), _dev_ptr(B, torch.float32, "B"),
                                      _dev_ptr(D, torch.int32, "D"), ci, _dev_ptr(C, torch.float32, "C"),
                                      ws_ptr, ws_bytes, _stream_ptr(stream)))


def prune_device(dense, n_keep: int, vec_len: int = 32, stream=None):
    """nmspmm_prune_device: vector-wise ``n_keep``:32 magnitude pruning of a dense (K, N)
    float32 CUDA tensor.  Returns (BT (W, N) float32, DT (W, N/32) int32) on the device."""
    torch = _torch()
    K, N = dense.shape
    W = K // 32 * n_keep
    BT = torch.empty((W, N), dtype=torch.float32, device=dense.device)
    DT = torch.empty((W, N // 32), dtype=torch.int32, device=dense.device)
    _check("nmspmm_prune_device",
           load_library().nmspmm_prune_device(_dev_ptr(dense, torch.float32, "dense"), BT.data_ptr(), DT.data_ptr(),
                                              K, N, n_keep, vec_len, _stream_ptr(stream)))
    return BT, DT


def gemm_gather(desc: GemmDesc, A, B, D, column_info, out_ptrs, ldc: int, col0: int, workspace=None, stream=None) -> None:
    """nmspmm_gemm_gather: the multiply of one rank's column slab, its finished tiles stored
    into every buffer of ``out_ptrs`` (device addresses as ints: this rank's full-width C and
    the peer-mapped full-width C of the other ranks) at column ``col0``, row stride ``ldc``."""
    torch = _torch()
    ws_ptr, ws_bytes = ctypes.c_void_p(0), 0
    if workspace is not None:
        ws_ptr, ws_bytes = ctypes.c_void_p(workspace.data_ptr()), workspace.numel() * workspace.element_size()
    ci = ctypes.c_void_p(0) if column_info is None else _dev_ptr(column_info, torch.int32, "column_info")
    ptrs = (ctypes.c_void_p * len(out_ptrs))(*[int(x) for x in out_ptrs])
    _check("nmspmm_gemm_gather",
           load_library().nmspmm_gemm_gather(ctypes.byref(desc), _dev_ptr(A, torch.float32, "A"), _dev_ptr(B, torch.float32, "B"),
                                             _dev_ptr(D, torch.int32, "D"), ci, ptrs, len(out_ptrs), int(ldc), int(col0),
                                             ws_ptr, ws_bytes, _stream_ptr(stream)))


def gemm_static_scratch(desc: GemmDesc, A, B, D, column_info, C, stream=None) -> None:
    """nmspmm_gemm_static_scratch on CUDA tensors: the multiply with the library's built-in
    scratch array instead of a caller workspace, for callers that may not allocate.  Calls
    that overlap on the GPU race on that array; sizes beyond STATIC_SCRATCH_BYTES raise."""
    torch = _torch()
    ci = ctypes.c_void_p(0) if column_info is None else _dev_ptr(column_info, torch.int32, "column_info")
    _check("nmspmm_gemm_static_scratch",
           load_library().nmspmm_gemm_static_scratch(
               ctypes.byref(desc), _dev_ptr(A, torch.float32, "A"), _dev_ptr(B, torch.float32, "B"),
               _dev_ptr(D, torch.int32, "D"), ci, _dev_ptr(C, torch.float32, "C"), _stream_ptr(stream)))


def device_status(clear: bool = True) -> int:
    """Raw device status word (0 = no bounded wait has given up)."""
    word = ctypes.c_int(0)
    rc = load_library().nmspmm_device_status(ctypes.byref(word), 1 if clear else 0)
    if rc not in (OK, DEVICE_TIMEOUT):
        raise NMSpMMError("nmspmm_device_status", rc)
    return word.value


_tuned_shadow = {}      # what this process has registered through the functions below (the C table has no read-back)


def set_tuned_plan(desc: GemmDesc, tile: int, split_k: int) -> None:
    """nmspmm_tuned_plan_set: descriptions like ``desc`` that leave tile and split to the library get these."""
    _check("nmspmm_tuned_plan_set", load_library().nmspmm_tuned_plan_set(ctypes.byref(desc), tile, split_k))
    _tuned_shadow[(desc.M, desc.N, desc.K, desc.n_keep, desc.format, desc.path, 64 if desc.vec_len == 64 else 32)] = (tile, split_k)


def load_tuned_plans(path: str) -> int:
    """Merges a table file (see tuner.py) into the running library.  Returns the entry count."""
    _check("nmspmm_tuned_plan_load", load_library().nmspmm_tuned_plan_load(path.encode()))
    _tuned_shadow.update(tuner.read_table(path))
    return int(load_library().nmspmm_tuned_plan_count())


def clear_tuned_plans() -> None:
    _check("nmspmm_tuned_plan_clear", load_library().nmspmm_tuned_plan_clear())
    _tuned_shadow.clear()


def tuned_plans_snapshot_and_clear():
    """For the tuner: candidates must be timed against the bare heuristics."""
    saved = dict(_tuned_shadow)
    default = tuner.default_table_path()
    env = os.environ.get("NMSPMM_TUNED_PLANS")
    src = env if env is not None else default
    if src and os.path.exists(src):
        saved = {**tuner.read_table(src), **saved}
    clear_tuned_plans()
    return saved


def tuned_plans_restore(saved) -> None:
    clear_tuned_plans()
    for key, (tile, split) in saved.items():
        M, N, K, n_keep, fmt, path, vec = key
        set_tuned_plan(make_desc(M, N, K, n_keep, fmt, 32, path, 0, 0, vec), tile, split)


def test_short_fill(enable: bool) -> int:
    """Test hook: while on, the multiply's stages never fill and its bounded waits run out
    (nmspmm_test_short_fill).  Returns the previous setting."""
    return int(load_library().nmspmm_test_short_fill(1 if enable else 0))


def _launcher(layout_ns: int, high: bool):
    def run(A, B, D, *rest):
        """Reference launcher signature on CUDA tensors:
        low : (A, B, D, C, M, N, K, W, sparsity, SPLIT_K)
        high: (A, B, D, column_info, C, M, N, K, W, sparsity, SPLIT_K)
        Runs on the current torch stream; scratch for split-K is cached by the library."""
        torch = _torch()
        if high:
            column_info, C, M, N, K, W, sparsity, SPLIT_K = rest
        else:
            (C, M, N, K, W, sparsity, SPLIT_K), column_info = rest, None
        n_keep = n_keep_of(sparsity)
        if high != (format_of(n_keep) == FORMAT_HIGH):
            # the reference prints "Not support!" and launches nothing (src/kernel_64x128_8x8.cu:264,584)
            raise NMSpMMError("launcher called for the other sparsity family", UNSUPPORTED)
        desc = make_desc(M, N, K, n_keep, FORMAT_HIGH if high else FORMAT_LOW, layout_ns,
                         split_k=SPLIT_K if SPLIT_K > 1 else 0)
        ci = ctypes.c_void_p(0) if column_info is None else _dev_ptr(column_info, torch.int32, "column_info")
        _check("nmspmm_gemm_with_cached_workspace",
               load_library().nmspmm_gemm_with_cached_workspace(
                   ctypes.byref(desc), _dev_ptr(A, torch.float32, "A"), _dev_ptr(B, torch.float32, "B"),
                   _dev_ptr(D, torch.int32, "D"), ci, _dev_ptr(C, torch.float32, "C"), _stream_ptr()))
    return run


nmGEMM_huge_matrices_low_sparsity = _launcher(128, False)
nmGEMM_huge_matrices_high_sparsity = _launcher(128, True)
nmGEMM_large_matrices_low_sparsity = _launcher(64, False)
nmGEMM_large_matrices_high_sparsity = _launcher(64, True)
nmGEMM_medium_matrices_low_sparsity = _launcher(64, False)
nmGEMM_medium_matrices_high_sparsity = _launcher(64, True)
nmGEMM_small_matrices_low_sparsity = _launcher(32, False)
nmGEMM_small_matrices_high_sparsity = _launcher(32, True)


def gemm_host(desc: GemmDesc, A_km, BT, DT, C, on_current_stream: bool = False) -> None:
    """End to end on HOST buffers (numpy arrays or pinned torch CPU tensors):
    H2D of A, B, raw DT; index packing and multiply on the GPU; D2H of C.
    Returns when C is complete.  ``on_current_stream`` issues the work on torch's
    current stream (so that CUDA events recorded there bracket it)."""
    lib = load_library()

    def ptr(x):
        return ctypes.c_void_p(x.ctypes.data if isinstance(x, np.ndarray) else x.data_ptr())
    st = _stream_ptr() if on_current_stream else ctypes.c_void_p(0)
    _check("nmspmm_gemm_host", lib.nmspmm_gemm_host(ctypes.byref(desc), ptr(A_km), ptr(BT), ptr(DT), ptr(C), st))


def gpu_numa_probe(device_index: int) -> dict:
    """Where the GPU hangs off the host, read from sysfs: ``{"bdf", "node", "cpus", "why_not"}``.
    ``cpus`` is None (and ``why_not`` says which step gave nothing) on single-node hosts, which
    report node -1, and where the container hides the PCI tree."""
    out = {"bdf": None, "node": None, "cpus": None, "why_not": None}
    try:
        pr = _torch().cuda.get_device_properties(device_index)
        out["bdf"] = bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
    except Exception as e:
        out["why_not"] = f"no PCI address from the device properties ({type(e).__name__})"
        return out
    try:
        out["node"] = node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
    except Exception as e:
        out["why_not"] = f"/sys/bus/pci/devices/{bdf}/numa_node unreadable ({type(e).__name__})"
        return out
    if node < 0:
        out["why_not"] = "sysfs reports NUMA node -1 for the GPU"
        return out
    try:
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        out["cpus"] = cpus or None
        if not cpus:
            out["why_not"] = f"node{node} lists no CPUs"
    except Exception as e:
        out["why_not"] = f"/sys/devices/system/node/node{node}/cpulist unreadable ({type(e).__name__})"
    return out


def gpu_numa_cpus(device_index: int):
    """CPUs of the NUMA node the GPU hangs off (from sysfs), or None when that cannot be read."""
    return gpu_numa_probe(device_index)["cpus"]


def bind_host_to_gpu(device_index: int) -> bool:
    """Pins the calling process to the CPUs next to the GPU, so that pinned host buffers
    allocated afterwards (first touch) and the copies that read them stay on that NUMA node:
    what the host-buffer entry point wants when every GPU of a box runs one.  Returns whether
    anything was changed; os.sched_setaffinity(0, saved) undoes it."""
    cpus = gpu_numa_cpus(device_index)
    if not cpus:
        return False
    allowed = os.sched_getaffinity(0) & cpus
    if not allowed:
        return False
    os.sched_setaffinity(0, allowed)
    return True


def dtype_id(torch_dtype) -> int:
    """nmspmm_dtype of a torch dtype (float32, float16, bfloat16)."""
    torch = _torch()
    try:
        return {torch.float32: DTYPE_F32, torch.float16: DTYPE_F16, torch.bfloat16: DTYPE_BF16}[torch_dtype]
    except KeyError:
        raise NMSpMMError("dtype_id", UNSUPPORTED) from None


def widen_device(t):
    """nmspmm_widen_device: a contiguous float16 / bfloat16 CUDA tensor (numel % 4 == 0) as float32,
    exactly -- what weights kept in 16 bits go through once, before they are pruned and compressed."""
    torch = _torch()
    assert t.is_contiguous()
    out = torch.empty(t.shape, dtype=torch.float32, device=t.device)
    _check("nmspmm_widen_device", load_library().nmspmm_widen_device(dtype_id(t.dtype), ctypes.c_void_p(t.data_ptr()),
                                                                     ctypes.c_void_p(out.data_ptr()), t.numel(), _stream_ptr()))
    return out


def set_tile_band(band: int) -> int:
    """nmspmm_set_tile_band: -1 automatic, 0 row by row, n bands of n tile columns (TF32 path).  Returns the previous value."""
    return int(load_library().nmspmm_set_tile_band(int(band)))


def measure_ffma_peak(packed: bool = False) -> float:
    """Sustained FP32 FMA rate of the current GPU in TFLOP/s (register-only kernel);
    ``packed`` selects the two-lane packed FMA of sm_100 instead of scalar FFMA."""
    out = ctypes.c_double(0.0)
    _check("nmspmm_measure_ffma_peak",
           load_library().nmspmm_measure_ffma_peak(ctypes.byref(out), 1 if packed else 0, _stream_ptr()))
    return out.value


class NMSpMM:
    """A vector-wise N:M sparse right-hand operand packed and resident on one GPU.

    ``B`` (W, N) float32 and the packed ``D`` / ``column_info`` live on the device;
    ``matmul`` multiplies any (K, M) col-major ``A`` against them."""

    def __init__(self, BT, DT, K: int, n_keep: int, layout_ns: int = 128, fmt: Optional[int] = None, device=None,
                 vec_len: int = VEC_LEN):
        torch = _torch()
        load_library()
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.K, self.n_keep, self.layout_ns = K, n_keep, layout_ns
        self.vec_len = vec_len      # 64: adjacent pairs of index lists are equal (what the generators and prune_device produce)
        self.format = format_of(n_keep) if fmt is None else fmt
        self.B = torch.as_tensor(BT, dtype=torch.float32).to(dev).contiguous()
        self.W, self.N = self.B.shape
        raw = torch.as_tensor(DT, dtype=torch.int32).to(dev).contiguous()
        assert raw.shape == (self.W, self.N // VEC_LEN)
        if self.format == FORMAT_HIGH:
            self.D, self.column_info = preprocess_high_device(raw, 32, n_keep, layout_ns, fuse_trans_index=True)
        else:
            self.D, self.column_info = preprocess_low_device(raw, layout_ns), None
        self._workspace = None

    @classmethod
    def from_problem(cls, p: "formats.NMProblem", layout_ns: int = 128, fmt: Optional[int] = None, device=None):
        return cls(p.BT, p.DT, p.K, p.n_keep, layout_ns, fmt, device, vec_len=p.vec_len)

    @classmethod
    def from_dense(cls, dense, n_keep: int, vec_len: int = 32, layout_ns: int = 128, fmt: Optional[int] = None):
        """Prune a dense (K, N) float32 CUDA weight to ``n_keep``:32 by per-vector L2 magnitude,
        compress and pack it, all on the device (prune_device, then the packing kernels)."""
        BT, DT = prune_device(dense, n_keep, vec_len)
        return cls(BT, DT, dense.shape[0], n_keep, layout_ns, fmt, dense.device, vec_len=vec_len)

    def desc(self, M: int, path: int = PATH_FP32, split_k: int = 0, tile: int = 0) -> GemmDesc:
        return make_desc(M, self.N, self.K, self.n_keep, self.format, self.layout_ns, path, split_k, tile, self.vec_len)

    def _scratch(self, nbytes: int):
        torch = _torch()
        if nbytes == 0:
            return None
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.B.device)
        return self._workspace

    def matmul(self, A, path: int = PATH_FP32, split_k: int = 0, tile: int = 0, out=None):
        """C (M, N) = A . B for ``A`` given as a (K, M) float32 CUDA tensor."""
        torch = _torch()
        K, M = A.shape
        assert K == self.K
        d = self.desc(M, path, split_k, tile)
        C = torch.empty((M, self.N), dtype=torch.float32, device=A.device) if out is None else out
        gemm(d, A, self.B, self.D, self.column_info, C, self._scratch(workspace_bytes(d)))
        return C

    def matmul_rows(self, x, path: int = PATH_FP32, split_k: int = 0, tile: int = 0, out=None):
        """C (M, N) = x . B for ``x`` given row-major as an (M, K) CUDA tensor (any M >= 1): the
        library transposes on the GPU ahead of the multiply (nmspmm_gemm_row_major).  ``x`` may
        be float32, or float16 / bfloat16: then the result has that dtype too, the widening is
        part of the transposition and one pass rounds the result (nmspmm_gemm_row_major_16)."""
        torch = _torch()
        M, K = x.shape
        assert K == self.K and x.is_contiguous()
        dtype = dtype_id(x.dtype)
        lib = load_library()
        d = self.desc(M, path, split_k, tile)
        sizer = lib.nmspmm_gemm_row_major_workspace_bytes if dtype == DTYPE_F32 else lib.nmspmm_gemm_row_major_16_workspace_bytes
        need = int(sizer(ctypes.byref(d)))
        if need == 0:
            raise NMSpMMError("nmspmm_gemm_row_major_workspace_bytes", UNSUPPORTED)
        ws = self._scratch(need)
        C = torch.empty((M, self.N), dtype=x.dtype, device=x.device) if out is None else out
        assert C.dtype == x.dtype and C.is_contiguous()
        col = ctypes.c_void_p(self.column_info.data_ptr()) if self.column_info is not None else ctypes.c_void_p(0)
        ptrs = (ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(self.B.data_ptr()), ctypes.c_void_p(self.D.data_ptr()), col,
                ctypes.c_void_p(C.data_ptr()), ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream_ptr())
        if dtype == DTYPE_F32:
            _check("nmspmm_gemm_row_major", lib.nmspmm_gemm_row_major(ctypes.byref(d), *ptrs))
        else:
            _check("nmspmm_gemm_row_major_16", lib.nmspmm_gemm_row_major_16(ctypes.byref(d), dtype, *ptrs))
        return C

    def matmul_into(self, A, out_ptrs, ldc: int, col0: int, path: int = PATH_FP32, split_k: int = 0, tile: int = 0) -> None:
        """The same multiply with its tiles stored into every buffer of ``out_ptrs`` (device
        addresses) at column ``col0`` with row stride ``ldc``: the fused all-gather of a
        column-sharded rank (see sharding.ShardedNMSpMM)."""
        K, M = A.shape
        assert K == self.K
        d = self.desc(M, path, split_k, tile)
        gemm_gather(d, A, self.B, self.D, self.column_info, out_ptrs, ldc, col0, self._scratch(workspace_bytes(d)))
