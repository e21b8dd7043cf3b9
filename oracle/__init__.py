"""ctypes front end of the parity checker.  TEST INFRASTRUCTURE ONLY.

``oracle`` wraps two shared objects that live beside this file:

* ``libnm_oracle.so``  -- the plain-C restatement in ``nm_oracle.c``;
* ``_ref/libnmspmm_ref.so`` -- the reference's own host code compiled unchanged
  (present when it was built where the reference checkout exists).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module.  The shipped package never does: its product path is the CUDA library.
All arrays are numpy; shapes follow the reference's formats
(include/utils.h:10-66 of the reference):

* ``A_km``   float32 (K, M) C-contiguous  == col-major M x K  (``A[i + k*M]``)
* ``B_col``  float32 (N, W) C-contiguous  == col-major W x N  (``B[w + j*W]``)
* ``D_col``  int32   (Q, W) C-contiguous  == ``D[w + a*W]``, global k
* ``DT``     int32   (W, Q) row-major, window-local k
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libnm_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libnmspmm_ref.so")

_i32p = ctypes.POINTER(ctypes.c_int)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def reference_checkout() -> str:
    """Where the reference's sources lie, if anywhere: the directory named by
    NMSPMM_REFERENCE_DIR, else a checkout called ``reference`` beside this repository."""
    for cand in (os.environ.get("NMSPMM_REFERENCE_DIR"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "src", "preprocessing.cu")):
            return cand
    return ""


def build(verbose: bool = False) -> None:
    """Compile the C restatement (and the reference objects when the reference
    checkout is present).  Building the checker is not using it."""
    cmd = ["make", "-C", _HERE, "all"]
    ref = reference_checkout()
    if ref:
        cmd.append("REF=" + ref)
    out = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or out.returncode != 0:
        print(out.stdout + out.stderr)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed")


def _ptr(a: np.ndarray, ty):
    return a.ctypes.data_as(ty)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class _Impl:
    """One implementation (restatement or compiled reference) behind one API."""

    def __init__(self, path: str, prefix: str, kind: str):
        self.kind = kind
        self.path = path
        self._lib = ctypes.CDLL(path)
        self._p = prefix
        g = lambda n: getattr(self._lib, prefix + n)
        self._trans = g("trans_index")
        self._high = g("preprocess_high")
        self._low = g("preprocess_low")
        self._nthreads = g("num_threads")
        self._nthreads.restype = ctypes.c_int
        self._set_threads = g("set_num_threads")

    # ---- preprocessing -------------------------------------------------
    def trans_index(self, DT, pruning_N: int, pruning_M: int):
        """src/preprocessing.cu:3-15.  Returns (DT', pruning_N', pruning_M')."""
        DT = _i32(DT).copy()
        W, Q = DT.shape
        pn, pm = ctypes.c_int(pruning_N), ctypes.c_int(pruning_M)
        self._trans(_ptr(DT, _i32p), W, Q * 32, Q, ctypes.byref(pn), ctypes.byref(pm))
        return DT, pn.value, pm.value

    def preprocess_low(self, DT, Ns: int) -> np.ndarray:
        """src/preprocessing.cu:80-100.  Returns the re-tiled index buffer (flat W*Q)."""
        DT = _i32(DT).copy()
        W, Q = DT.shape
        self._low(_ptr(DT, _i32p), W, Q, Ns)
        return DT.reshape(-1)

    def preprocess_high(self, DT, pruning_M: int, pruning_N: int, Ns: int, tail_fill: int = -7):
        """src/preprocessing.cu:17-78.  Returns (D flat, column_info flat).

        ``column_info`` has the caller-side size of the reference driver
        (tests/test_nmspmm.cu:23): one extra window that the function never
        writes; it keeps ``tail_fill`` so that tests can see it untouched."""
        DT = _i32(DT).copy()
        W, Q = DT.shape
        n_ci = ((W // pruning_N) * (Q * 32 // Ns) + 1) * pruning_M
        ci = np.full(n_ci, tail_fill, dtype=np.int32)
        self._high(_ptr(ci, _i32p), pruning_M, pruning_N, _ptr(DT, _i32p), W, Q, Q * 32, Ns)
        return DT.reshape(-1), ci

    # ---- multiply ------------------------------------------------------
    def num_threads(self) -> int:
        return int(self._nthreads())

    def set_num_threads(self, n: int) -> None:
        self._set_threads(int(n))

    def nm_gemm_f32(self, A_km, B_col, D_col, C0=None) -> np.ndarray:
        """include/utils.h:82-95: C(+)= A*B, float accumulation.  Returns C (M, N)."""
        A_km, B_col, D_col = _f32(A_km), _f32(B_col), _i32(D_col)
        K, M = A_km.shape
        N, W = B_col.shape
        C = np.zeros((M, N), dtype=np.float32) if C0 is None else _f32(C0).copy()
        if self.kind == "reference":
            self._lib.ref_nm_gemm_cpu(_ptr(A_km, _f32p), _ptr(B_col, _f32p), _ptr(D_col, _i32p),
                                      _ptr(C, _f32p), M, N, K, W)
        else:
            self._lib.oracle_nm_gemm_f32(_ptr(A_km, _f32p), _ptr(B_col, _f32p), _ptr(D_col, _i32p),
                                         _ptr(C, _f32p), M, N, K, W, 0, M)
        return C


class _Oracle(_Impl):
    def nm_gemm_f64(self, A_km, B_col, D_col) -> np.ndarray:
        """The same sum in double precision (tolerance anchor of the TF32 path)."""
        A_km, B_col, D_col = _f32(A_km), _f32(B_col), _i32(D_col)
        K, M = A_km.shape
        N, W = B_col.shape
        C = np.zeros((M, N), dtype=np.float64)
        self._lib.oracle_nm_gemm_f64(_ptr(A_km, _f32p), _ptr(B_col, _f32p), _ptr(D_col, _i32p),
                                     _ptr(C, _f64p), M, N, K, W, 0, M)
        return C

    def nm_gemm_packed(self, A_km, BT, D_packed, column_info, ws: int, Ns: int) -> np.ndarray:
        """The product from the GPU-side operands (row-major BT, re-tiled D,
        optional column_info), indexed as the reference kernels index them."""
        A_km, BT, D_packed = _f32(A_km), _f32(BT), _i32(D_packed)
        K, M = A_km.shape
        W, N = BT.shape
        C = np.zeros((M, N), dtype=np.float32)
        ci = None if column_info is None else _ptr(_i32(column_info), _i32p)
        self._lib.oracle_nm_gemm_packed(_ptr(A_km, _f32p), _ptr(BT, _f32p), _ptr(D_packed, _i32p), ci,
                                        _ptr(C, _f32p), M, N, K, W, ws, Ns)
        return C


def have_reference() -> bool:
    return os.path.exists(_REF_SO)


_cache = {}


def restatement() -> _Oracle:
    """The C restatement (built on first use if the shared object is missing)."""
    if "o" not in _cache:
        if not os.path.exists(_ORACLE_SO):
            build()
        _cache["o"] = _Oracle(_ORACLE_SO, "oracle_", "port")
    return _cache["o"]


def reference() -> _Impl:
    """The reference's own host code, compiled unchanged.  Raises if it was not built."""
    if "r" not in _cache:
        if not have_reference():
            raise FileNotFoundError(_REF_SO + " (run `make -C oracle ref` where the reference checkout exists)")
        _cache["r"] = _Impl(_REF_SO, "ref_", "reference")
    return _cache["r"]
