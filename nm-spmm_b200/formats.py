"""Seeded synthetic operands in the reference's on-host formats.

The reference fills its operands with ``rand()`` / ``std::random_device``
(include/utils.h:22,51 of the reference), which cannot be reproduced.  This
module produces the same *formats* (include/utils.h:10-66) from one counter-based
generator (splitmix64 keyed by seed, tensor id and element number), so that a
test, the benchmark and the CPU checker all see identical inputs.

Formats (V = 32 columns share one index list; windows of 32 consecutive k):

* ``A_km``   float32 (K, M) C-contiguous == col-major M x K, ``A[i + k*M]``
* ``BT``     float32 (W, N) row-major compressed values (what the GPU reads)
* ``B_col``  float32 (N, W) == col-major ``B[w + j*W]`` (what the CPU multiply reads)
* ``DT``     int32   (W, Q) window-local k of every kept row, ascending per window
* ``D_col``  int32   (Q, W) == ``D[w + a*W]``, global k
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

VEC_LEN = 32
WINDOW = 32

_U64 = np.uint64
_MASK = (1 << 64) - 1


def _splitmix64(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on a uint64 array (wraps modulo 2**64)."""
    with np.errstate(over="ignore"):
        z = x + _U64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> _U64(30))) * _U64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> _U64(27))) * _U64(0x94D049BB133111EB)
        return z ^ (z >> _U64(31))


def random_bits(seed: int, tensor_id: int, n: int, offset: int = 0) -> np.ndarray:
    """64 random bits for elements offset..offset+n-1 of tensor ``tensor_id``."""
    key = int(_splitmix64(np.array([(seed * 0x100000001B3 + tensor_id * 0x9E3779B1) & _MASK], dtype=_U64))[0])
    ctr = np.arange(offset, offset + n, dtype=_U64)
    with np.errstate(over="ignore"):
        return _splitmix64(ctr * _U64(0xD1342543DE82EF95) + _U64(key))


def uniform_pm1(seed: int, tensor_id: int, n: int) -> np.ndarray:
    """float32 uniform in [-1, 1) from the top 24 bits."""
    bits = random_bits(seed, tensor_id, n) >> _U64(40)
    return (bits.astype(np.float32) * np.float32(2.0 / (1 << 24)) - np.float32(1.0)).astype(np.float32)


def normal(seed: int, tensor_id: int, n: int, std: float = 1.0) -> np.ndarray:
    """float32 N(0, std^2) by Box-Muller on two 32-bit halves of the stream."""
    bits = random_bits(seed, tensor_id, n)
    u1 = ((bits >> _U64(32)).astype(np.float64) + 1.0) / 4294967296.0  # (0, 1]
    u2 = (bits & _U64(0xFFFFFFFF)).astype(np.float64) / 4294967296.0
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)


@dataclass
class NMProblem:
    """One C(M x N) = A(M x K) . B(K x N) instance with B in N:M vector-wise form."""

    M: int
    N: int
    K: int
    n_keep: int          # kept rows per 32-row window (the "N" of N:M)
    A_km: np.ndarray
    BT: np.ndarray
    DT: np.ndarray
    vec_len: int = VEC_LEN   # 32, or 64 (stored as duplicated adjacent 32-wide index vectors)

    @property
    def W(self) -> int:
        return self.K // WINDOW * self.n_keep

    @property
    def Q(self) -> int:
        return self.N // VEC_LEN

    @property
    def sparsity(self) -> float:
        return 1.0 - self.n_keep / WINDOW

    @property
    def B_col(self) -> np.ndarray:
        return np.ascontiguousarray(self.BT.T)

    @property
    def D_col(self) -> np.ndarray:
        """Global-k indices, col-major (include/utils.h:60 of the reference)."""
        w = np.arange(self.W, dtype=np.int32)[:, None]
        return np.ascontiguousarray((self.DT + (w // self.n_keep) * WINDOW).T.astype(np.int32))

    def dense_B(self) -> np.ndarray:
        """B expanded to (K, N) with explicit zeros (small problems only)."""
        B = np.zeros((self.K, self.N), dtype=np.float32)
        kk = self.D_col.T                                  # (W, Q) global k
        cols = np.arange(self.N)
        for w in range(self.W):
            B[kk[w, cols // VEC_LEN], cols] = self.BT[w]
        return B

    def useful_flops(self) -> float:
        return 2.0 * self.M * self.N * self.W

    def dense_flops(self) -> float:
        return 2.0 * self.M * self.N * self.K


def random_indices(seed: int, K: int, Q: int, n_keep: int, vec_len: int = VEC_LEN, tensor_id: int = 3) -> np.ndarray:
    """``DT`` (W, Q): per (32-row window, vector) choose ``n_keep`` rows without
    replacement, ascending -- the distribution of include/utils.h:49-63 of the
    reference.  ``vec_len`` 64 makes column pairs of 32-wide vectors share a list."""
    nwin = K // WINDOW
    qv = Q // (vec_len // VEC_LEN)
    keys = random_bits(seed, tensor_id, nwin * qv * WINDOW).reshape(nwin, qv, WINDOW)
    order = np.argsort(keys, axis=2, kind="stable")[:, :, :n_keep]
    local = np.sort(order, axis=2).astype(np.int32)            # (nwin, qv, n_keep)
    DT = local.transpose(0, 2, 1).reshape(nwin * n_keep, qv)    # (W, qv)
    if vec_len != VEC_LEN:
        DT = np.repeat(DT, vec_len // VEC_LEN, axis=1)
    return np.ascontiguousarray(DT)


def make_random(M: int, N: int, K: int, n_keep: int, seed: int = 0, vec_len: int = VEC_LEN,
                a_dist: str = "uniform") -> NMProblem:
    """Uniform[-1,1) A and kept values, random sorted indices."""
    assert K % WINDOW == 0 and N % vec_len == 0
    W = K // WINDOW * n_keep
    a = uniform_pm1(seed, 1, M * K) if a_dist == "uniform" else normal(seed, 1, M * K)
    A_km = np.ascontiguousarray(a.reshape(M, K).T)             # logical A[i][k] -> stored (K, M)
    BT = uniform_pm1(seed, 2, W * N).reshape(W, N)
    DT = random_indices(seed, K, N // VEC_LEN, n_keep, vec_len)
    return NMProblem(M, N, K, n_keep, A_km, BT, DT, vec_len)


def prune_magnitude(Bd: np.ndarray, n_keep: int, vec_len: int = VEC_LEN):
    """Vector-wise N:M magnitude pruning of a dense (K, N) weight: in every
    32-row window keep, per vector, the ``n_keep`` rows of largest L2 norm over
    the vector's columns (ties to the lower row); indices ascending.
    Returns (BT (W, N), DT (W, Q))."""
    K, N = Bd.shape
    nwin, qv = K // WINDOW, N // vec_len
    blk = Bd.reshape(nwin, WINDOW, qv, vec_len)
    score = (blk.astype(np.float64) ** 2).sum(axis=3)                     # (nwin, 32, qv)
    order = np.argsort(-score, axis=1, kind="stable")[:, :n_keep, :]
    local = np.sort(order, axis=1).astype(np.int32)                       # (nwin, n_keep, qv)
    rows = local + (np.arange(nwin, dtype=np.int32) * WINDOW)[:, None, None]
    rows_full = np.repeat(rows.reshape(nwin * n_keep, qv), vec_len, axis=1)  # (W, N)
    BT = np.take_along_axis(Bd, rows_full, axis=0).astype(np.float32)
    DT = np.repeat(local.reshape(nwin * n_keep, qv), vec_len // VEC_LEN, axis=1)
    return np.ascontiguousarray(BT), np.ascontiguousarray(DT)


def make_llm_linear(tokens: int, N: int = 11008, K: int = 4096, n_keep: int = 8, seed: int = 0) -> NMProblem:
    """Activations N(0,1) (tokens x K) against a N(0, 0.02^2) weight pruned to
    ``n_keep``:32 by per-vector L2 magnitude."""
    a = normal(seed, 1, tokens * K)
    A_km = np.ascontiguousarray(a.reshape(tokens, K).T)
    Bd = normal(seed, 2, K * N, std=0.02).reshape(K, N)
    BT, DT = prune_magnitude(Bd, n_keep)
    return NMProblem(tokens, N, K, n_keep, A_km, BT, DT)


# ---- host-side restatement of the index packing (numpy, vectorised) -------------
# Used by the sharding logic and by CPU tests of the host code; the product's
# packing runs on the GPU (csrc/preprocess.cu).

def retile(DT: np.ndarray, Ns: int) -> np.ndarray:
    """[W][Q] -> [Q/Qs][W][Qs] (flat), Qs = Ns/32 (src/preprocessing.cu:80-100 of the reference)."""
    W, Q = DT.shape
    Qs = Ns // VEC_LEN
    return np.ascontiguousarray(DT.reshape(W, Q // Qs, Qs).transpose(1, 0, 2)).reshape(-1)


def column_info_ints(W: int, N: int, pruning_N: int, pruning_M: int, Ns: int) -> int:
    """Size the reference driver allocates for ``column_info`` (tests/test_nmspmm.cu:23):
    one list per (Ns block, window) plus one extra window."""
    return ((W // pruning_N) * (N // Ns) + 1) * pruning_M
