"""Seeded random shapes through both arithmetic paths, every schedule the planner can pick
(whole tiles, balanced tail, in-kernel and separate reductions, K slices) against the CPU
checker.  Shapes are small enough for the checker to finish in well under a second each."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cases():
    rng = np.random.default_rng(2024)
    out = []
    for i in range(40):
        n_keep = int(rng.choice([32, 16, 12, 8, 4]))
        M = int(rng.integers(1, 80)) * 4                       # any multiple of 4 up to 316
        N = int(rng.integers(1, 9)) * 128
        K = int(rng.integers(1, 33)) * 64
        layout = int(rng.choice([32, 64, 128]))
        split_k = int(rng.choice([0, 0, 1, 2, 3, 5, 9]))
        tile = int(rng.choice([0, 0, 1, 2, 3, 4, 5]))
        out.append((i, M, N, K, n_keep, layout, split_k, tile))
    return out


@pytest.mark.parametrize("case", _cases(), ids=lambda c: "m%d_n%d_k%d_keep%d_ns%d_s%d_t%d" % c[1:])
def test_random_shapes_both_paths(pkg, orc, case):
    i, M, N, K, n_keep, layout, split_k, tile = case
    p = pkg.formats.make_random(M, N, K, n_keep, seed=5000 + i)
    op = pkg.NMSpMM.from_problem(p, layout_ns=layout)
    A = torch.from_numpy(p.A_km).cuda()
    want32 = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col).astype(np.float64)
    scale = np.linalg.norm(want32)
    got = op.matmul(A, split_k=split_k, tile=tile).cpu().numpy()
    assert np.linalg.norm(got - want32) / scale <= 1e-5
    tf_tile = tile if tile in (0, 1, 5) else 0               # the tensor-core path has the 128-row tiles only
    got_tf = op.matmul(A, path=pkg.PATH_TF32, split_k=split_k, tile=tf_tile).cpu().numpy()
    assert np.linalg.norm(got_tf - want32) / scale <= 2e-3
    assert pkg.device_status() == 0
