"""Pins the CPU checker (oracle/nm_oracle.c) to the reference: against fixtures
the reference's own code produced (tests/golden/make_golden.py), against the
worked index-packing example, and -- where the compiled reference is present --
against the reference itself on fresh inputs."""
import numpy as np
import pytest

import oracle

KAT_DT = np.array([1, 0, 2, 3, 5, 7, 6, 4, 0, 2, 2, 1, 3, 3, 7, 6,
                   4, 0, 1, 1, 6, 5, 2, 7, 0, 1, 3, 2, 2, 4, 5, 3], dtype=np.int32).reshape(8, 4)
KAT_LOW = [1, 0, 5, 7, 0, 2, 3, 3, 4, 0, 6, 5, 0, 1, 2, 4, 2, 3, 6, 4, 2, 1, 7, 6, 1, 1, 2, 7, 3, 2, 5, 3]
KAT_TRANS = [1, 0, 2, 3, 5, 7, 6, 4, 8, 10, 10, 9, 11, 11, 15, 14, 4, 0, 1, 1, 6, 5, 2, 7, 8, 9, 11, 10, 10, 12, 13, 11]
KAT_HIGH_D = [1, 0, 2, 3, 4, 5, 6, 6, 1, 0, 3, 2, 4, 5, 6, 7, 0, 1, 3, 2, 5, 4, 7, 6, 0, 0, 1, 2, 4, 3, 5, 4]
KAT_HIGH_CI = [[0, 1, 5, 7, 8, 10, 11] + [-1] * 9, [0, 4, 5, 6, 8, 9, 10, 12] + [-1] * 8,
               [2, 3, 4, 6, 9, 10, 14, 15] + [-1] * 8, [1, 2, 7, 10, 11, 13] + [-1] * 10]


def test_worked_example(orc):
    """N=128 (Q=4), Ns=64, window 8 keep 2, W=8: outputs of the reference's
    src/preprocessing.cu for this input."""
    assert orc.preprocess_low(KAT_DT, 64).tolist() == KAT_LOW
    DT2, pn, pm = orc.trans_index(KAT_DT, 2, 8)
    assert (pn, pm) == (4, 16) and DT2.reshape(-1).tolist() == KAT_TRANS
    D, ci = orc.preprocess_high(DT2, pm, pn, 64)
    assert D.tolist() == KAT_HIGH_D
    assert ci[:64].reshape(4, 16).tolist() == KAT_HIGH_CI
    assert (ci[64:] == -7).all(), "the extra window must stay untouched"


def _pre_cases():
    for n_keep in (32, 16, 12, 8, 4):
        for Ns in (32, 64, 128):
            for K, N in ((256, 256), (128, 384)):
                yield n_keep, Ns, K, N


@pytest.mark.parametrize("n_keep,Ns,K,N", list(_pre_cases()))
def test_preprocess_against_reference_fixtures(orc, golden, pkg_host, n_keep, Ns, K, N):
    g = golden["pre"]
    tag = f"n{n_keep}_Ns{Ns}_K{K}_N{N}"
    DT = g[tag + "_DT"]
    seed = 11 if (K, N) == (256, 256) else 12
    assert np.array_equal(DT, pkg_host.formats.random_indices(seed, K, N // 32, n_keep)), "generator drifted"
    if n_keep >= 12:
        assert np.array_equal(orc.preprocess_low(DT, Ns), g[tag + "_D"])
        assert np.array_equal(pkg_host.formats.retile(DT, Ns), g[tag + "_D"])
    else:
        DT2, pn, pm = orc.trans_index(DT, n_keep, 32)
        assert (pn, pm) == (2 * n_keep, 64)
        assert np.array_equal(DT2, g[tag + "_DT2"])
        D, ci = orc.preprocess_high(DT2, pm, pn, Ns)
        assert np.array_equal(D, g[tag + "_D"])
        assert np.array_equal(ci, g[tag + "_ci"])


@pytest.mark.parametrize("tag", ["c1", "r12", "r8", "r4", "r32"])
def test_multiply_against_reference_fixtures(orc, golden, pkg_host, tag):
    g = golden["gemm"]
    M, N, K, n_keep, seed = (int(x) for x in g[tag + "_shape"])
    p = pkg_host.formats.make_random(M, N, K, n_keep, seed=seed)
    sums = [p.A_km.astype(np.float64).sum(), p.BT.astype(np.float64).sum(), float(p.DT.astype(np.int64).sum())]
    assert np.allclose(sums, g[tag + "_sumA"], rtol=0, atol=1e-9), "generator drifted"
    C = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    assert np.array_equal(C, g[tag + "_C"]), "float restatement must be bit-identical to the reference's host multiply"
    # the double-precision anchor and the dense product agree with it
    C64 = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    assert np.linalg.norm(C - C64) / np.linalg.norm(C64) < 1e-6
    dense = p.A_km.T.astype(np.float64) @ p.dense_B().astype(np.float64)
    assert np.linalg.norm(dense - C64) / np.linalg.norm(C64) < 1e-12


@pytest.mark.parametrize("n_keep,Ns", [(16, 128), (12, 64), (32, 32), (8, 128), (4, 64), (8, 32)])
def test_packed_multiply_matches_unpacked(orc, pkg_host, n_keep, Ns):
    """The product read from the GPU-side operands (row-major B, packed D,
    column_info) equals the product read from the CPU-side ones, bit for bit."""
    p = pkg_host.formats.make_random(48, 256, 256, n_keep, seed=21)
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    if n_keep >= 12:
        D, ci, ws = orc.preprocess_low(p.DT, Ns), None, n_keep
    else:
        DT2, pn, pm = orc.trans_index(p.DT, n_keep, 32)
        D, ci = orc.preprocess_high(DT2, pm, pn, Ns)
        ws = pn
    got = orc.nm_gemm_packed(p.A_km, p.BT, D, ci, ws, Ns)
    assert np.array_equal(got, want)


@pytest.mark.skipif(not oracle.have_reference(), reason="compiled reference not present")
def test_restatement_equals_compiled_reference_on_fresh_inputs(orc, pkg_host):
    ref = oracle.reference()
    for seed, (M, N, K, n_keep) in enumerate([(32, 128, 128, 16), (16, 256, 192, 12), (64, 128, 256, 4), (8, 384, 128, 8)]):
        p = pkg_host.formats.make_random(M, N, K, n_keep, seed=100 + seed)
        assert np.array_equal(orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col), ref.nm_gemm_f32(p.A_km, p.B_col, p.D_col))
        for Ns in (32, 64, 128):
            if n_keep >= 12:
                assert np.array_equal(orc.preprocess_low(p.DT, Ns), ref.preprocess_low(p.DT, Ns))
            else:
                a, b = orc.trans_index(p.DT, n_keep, 32), ref.trans_index(p.DT, n_keep, 32)
                assert np.array_equal(a[0], b[0]) and a[1:] == b[1:]
                x, y = orc.preprocess_high(a[0], a[2], a[1], Ns), ref.preprocess_high(b[0], b[2], b[1], Ns)
                assert np.array_equal(x[0], y[0]) and np.array_equal(x[1], y[1])


def test_generator_formats(pkg_host):
    fm = pkg_host.formats
    p = fm.make_random(16, 128, 128, 8, seed=3, vec_len=64)
    assert p.DT.shape == (32, 4) and p.BT.shape == (32, 128) and p.A_km.shape == (128, 16)
    assert np.array_equal(p.DT[:, 0], p.DT[:, 1]) and np.array_equal(p.DT[:, 2], p.DT[:, 3])   # V=64 pairs share
    win = p.DT.reshape(4, 8, 4)
    assert (np.diff(win, axis=1) > 0).all() and win.min() >= 0 and win.max() < 32             # sorted, distinct, local
    assert abs(float(p.A_km.mean())) < 0.1 and p.A_km.min() >= -1 and p.A_km.max() < 1
    # magnitude pruning keeps the rows of largest per-vector L2 norm
    Bd = fm.normal(7, 2, 64 * 64, std=0.02).reshape(64, 64)
    BT, DT = fm.prune_magnitude(Bd, 8)
    for w0 in range(2):
        for v in range(2):
            norms = (Bd[w0 * 32:(w0 + 1) * 32, v * 32:(v + 1) * 32].astype(np.float64) ** 2).sum(axis=1)
            kept = DT[w0 * 8:(w0 + 1) * 8, v]
            assert sorted(np.argsort(-norms, kind="stable")[:8].tolist()) == kept.tolist()
            assert np.array_equal(BT[w0 * 8:(w0 + 1) * 8, v * 32:(v + 1) * 32], Bd[w0 * 32 + kept, v * 32:(v + 1) * 32])
