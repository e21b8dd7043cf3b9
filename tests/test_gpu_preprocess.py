"""Bit-exact parity of the GPU index-packing kernels with the CPU checker and with
the fixtures the reference's own preprocessing produced.  All calls go through the
C-ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n_keep", [32, 16, 12])
@pytest.mark.parametrize("Ns", [32, 64, 128])
@pytest.mark.parametrize("K,N", [(256, 256), (128, 384), (4096, 1152)])
def test_low_packing_bit_exact(pkg, orc, golden, n_keep, Ns, K, N):
    seed = {(256, 256): 11, (128, 384): 12}.get((K, N), 13)
    DT = pkg.formats.random_indices(seed, K, N // 32, n_keep)
    want = orc.preprocess_low(DT, Ns)
    tag = f"n{n_keep}_Ns{Ns}_K{K}_N{N}_D"
    if tag in golden["pre"]:
        assert np.array_equal(want, golden["pre"][tag])
    got = pkg.preprocess_low_device(_dev(DT), Ns).cpu().numpy()
    assert np.array_equal(got, want)
    # host-pointer form with the reference's in-place semantics
    host = DT.copy().reshape(-1)
    pkg.PreProcessing_low_sparsity(host, DT.shape[0], DT.shape[1], Ns)
    assert np.array_equal(host, want)


@pytest.mark.parametrize("n_keep", [8, 4])
@pytest.mark.parametrize("Ns", [32, 64, 128])
@pytest.mark.parametrize("K,N", [(256, 256), (128, 384), (4096, 1152), (64, 128 * 40)])
def test_high_packing_bit_exact(pkg, orc, golden, n_keep, Ns, K, N):
    seed = {(256, 256): 11, (128, 384): 12}.get((K, N), 14)
    DT = pkg.formats.random_indices(seed, K, N // 32, n_keep)
    W, Q = DT.shape
    DT2, pn, pm = orc.trans_index(DT, n_keep, 32)
    wantD, wantci = orc.preprocess_high(DT2, pm, pn, Ns)
    tag = f"n{n_keep}_Ns{Ns}_K{K}_N{N}"
    if tag + "_D" in golden["pre"]:
        assert np.array_equal(wantD, golden["pre"][tag + "_D"]) and np.array_equal(wantci, golden["pre"][tag + "_ci"])
    n_lists = wantci.size - pm

    # 1. separate transIndex kernel, then the packing kernel
    d = _dev(DT)
    pkg.trans_index_device(d, n_keep, 32)
    assert np.array_equal(d.cpu().numpy(), DT2)
    D, ci = pkg.preprocess_high_device(d, pm, pn, Ns)
    assert np.array_equal(D.cpu().numpy(), wantD)
    ci = ci.cpu().numpy()
    assert np.array_equal(ci[:n_lists], wantci[:n_lists])
    assert (ci[n_lists:] == -1).all(), "the device form defines the extra window as -1"

    # 2. transIndex folded into the packing kernel
    D2, ci2 = pkg.preprocess_high_device(_dev(DT), 32, n_keep, Ns, fuse_trans_index=True)
    assert np.array_equal(D2.cpu().numpy(), wantD) and np.array_equal(ci2.cpu().numpy()[:n_lists], wantci[:n_lists])

    # 3. host-pointer forms, in place, extra window untouched like the reference
    host = DT.copy().reshape(-1)
    pn_h, pm_h = pkg.transIndex(host, W, N, Q, n_keep, 32)
    assert (pn_h, pm_h) == (pn, pm) and np.array_equal(host, DT2.reshape(-1))
    ci_h = np.full(wantci.size, -7, dtype=np.int32)
    pkg.PreProcessing_high_sparsity(ci_h, pm_h, pn_h, host, W, Q, N, Ns)
    assert np.array_equal(host, wantD) and np.array_equal(ci_h, wantci)


def test_deep_k_packing_bit_exact_full_size(pkg, orc):
    """The deep-K configuration's index buffer (131072 x 1024, 4:32) at full size."""
    K, N, n_keep, Ns = 131072, 1024, 4, 128
    DT = pkg.formats.random_indices(5, K, N // 32, n_keep)
    DT2, pn, pm = orc.trans_index(DT, n_keep, 32)
    wantD, wantci = orc.preprocess_high(DT2, pm, pn, Ns)
    D, ci = pkg.preprocess_high_device(_dev(DT), 32, n_keep, Ns, fuse_trans_index=True)
    assert np.array_equal(D.cpu().numpy(), wantD)
    assert np.array_equal(ci.cpu().numpy()[:wantci.size - pm], wantci[:-pm])
    # ranks point back at the original columns: column_info[rank] == merged local index
    nwin, Qs = DT2.shape[0] // pn, Ns // 32
    cim = wantci[:-pm].reshape(N // Ns, nwin, pm)
    Dm = wantD.reshape(N // Ns, DT2.shape[0], Qs)
    blk, w, q = 3, 1234, 2
    assert cim[blk, w // pn, Dm[blk, w, q]] == DT2[w, blk * Qs + q]


@pytest.mark.parametrize("n_keep", [4, 8, 12, 16, 32])
@pytest.mark.parametrize("vec_len", [32, 64])
def test_prune_device_matches_the_host_generator(pkg, n_keep, vec_len):
    """Magnitude pruning on the GPU: kept rows and values equal, bit for bit, to the host
    generator's (formats.prune_magnitude), including ties (equal rows keep the lower one)."""
    rng = np.random.default_rng(300 + n_keep)
    K, N = 256, 384
    Bd = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    Bd[5] = Bd[3]                       # ties inside a window
    Bd[40:44, :64] = Bd[36:40, :64]
    Bd[64:96, 128:192] = 0.0            # a window of one vector that is all ties
    BT, DT = pkg.prune_device(torch.from_numpy(Bd).cuda(), n_keep, vec_len)
    want_BT, want_DT = pkg.formats.prune_magnitude(Bd, n_keep, vec_len)
    assert np.array_equal(DT.cpu().numpy(), want_DT)
    assert np.array_equal(BT.cpu().numpy(), want_BT)


@pytest.mark.parametrize("vec_len", [32, 64])
def test_prune_device_against_an_independent_statement_of_the_rule(pkg, vec_len):
    """The LLM-linear weight (4096 x 11008, N(0, 0.02^2)) pruned on the GPU, checked against the
    rule stated from scratch rather than against the package's own generator: per (32-row
    window, vector) the kept rows are the 8 with the largest FP64 sum of squares, ascending; the
    values are the weight's own at those rows."""
    K, N, n_keep = 4096, 11008, 8
    Bd = pkg.formats.normal(91, 2, K * N, std=0.02).reshape(K, N)
    BT, DT = pkg.prune_device(torch.from_numpy(Bd).cuda(), n_keep, vec_len)
    BT, DT = BT.cpu().numpy(), DT.cpu().numpy()
    nwin, nvec = K // 32, N // vec_len
    norms = np.square(Bd.astype(np.float64)).reshape(nwin, 32, nvec, vec_len).sum(axis=3)      # (window, row, vector)
    kept = np.sort(np.argsort(-norms, axis=1, kind="stable")[:, :n_keep, :], axis=1)             # (window, n_keep, vector)
    # no near-ties at the cut in this weight: the 8th and 9th largest norms differ clearly
    ranked = -np.sort(-norms, axis=1)
    assert float(((ranked[:, n_keep - 1] - ranked[:, n_keep]) / ranked[:, n_keep - 1]).min()) > 1e-9
    want_DT = np.repeat(kept.reshape(nwin * n_keep, nvec), vec_len // 32, axis=1)
    assert np.array_equal(DT, want_DT)
    rows = (kept + (np.arange(nwin) * 32)[:, None, None]).reshape(nwin * n_keep, nvec)
    assert np.array_equal(BT, np.take_along_axis(Bd, np.repeat(rows, vec_len, axis=1), axis=0))


def test_from_dense_runs_prune_pack_and_multiply_on_the_device(pkg, orc):
    p = pkg.formats.make_llm_linear(64, N=1408, K=1024, n_keep=8, seed=77)
    Bd = pkg.formats.normal(77, 2, 1024 * 1408, std=0.02).reshape(1024, 1408)
    op = pkg.NMSpMM.from_dense(torch.from_numpy(Bd).cuda(), 8)
    C = op.matmul(torch.from_numpy(p.A_km).cuda()).cpu().numpy()
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    assert np.linalg.norm(C - want) / np.linalg.norm(want) <= 1e-5


def test_prune_device_rejects_bad_shapes(pkg):
    x = torch.zeros((48, 64), device="cuda")
    with pytest.raises(pkg.NMSpMMError):
        pkg.prune_device(x, 8)                          # K not a multiple of 32
    with pytest.raises(pkg.NMSpMMError):
        pkg.prune_device(torch.zeros((64, 96), device="cuda"), 8, 64)    # N not a multiple of the vector width
