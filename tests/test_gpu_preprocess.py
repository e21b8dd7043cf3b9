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
