"""The bounded device-side waits, made to run out without faulting or hanging anything.

While nmspmm_test_short_fill is on, the launchers encode a tensor map (B's; A's on the TF32
form that reads B with plain loads) with a box one row short: every stage receives fewer bytes
than its mbarrier expects, the kernels' waits
give up after about a second of SM clock, the CTAs leave through their barriers without
storing, and the status word says so.  The kernels are the shipped ones, unchanged."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("path,tile,fmt,rows", [(0, 0, 1, 128), (1, 5, 1, 128), (1, 9, 0, 128), (1, 2, 1, 64)])
def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable(pkg, orc, path, tile, fmt, rows):
    """Exact path, TF32 gather form, TF32 form that expands B (tile id 9), TF32 few-rows form
    (tile id 2, at most 64 rows)."""
    p = pkg.formats.make_random(rows, 256, 512, 8, seed=300)
    op = pkg.NMSpMM.from_problem(p, fmt=fmt)
    A = torch.from_numpy(p.A_km).cuda()
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    assert pkg.device_status() == 0
    C = torch.full((rows, 256), 7.0, device="cuda")
    assert pkg.test_short_fill(True) == 0
    try:
        op.matmul(A, path=path, tile=tile, out=C, split_k=2)       # two slices per tile: scratch and counters are in play
        torch.cuda.synchronize()                        # returns: no hang, no fault
    finally:
        pkg.test_short_fill(False)
    assert bool((C == 7.0).all()), "a CTA whose wait gave up must not store"
    word = pkg.device_status(clear=False)
    assert word != 0
    assert pkg.load_library().nmspmm_device_status(None, 1) == pkg.DEVICE_TIMEOUT
    assert pkg.device_status() == 0                     # cleared
    # the next multiply on the same operator (same scratch, counters possibly left behind) is right
    got = op.matmul(A, path=path, tile=tile, split_k=2).cpu().numpy()
    err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    assert err <= (1e-5 if path == 0 else 2e-3)
    assert pkg.device_status() == 0
