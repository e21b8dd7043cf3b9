"""Regenerates tests/golden/*.npz by running the REFERENCE's own host code.

Run where the reference checkout exists (it is compiled unchanged into
oracle/_ref/libnmspmm_ref.so by `make -C oracle ref`):

    python tests/golden/make_golden.py

Inputs come from the package's seeded generator; outputs are what the
reference's transIndex / PreProcessing_* / nmGEMM_on_cpu return for them.  The
fixtures pin the C restatement (oracle/nm_oracle.c) and, through it, the CUDA
library.  The fixtures travel; the reference does not.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from __graft_entry__ import load_package  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    pkg = load_package(native=False)
    fm = pkg.formats
    ref = oracle.reference()
    ref.set_num_threads(1)

    # --- index packing: every layout (Ns) x every N:M the reference supports ----
    pre = {}
    for n_keep in (32, 16, 12, 8, 4):
        for Ns in (32, 64, 128):
            for (K, N, seed) in ((256, 256, 11), (128, 384, 12)):
                DT = fm.random_indices(seed, K, N // 32, n_keep)
                tag = f"n{n_keep}_Ns{Ns}_K{K}_N{N}"
                pre[tag + "_DT"] = DT
                if n_keep >= 12:
                    pre[tag + "_D"] = ref.preprocess_low(DT, Ns)
                else:
                    DT2, pn, pm = ref.trans_index(DT, n_keep, 32)
                    assert (pn, pm) == (2 * n_keep, 64)
                    D, ci = ref.preprocess_high(DT2, pm, pn, Ns)
                    pre[tag + "_DT2"] = DT2
                    pre[tag + "_D"] = D
                    pre[tag + "_ci"] = ci
    np.savez_compressed(os.path.join(HERE, "preprocess.npz"), **pre)

    # --- the multiply: config 1 of the baseline (256x256x512, 16:32, seed 0) and
    #     one small case per remaining ratio -------------------------------------
    mm = {}
    cases = [("c1", 256, 256, 512, 16, 0), ("r12", 64, 128, 256, 12, 1), ("r8", 64, 128, 256, 8, 2),
             ("r4", 32, 64, 512, 4, 3), ("r32", 32, 64, 64, 32, 4)]
    for tag, M, N, K, n_keep, seed in cases:
        p = fm.make_random(M, N, K, n_keep, seed=seed)
        C = ref.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
        mm[tag + "_shape"] = np.array([M, N, K, n_keep, seed], dtype=np.int64)
        mm[tag + "_C"] = C
        # input checksums so that a drift of the generator is caught, not hidden
        mm[tag + "_sumA"] = np.array([p.A_km.astype(np.float64).sum(), p.BT.astype(np.float64).sum(),
                                      float(p.DT.astype(np.int64).sum())])
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **mm)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
