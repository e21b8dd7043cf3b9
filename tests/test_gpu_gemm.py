"""Parity of the CUDA multiply with the CPU checker, through the C-ABI.

Tolerance of the exact-FP32 path: relative Frobenius error <= 1e-5 against the
checker's float product (the reference's own host multiply), as the baseline
states.  Split-K results must be bit-identical from run to run."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5


def rel_err(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) / np.linalg.norm(want.astype(np.float64)))


def run(pkg, p, layout_ns=128, fmt=None, **kw):
    op = pkg.NMSpMM.from_problem(p, layout_ns=layout_ns, fmt=fmt)
    C = op.matmul(torch.from_numpy(p.A_km).cuda(), **kw)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    return C.cpu().numpy()


@pytest.mark.parametrize("tag", ["c1", "r12", "r8", "r4", "r32"])
def test_against_reference_fixtures(pkg, golden, tag):
    """Config 1 (256x256x512, 16:32, seed 0) and one case per ratio: outputs of the
    reference's host multiply, committed as fixtures."""
    g = golden["gemm"]
    M, N, K, n_keep, seed = (int(x) for x in g[tag + "_shape"])
    p = pkg.formats.make_random(M, N, K, n_keep, seed=seed)
    for Ns in (32, 64, 128) if N % 128 == 0 else (32, 64):
        assert rel_err(run(pkg, p, layout_ns=Ns), g[tag + "_C"]) <= FP32_TOL


@pytest.mark.parametrize("n_keep", [32, 16, 12, 8, 4])
@pytest.mark.parametrize("Ns", [32, 64, 128])
@pytest.mark.parametrize("M", [16, 64, 136, 256])
def test_every_ratio_layout_and_row_count(pkg, orc, n_keep, Ns, M):
    p = pkg.formats.make_random(M, 384, 512, n_keep, seed=30 + n_keep)
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    assert rel_err(run(pkg, p, layout_ns=Ns), want) <= FP32_TOL


@pytest.mark.parametrize("tile", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("n_keep,fmt", [(16, 0), (12, 0), (32, 0), (8, 0), (8, 1), (4, 1)])
@pytest.mark.parametrize("layout", [32, 64, 128])
def test_every_compiled_tile(pkg, orc, tile, n_keep, fmt, layout):
    """Every tile x ratio x index layout, on a shape with ragged rows (200 = 128 + 72)
    and a ragged last column tile (640 = 2*256 + 128)."""
    p = pkg.formats.make_random(200, 640, 256, n_keep, seed=40 + tile)
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    assert rel_err(run(pkg, p, layout_ns=layout, fmt=fmt, tile=tile), want) <= FP32_TOL


@pytest.mark.parametrize("split_k", [2, 3, 5, 8, 64])
@pytest.mark.parametrize("n_keep", [16, 8])
def test_split_k_is_exact_and_deterministic(pkg, orc, n_keep, split_k):
    p = pkg.formats.make_random(128, 256, 1024, n_keep, seed=50)
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    first = op.matmul(A, split_k=split_k).cpu().numpy()
    assert rel_err(first, want) <= FP32_TOL
    for _ in range(3):                       # same scratch reused: counters must have been left at zero
        assert np.array_equal(op.matmul(A, split_k=split_k).cpu().numpy(), first)
    assert pkg.device_status() == 0


def test_single_window_and_more_slices_than_windows(pkg, orc):
    p = pkg.formats.make_random(64, 128, 64, 8, seed=51)     # high path: exactly one 64-k window
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    assert rel_err(run(pkg, p), want) <= FP32_TOL
    assert rel_err(run(pkg, p, split_k=4), want) <= FP32_TOL  # clamped to one slice
    p = pkg.formats.make_random(32, 128, 32, 16, seed=52)    # low path: one 32-k window
    assert rel_err(run(pkg, p), orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)) <= FP32_TOL


def test_vector_width_64_as_duplicated_index_vectors(pkg, orc):
    p = pkg.formats.make_random(128, 512, 512, 8, seed=53, vec_len=64)
    assert rel_err(run(pkg, p), orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)) <= FP32_TOL


def test_llm_linear_magnitude_pruned(pkg, orc):
    for tokens in (16, 64):
        p = pkg.formats.make_llm_linear(tokens, N=1408, K=1024, n_keep=8, seed=54)
        assert rel_err(run(pkg, p), orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)) <= FP32_TOL


def test_reference_named_launchers(pkg, orc):
    """The eight launchers, called with the reference's argument lists."""
    for n_keep, sparsity in ((16, 0.5), (12, 0.625), (32, 0.0), (8, 0.75), (4, 0.875)):
        p = pkg.formats.make_random(128, 256, 256, n_keep, seed=60 + n_keep)
        want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
        A, B = torch.from_numpy(p.A_km).cuda(), torch.from_numpy(p.BT).cuda()
        for name, Ns in (("huge", 128), ("large", 64), ("medium", 64), ("small", 32)):
            for split in (1, 4):
                C = torch.full((p.M, p.N), 7.0, device="cuda")          # stale contents must be overwritten
                if n_keep >= 12:
                    D = pkg.preprocess_low_device(torch.from_numpy(p.DT).cuda(), Ns)
                    getattr(pkg, f"nmGEMM_{name}_matrices_low_sparsity")(A, B, D, C, p.M, p.N, p.K, p.W, sparsity, split)
                else:
                    D, ci = pkg.preprocess_high_device(torch.from_numpy(p.DT).cuda(), 32, n_keep, Ns, fuse_trans_index=True)
                    getattr(pkg, f"nmGEMM_{name}_matrices_high_sparsity")(A, B, D, ci, C, p.M, p.N, p.K, p.W, sparsity, split)
                assert rel_err(C.cpu().numpy(), want) <= FP32_TOL, (name, n_keep, split)
    with pytest.raises(pkg.NMSpMMError):
        pkg.nmGEMM_huge_matrices_low_sparsity(A, B, D, C, p.M, p.N, p.K, p.W, 0.75, 1)


def test_host_buffer_entry_point(pkg, orc):
    for n_keep in (16, 8):
        p = pkg.formats.make_random(128, 384, 512, n_keep, seed=70)
        C = np.empty((p.M, p.N), dtype=np.float32)
        d = pkg.make_desc(p.M, p.N, p.K, n_keep, pkg.format_of(n_keep), 128)
        pkg.gemm_host(d, p.A_km, p.BT, p.DT, C)
        assert rel_err(C, orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)) <= FP32_TOL


@pytest.mark.parametrize("M,n_keep", [(2308, 8), (3072, 16), (1024, 4)])
def test_host_buffer_entry_point_row_blocks(pkg, M, n_keep):
    """With M >= 2048 the host-buffer call moves A in and C out in row blocks (the last
    one ragged here) while other blocks are multiplied; the result agrees with the resident path's (not
    bit for bit: a row block may be scheduled with other k splits than the whole matrix), and
    a second call on the same thread reuses streams and events."""
    p = pkg.formats.make_random(M, 256, 1024, n_keep, seed=72)
    op = pkg.NMSpMM.from_problem(p)
    want = op.matmul(torch.from_numpy(p.A_km).cuda()).cpu().numpy()
    d = pkg.make_desc(p.M, p.N, p.K, n_keep, pkg.format_of(n_keep), 128)
    for _ in range(2):
        C = np.full((p.M, p.N), np.nan, dtype=np.float32)
        pkg.gemm_host(d, p.A_km, p.BT, p.DT, C)
        assert rel_err(C, want) <= 1e-6
    assert pkg.device_status() == 0


def test_workspace_too_small_and_bad_pointers(pkg):
    p = pkg.formats.make_random(128, 256, 1024, 16, seed=71)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    C = torch.empty((p.M, p.N), device="cuda")
    d = op.desc(p.M, split_k=4)
    with pytest.raises(pkg.NMSpMMError) as e:
        pkg.gemm(d, A, op.B, op.D, None, C, torch.zeros(1024, dtype=torch.uint8, device="cuda"))
    assert e.value.status == pkg.WORKSPACE_TOO_SMALL
    rc = pkg.load_library().nmspmm_gemm(ctypes.byref(op.desc(p.M)), None, None, None, None, None, None, 0, None)
    assert rc == pkg.INVALID_ARGUMENT


@pytest.mark.parametrize("n_keep", [16, 12, 8, 4])
def test_square_4096_full_size(pkg, orc, n_keep):
    """Full-size square case: sampled rows against the checker, plus linearity in A
    (a size-independent property) over the whole output."""
    M = N = K = 4096
    p = pkg.formats.make_random(M, N, K, n_keep, seed=80)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    C = op.matmul(A)
    rows = np.array([0, 1, 63, 64, 127, 128, 2047, 2048, 4031, 4095])
    sub = np.ascontiguousarray(p.A_km[:, rows])
    want = orc.nm_gemm_f32(sub, p.B_col, p.D_col)
    assert rel_err(C[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= FP32_TOL
    # one whole row block of tiles (128 rows x all columns: every column tile, every thread's fragment)
    blk = np.arange(1920, 2048)
    want_blk = orc.nm_gemm_f32(np.ascontiguousarray(p.A_km[:, blk]), p.B_col, p.D_col)
    assert rel_err(C[1920:2048].cpu().numpy(), want_blk) <= FP32_TOL
    A2 = torch.roll(A, 17, dims=1) * 0.5
    C2 = op.matmul(A2)
    C12 = op.matmul(A + A2)
    lin = (C12 - (C + C2)).norm() / C12.norm()
    assert float(lin) <= 2e-6
    assert pkg.device_status() == 0


def test_llm_linear_full_size(pkg, orc):
    """LLM-linear configuration at full size (K = 4096, N = 11008, 8:32 by per-vector L2
    magnitude): tokens 16, 64 and 256 against the checker, both paths of the split schedule."""
    base = pkg.formats.make_llm_linear(256, seed=81)
    op = pkg.NMSpMM.from_problem(base)
    for tokens in (16, 64, 256):
        A_km = np.ascontiguousarray(base.A_km[:, :tokens])
        want = orc.nm_gemm_f32(A_km, base.B_col, base.D_col)
        got = op.matmul(torch.from_numpy(A_km).cuda()).cpu().numpy()
        assert rel_err(got, want) <= FP32_TOL, tokens
        again = op.matmul(torch.from_numpy(A_km).cuda()).cpu().numpy()
        assert np.array_equal(got, again)
    assert pkg.device_status() == 0


def test_deep_k_full_size(pkg, orc):
    """Deep-K configuration at full size: A 128 x 131072, B 131072 x 1024, 4:32."""
    p = pkg.formats.make_random(128, 1024, 131072, 4, seed=82)
    want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    got = op.matmul(A).cpu().numpy()
    assert rel_err(got, want) <= FP32_TOL
    for split in (7, 32):                       # explicit K slices agree with the automatic schedule
        assert rel_err(op.matmul(A, split_k=split).cpu().numpy(), want) <= FP32_TOL
    assert pkg.device_status() == 0


def test_large_sharded_full_size(pkg, orc):
    """Large configuration at full size (8192 x 28672 x 8192, 8:32, V = 64): sampled rows
    against the checker, and the column slabs of a 4-way shard (computed one after the other
    on this GPU through the package's partition code) agree with the unsharded result (to rounding:
    a slab's nearly empty last wave is cut along k, which the unsharded launch's is not)."""
    M, N, K = 8192, 28672, 8192
    p = pkg.formats.make_random(M, N, K, 8, seed=83, vec_len=64)
    A = torch.from_numpy(p.A_km).cuda()
    full = pkg.NMSpMM.from_problem(p).matmul(A)
    rows = np.array([0, 127, 128, 4095, 4096, 8191])
    want = orc.nm_gemm_f32(np.ascontiguousarray(p.A_km[:, rows]), p.B_col, p.D_col)
    assert rel_err(full[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= FP32_TOL
    world = 4
    for rank in (0, 3):
        bt, dt, (c0, c1) = pkg.sharding.shard_operands(p.BT, p.DT, rank, world, 128)
        slab = pkg.NMSpMM(bt, dt, K, 8, 128).matmul(A)
        ref = full[:, c0:c1]
        assert float((slab - ref).norm() / ref.norm()) <= 1e-6, rank
    assert pkg.device_status() == 0


def test_one_scratch_buffer_serves_different_plans_in_turn(pkg):
    """The boundary between arrival counters and slots moves with the plan.  One operator
    (one cached scratch buffer) multiplies 512, 128 and 512 rows, then FP32, TF32, FP32:
    the slots of one plan land on the counters of the other, and every result must still
    be complete.  Checked against whole-tile launches (no scratch at all)."""
    p = pkg.formats.make_random(512, 4096, 4096, 8, seed=77)
    op = pkg.NMSpMM.from_problem(p)
    ref_op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    plans = [pkg.plan(op.desc(m)) for m in (512, 128)]
    assert any(pl.n_virtual > pl.n_dp for pl in plans), "at least one of the two plans must split tiles"

    def check(rows, path):
        a = A[:, :rows].contiguous()
        got = op.matmul(a, path=path, out=torch.full((rows, 4096), float("nan"), device="cuda"))
        want = ref_op.matmul(a, path=path, split_k=1)
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        err = float((got.double() - want.double()).norm() / want.double().norm())
        assert err <= (FP32_TOL if path == pkg.PATH_FP32 else 2e-3), (rows, path, err)
        assert not bool(torch.isnan(got).any())

    for rows in (512, 128, 512, 128, 512):
        check(rows, pkg.PATH_FP32)
    for path in (pkg.PATH_FP32, pkg.PATH_TF32, pkg.PATH_FP32, pkg.PATH_TF32, pkg.PATH_FP32):
        check(384, path)
