"""The tcgen05 kind::tf32 path against a double-precision host product.

Tolerance: TF32 keeps 10 mantissa bits and the tensor core takes the FP32 operands
as they are (the low 13 bits are dropped, not rounded), so every product carries a
relative error of up to 2^-9 with a bias of about -2^-10 that does not average out.
The stated bound is 2e-3 relative Frobenius error against the FP64 product of the
same FP32 inputs; measured values are around 7e-4.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3


def rel_err(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want))


def run(pkg, p, layout_ns=128, fmt=None, tile=0):
    op = pkg.NMSpMM.from_problem(p, layout_ns=layout_ns, fmt=fmt)
    C = op.matmul(torch.from_numpy(p.A_km).cuda(), path=pkg.PATH_TF32, tile=tile)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    return C.cpu().numpy()


@pytest.mark.parametrize("n_keep,fmt", [(16, 0), (12, 0), (32, 0), (8, 0), (8, 1), (4, 1)])
@pytest.mark.parametrize("layout", [32, 64, 128])
@pytest.mark.parametrize("tile", [1, 5])
def test_tf32_every_supported_ratio_layout_and_tile(pkg, orc, n_keep, fmt, layout, tile):
    """Tile 1 = 128 x 128 (two CTAs per SM), tile 5 = 128 x 256 (one)."""
    p = pkg.formats.make_random(256, 512, 512, n_keep, seed=200 + n_keep)
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    err = rel_err(run(pkg, p, layout_ns=layout, fmt=fmt, tile=tile), want)
    assert err <= TF32_TOL, err


@pytest.mark.parametrize("M,N", [(200, 640), (16, 128), (128, 96), (392, 1056)])
@pytest.mark.parametrize("n_keep,tile", [(8, 1), (8, 5), (12, 1), (16, 5)])
def test_tf32_ragged_rows_and_columns(pkg, orc, M, N, n_keep, tile):
    p = pkg.formats.make_random(M, N, 256, n_keep, seed=210)
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    assert rel_err(run(pkg, p, layout_ns=32, tile=tile), want) <= TF32_TOL


def test_tf32_single_window(pkg, orc):
    p = pkg.formats.make_random(128, 256, 64, 8, seed=211)
    assert rel_err(run(pkg, p), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


def test_tf32_is_deterministic_and_close_to_the_exact_path(pkg):
    p = pkg.formats.make_random(256, 512, 1024, 8, seed=212)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    a = op.matmul(A, path=pkg.PATH_TF32)
    b = op.matmul(A, path=pkg.PATH_TF32)
    exact = op.matmul(A)
    assert torch.equal(a, b)
    assert float((a - exact).norm() / exact.norm()) <= TF32_TOL


@pytest.mark.parametrize("n_keep,tile,split_k", [(8, 1, 2), (8, 5, 3), (16, 1, 5), (12, 1, 2), (4, 5, 7), (8, 1, 64)])
def test_tf32_k_slices(pkg, orc, n_keep, tile, split_k):
    """K slices on the tensor-core path: each slice's accumulators go to scratch and the
    reduction kernel adds them in k order (same result every run)."""
    p = pkg.formats.make_random(200, 384, 1024, n_keep, seed=214)
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    first = op.matmul(A, path=pkg.PATH_TF32, tile=tile, split_k=split_k)
    assert rel_err(first.cpu().numpy(), want) <= TF32_TOL
    assert torch.equal(op.matmul(A, path=pkg.PATH_TF32, tile=tile, split_k=split_k), first)
    assert pkg.device_status() == 0


def test_tf32_deep_k_automatic_slices(pkg, orc):
    p = pkg.formats.make_random(128, 256, 16384, 4, seed=215)
    info = pkg.plan(pkg.NMSpMM.from_problem(p).desc(p.M, path=pkg.PATH_TF32))
    assert info.split_k > 1
    assert rel_err(run(pkg, p), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


def test_tf32_12_of_32_with_an_odd_number_of_windows(pkg, orc):
    """12:32 gathers 16 columns per vector of which 4 stay zero, one 32-k window per step:
    the number of windows need not be even, and the last window's 16-row box of B runs
    past the end of B (those rows read as zeros)."""
    p = pkg.formats.make_random(128, 256, 96, 12, seed=213)
    assert rel_err(run(pkg, p), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


@pytest.mark.parametrize("n_keep", [16, 12, 8, 4])
def test_tf32_square_4096_full_size(pkg, orc, n_keep):
    p = pkg.formats.make_random(4096, 4096, 4096, n_keep, seed=80)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    C = op.matmul(A, path=pkg.PATH_TF32)
    rows = np.array([0, 1, 127, 128, 2047, 2048, 4095])
    want = orc.nm_gemm_f64(np.ascontiguousarray(p.A_km[:, rows]), p.B_col, p.D_col)
    assert rel_err(C[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= TF32_TOL
    exact = op.matmul(A)
    assert float((C - exact).norm() / exact.norm()) <= TF32_TOL
    assert pkg.device_status() == 0


@pytest.mark.parametrize("n_keep,fmt", [(16, 0), (12, 0), (8, 0), (8, 1), (4, 1)])
@pytest.mark.parametrize("M,N,K", [(256, 512, 512), (200, 640, 256), (128, 64, 64)])
def test_tf32_vectors_of_64_columns(pkg, orc, n_keep, fmt, M, N, K):
    """vec_len = 64: adjacent pairs of 32-wide index lists are equal and the kernel gathers
    once per 64 columns (N = 64 products).  Ragged last tile (640 = 2 x 256 + 128)."""
    p = pkg.formats.make_random(M, N, K, n_keep, seed=220 + n_keep, vec_len=64)
    op = pkg.NMSpMM.from_problem(p, fmt=fmt, layout_ns=128 if N % 128 == 0 else 64)
    assert op.vec_len == 64 and op.desc(M, path=pkg.PATH_TF32).vec_len == 64
    C = op.matmul(torch.from_numpy(p.A_km).cuda(), path=pkg.PATH_TF32)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert rel_err(C.cpu().numpy(), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


def test_tf32_llm_linear_full_size(pkg, orc):
    """LLM-linear configuration at full size on the tensor-core path, 16 / 64 / 256 tokens."""
    base = pkg.formats.make_llm_linear(256, seed=81)
    op = pkg.NMSpMM.from_problem(base)
    for tokens in (16, 64, 256):
        A_km = np.ascontiguousarray(base.A_km[:, :tokens])
        want = orc.nm_gemm_f64(A_km, base.B_col, base.D_col)
        got = op.matmul(torch.from_numpy(A_km).cuda(), path=pkg.PATH_TF32).cpu().numpy()
        assert rel_err(got, want) <= TF32_TOL, tokens
    assert pkg.device_status() == 0


def test_tf32_deep_k_full_size(pkg, orc):
    """Deep-K configuration at full size (A 128 x 131072, B 131072 x 1024, 4:32): 2048 merged
    windows per tile cut into K slices, added by the reduction kernel."""
    p = pkg.formats.make_random(128, 1024, 131072, 4, seed=82)
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    got = run(pkg, p)
    assert rel_err(got, want) <= TF32_TOL


def test_tf32_large_sharded_full_size(pkg, orc):
    """Large configuration at full size (8192 x 28672 x 8192, 8:32, V = 64) on the tensor-core
    path, gathering once per 64 columns: sampled rows of the whole product and of one rank's slab
    of a 4-way shard against the FP64 checker; the same product with 32-wide gathers agrees."""
    M, N, K = 8192, 28672, 8192
    p = pkg.formats.make_random(M, N, K, 8, seed=83, vec_len=64)
    A = torch.from_numpy(p.A_km).cuda()
    op = pkg.NMSpMM.from_problem(p)
    assert op.vec_len == 64
    full = op.matmul(A, path=pkg.PATH_TF32)
    rows = np.array([0, 127, 128, 4095, 4096, 8191])
    want = orc.nm_gemm_f64(np.ascontiguousarray(p.A_km[:, rows]), p.B_col, p.D_col)
    assert rel_err(full[torch.from_numpy(rows).cuda()].cpu().numpy(), want) <= TF32_TOL
    op.vec_len = 32                                            # the same operand read as 32-wide vectors
    narrow = op.matmul(A, path=pkg.PATH_TF32)
    assert float((narrow - full).norm() / full.norm()) <= 1e-6
    del narrow
    bt, dt, (c0, c1) = pkg.sharding.shard_operands(p.BT, p.DT, 2, 4, 128)
    slab = pkg.NMSpMM(bt, dt, K, 8, 128, vec_len=64).matmul(A, path=pkg.PATH_TF32)
    ref = full[:, c0:c1]
    assert float((slab - ref).norm() / ref.norm()) <= 1e-6
    assert pkg.device_status() == 0


# ---------------------------------------------------------------------------- the form that expands B

@pytest.mark.parametrize("n_keep", [16, 12, 8])
@pytest.mark.parametrize("M,N,K,split_k", [(128, 256, 64, 0), (256, 512, 512, 0), (200, 640, 256, 1), (132, 384, 2048, 0),
                                           (132, 384, 2048, 3), (1024, 1024, 1024, 0)])
def test_tf32_expanded_b_form(pkg, orc, n_keep, M, N, K, split_k):
    """Tile id 9: the A window multiplied whole by B expanded with zeros (32-k formats).  Ragged
    rows, a last tile with fewer vectors, K slices, and the automatic schedule."""
    p = pkg.formats.make_random(M, N, K, n_keep, seed=230 + n_keep)
    op = pkg.NMSpMM.from_problem(p, fmt=0)
    A = torch.from_numpy(p.A_km).cuda()
    assert pkg.plan(op.desc(M, path=pkg.PATH_TF32, tile=pkg.TILE_128x256_EXPAND, split_k=split_k)).tile == pkg.TILE_128x256_EXPAND
    C = op.matmul(A, path=pkg.PATH_TF32, tile=pkg.TILE_128x256_EXPAND, split_k=split_k)
    assert torch.equal(op.matmul(A, path=pkg.PATH_TF32, tile=pkg.TILE_128x256_EXPAND, split_k=split_k), C)
    assert pkg.device_status() == 0
    assert rel_err(C.cpu().numpy(), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


@pytest.mark.parametrize("n_keep", [16, 12, 8])
def test_tf32_forms_agree_on_an_index_list_with_repeated_rows(pkg, orc, n_keep):
    """The reference's sum takes a repeated index twice (include/utils.h:82-95).  The gather
    form does so by construction; the expanding form has to add the two values of B in
    the row they share."""
    M, N, K = 256, 512, 1024
    p = pkg.formats.make_random(M, N, K, n_keep, seed=236)
    DT = p.DT.copy().reshape(K // 32, n_keep, N // 32)
    DT[::2, 1, :] = DT[::2, 0, :]
    DT[1::4, 3, ::3] = DT[1::4, 2, ::3]
    p.DT[...] = DT.reshape(p.DT.shape)
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    op = pkg.NMSpMM.from_problem(p, fmt=0)
    A = torch.from_numpy(p.A_km).cuda()
    for tile in (pkg.TILE_128x256_GATHER, pkg.TILE_128x256_EXPAND):
        C = op.matmul(A, path=pkg.PATH_TF32, tile=tile)
        assert pkg.device_status() == 0
        assert rel_err(C.cpu().numpy(), want) <= TF32_TOL, tile


def test_tf32_expanded_b_form_at_4096_cubed(pkg, orc):
    p = pkg.formats.make_random(4096, 4096, 4096, 16, seed=81)
    op = pkg.NMSpMM.from_problem(p, fmt=0)
    A = torch.from_numpy(p.A_km).cuda()
    C = op.matmul(A, path=pkg.PATH_TF32, tile=pkg.TILE_128x256_EXPAND)
    exact = op.matmul(A)
    assert float((C - exact).norm() / exact.norm()) <= TF32_TOL
    assert pkg.device_status() == 0


# ---------------------------------------------------------------------------- few rows of A (M <= 64)

FEW_ROWS_TILE = {16: 4, 32: 3, 64: 2}        # nmspmm_tile_id of the 16 / 32 / 64 x 128 tiles


@pytest.mark.parametrize("n_keep,fmt", [(8, 1), (4, 1), (16, 0), (8, 0)])
@pytest.mark.parametrize("M,N,K", [(16, 256, 512), (4, 128, 128), (12, 384, 1024), (20, 160, 512), (32, 1024, 2048), (64, 640, 1024),
                                   (60, 1408, 4096)])
@pytest.mark.parametrize("split_k", [0, 3])
def test_tf32_few_rows_tiles(pkg, orc, n_keep, fmt, M, N, K, split_k):
    """The warp-level MMA tiles for M <= 64: every supported ratio and format, rows short of the
    tile, a last tile with fewer than four vectors, automatic and explicit K slices; the automatic
    choice for these shapes is this form."""
    ms = 16 if M <= 16 else (32 if M <= 32 else 64)
    p = pkg.formats.make_random(M, N, K, n_keep, seed=240 + M)
    op = pkg.NMSpMM.from_problem(p, fmt=fmt, layout_ns=128 if N % 128 == 0 else 32)
    A = torch.from_numpy(p.A_km).cuda()
    want = orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)
    d = op.desc(M, path=pkg.PATH_TF32, tile=FEW_ROWS_TILE[ms], split_k=split_k)
    if split_k and (K // (64 if fmt == 1 else 32)) / split_k > 24:
        with pytest.raises(pkg.NMSpMMError):              # a slice of more windows than a CTA's index list holds
            pkg.plan(d)
        return
    info = pkg.plan(d)
    assert (info.tile_m, info.tile_n) == (ms, 128)
    C = op.matmul(A, path=pkg.PATH_TF32, tile=FEW_ROWS_TILE[ms], split_k=split_k)
    assert torch.equal(op.matmul(A, path=pkg.PATH_TF32, tile=FEW_ROWS_TILE[ms], split_k=split_k), C)
    assert pkg.device_status() == 0
    assert rel_err(C.cpu().numpy(), want) <= TF32_TOL
    auto = pkg.plan(op.desc(M, path=pkg.PATH_TF32))
    assert (auto.tile_m, auto.tile_n) == (ms, 128)


def test_tf32_few_rows_refuses_more_rows_than_the_tile(pkg):
    with pytest.raises(pkg.NMSpMMError):
        pkg.plan(pkg.make_desc(128, 1024, 1024, 8, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32, 0, FEW_ROWS_TILE[64]))
    assert pkg.plan(pkg.make_desc(128, 1024, 1024, 8, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32)).tile_m == 128
    assert pkg.plan(pkg.make_desc(16, 1024, 1024, 12, pkg.FORMAT_LOW, 128, pkg.PATH_TF32)).tile_m == 128   # 12:32 has no such tile


def test_tf32_few_rows_deep_k(pkg, orc):
    p = pkg.formats.make_random(64, 256, 32768, 4, seed=247)
    op = pkg.NMSpMM.from_problem(p)
    C = op.matmul(torch.from_numpy(p.A_km).cuda(), path=pkg.PATH_TF32)
    assert pkg.plan(op.desc(64, path=pkg.PATH_TF32)).tile_m == 64
    assert pkg.device_status() == 0
    assert rel_err(C.cpu().numpy(), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL


@pytest.mark.parametrize("n_keep,fmt,tile", [(8, 1, 5), (16, 0, 5), (8, 0, 1), (16, 0, 9)])
@pytest.mark.parametrize("M,N,K,band,split_k", [(512, 1280, 512, 2, 0), (392, 1024, 1024, 3, 0), (512, 1536, 512, 2, 2), (1024, 4096, 256, 4, 0)])
def test_tf32_tiles_walked_in_bands_of_columns(pkg, orc, n_keep, fmt, tile, M, N, K, band, split_k):
    """The tile order the library takes by itself when B outgrows L2, forced here on small shapes:
    bands of `band` tile columns, the last band narrower, ragged rows, whole tiles and K slices
    (the reduction kernel has to map tiles the same way).  Same result as row by row, bit for bit."""
    p = pkg.formats.make_random(M, N, K, n_keep, seed=250 + band)
    op = pkg.NMSpMM.from_problem(p, fmt=fmt)
    A = torch.from_numpy(p.A_km).cuda()
    was = pkg.set_tile_band(0)
    try:
        plain = op.matmul(A, path=pkg.PATH_TF32, tile=tile, split_k=split_k)
        assert pkg.set_tile_band(band) == 0
        banded = op.matmul(A, path=pkg.PATH_TF32, tile=tile, split_k=split_k)
    finally:
        pkg.set_tile_band(was)
    assert pkg.device_status() == 0
    assert torch.equal(banded, plain)
    assert rel_err(banded.cpu().numpy(), orc.nm_gemm_f64(p.A_km, p.B_col, p.D_col)) <= TF32_TOL
