"""CPU-side checks of the boundary: the library loads and exports every symbol the
header declares, argument validation and plan selection behave, and the drop-in C++
names exist with the reference's mangling.  No kernel is launched."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    header = open(os.path.join(ROOT, "include", "nmspmm_b200.h")).read()
    declared = set(re.findall(r"\b(nmspmm_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(pkg.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/nmspmm_b200.h but not exported"
    assert declared == set(pkg.C_ABI_SYMBOLS)


def test_dropin_cpp_symbols_have_reference_mangling(pkg):
    """The reference's header declares C++ free functions (one takes int&), so the
    drop-in must export the same mangled names."""
    out = subprocess.run(["nm", "-D", "--defined-only", pkg.LIB_PATH], capture_output=True, text=True).stdout
    names = set(line.split()[-1] for line in out.splitlines() if line.strip())
    want = ["_Z26PreProcessing_low_sparsityPiiii", "_Z27PreProcessing_high_sparsityPiiiS_iiii", "_Z10transIndexPiiiiRiS0_"]
    for size in ("huge", "large", "medium", "small"):
        want.append(f"_Z{len('nmGEMM_' + size + '_matrices_low_sparsity')}nmGEMM_{size}_matrices_low_sparsityPfS_PiS_iiiifi")
        want.append(f"_Z{len('nmGEMM_' + size + '_matrices_high_sparsity')}nmGEMM_{size}_matrices_high_sparsityPfS_PiS0_S_iiiifi")
    for w in want:
        assert w in names, w


def test_status_strings(pkg):
    lib = pkg.load_library()
    assert lib.nmspmm_status_string(0) == b"ok"
    assert b"unsupported" in lib.nmspmm_status_string(pkg.UNSUPPORTED)
    assert lib.nmspmm_version() >= 0x000100


@pytest.mark.parametrize("M,N,K,n_keep,fmt,Ns,expect_tile", [
    (4096, 4096, 4096, 16, 0, 128, (128, 128)),
    (4096, 4096, 4096, 8, 1, 128, (128, 128)),
    (16, 11008, 4096, 8, 1, 128, (16, 128)),
    (64, 11008, 4096, 8, 1, 128, (64, 128)),
    (256, 11008, 4096, 8, 1, 128, (128, 128)),
    (192, 1024, 1024, 16, 0, 64, (64, 128)),
    (8192, 28672, 8192, 8, 1, 32, (128, 128)),
])
def test_plan_selection(pkg, M, N, K, n_keep, fmt, Ns, expect_tile):
    d = pkg.make_desc(M, N, K, n_keep, fmt, Ns)
    info = pkg.plan(d)
    assert (info.tile_m, info.tile_n) == expect_tile
    assert info.tiles_x == -(-N // info.tile_n) and info.tiles_y == -(-M // info.tile_m)
    ws = n_keep if fmt == 0 else 2 * n_keep
    n_win = K // 32 * n_keep // ws
    tiles = info.tiles_x * info.tiles_y
    assert info.stream_k == 1 and 1 <= info.n_virtual <= tiles * n_win
    assert info.grid == info.n_virtual and 0 <= info.n_dp <= tiles
    assert info.stages >= 2 and info.smem_bytes <= 227 * 1024
    need = pkg.workspace_bytes(d)
    assert need == 0 or need >= 2 * (info.n_virtual - info.n_dp) * info.tile_m * info.tile_n * 4


def _ranges(n_tiles, n_win, nv, n_dp):
    """Host restatement of the automatic unit schedule (virtual_range in gemm_args.h)."""
    out = [(v * n_win, (v + 1) * n_win) for v in range(n_dp)]
    base, total, n_sk = n_dp * n_win, (n_tiles - n_dp) * n_win, nv - n_dp
    out += [(base + i * total // n_sk, base + (i + 1) * total // n_sk) for i in range(n_sk)]
    return out


@pytest.mark.parametrize("n_tiles,n_win,nv,n_dp", [(1024, 64, 888 + 296, 888), (86, 64, 592, 0), (8, 2048, 296, 0),
                                                   (3, 5, 7, 0), (5, 1, 5, 0), (7, 3, 21, 0), (10, 4, 6 + 5, 6)])
def test_automatic_schedule_covers_every_unit_once(n_tiles, n_win, nv, n_dp):
    r = _ranges(n_tiles, n_win, nv, n_dp)
    assert r[0][0] == 0 and r[-1][1] == n_tiles * n_win and all(a[1] == b[0] for a, b in zip(r, r[1:]))
    total, n_sk = (n_tiles - n_dp) * n_win, nv - n_dp
    for t in range(n_tiles):
        holders = [v for v, (a, b) in enumerate(r) if a <= t * n_win + n_win - 1 and b > t * n_win]
        if t < n_dp:
            assert holders == [t]
        else:                                                   # tile_contributors() in gemm_args.h
            x0, x1 = (t - n_dp) * n_win, (t - n_dp) * n_win + n_win - 1
            v_first, v_last = n_dp + ((x0 + 1) * n_sk - 1) // total, n_dp + ((x1 + 1) * n_sk - 1) // total
            assert holders == list(range(v_first, v_last + 1))


def test_plan_balances_the_last_wave(pkg):
    info = pkg.plan(pkg.make_desc(2048, 3072, 4096, 8, 1, 128))               # 384 tiles: one full wave of 296 + 88
    tiles = info.tiles_x * info.tiles_y
    assert info.stream_k == 1 and 0 < info.n_dp < tiles and info.n_dp % (info.n_virtual - info.n_dp) == 0
    many = pkg.plan(pkg.make_desc(4096, 4096, 4096, 8, 1, 128))               # 1024 tiles: whole tiles only
    assert many.n_dp == many.n_virtual == 1024
    slab = pkg.plan(pkg.make_desc(8192, 3584, 8192, 8, 1, 128))                # 1792 tiles = 6 waves + 16 tiles: a nearly empty last wave is cut along k
    assert slab.n_dp == 6 * 296 and slab.n_virtual == 6 * 296 + 296
    exact = pkg.plan(pkg.make_desc(128 * 296 // 8, 1024, 4096, 8, 1, 128))      # 37 x 8 = 296 tiles: nothing to balance
    assert exact.n_dp == exact.tiles_x * exact.tiles_y == exact.n_virtual
    assert pkg.workspace_bytes(pkg.make_desc(128 * 296 // 8, 1024, 4096, 8, 1, 128)) == 0


def test_split_k_fills_the_machine_for_skinny_shapes(pkg):
    big = pkg.plan(pkg.make_desc(4096, 4096, 4096, 8, 1, 128))
    assert big.split_k == 1 and big.grid == big.n_virtual
    skinny = pkg.plan(pkg.make_desc(16, 11008, 4096, 8, 1, 128))
    assert skinny.split_k > 1 and skinny.n_virtual > 86
    deep = pkg.plan(pkg.make_desc(128, 1024, 131072, 4, 1, 128))
    assert deep.split_k >= 16
    forced = pkg.plan(pkg.make_desc(128, 1024, 131072, 4, 1, 128, split_k=7))
    assert forced.split_k == 7 and forced.stream_k == 0 and forced.n_virtual == 8 * 7
    clamped = pkg.plan(pkg.make_desc(128, 128, 64, 16, 0, 128, split_k=9))
    assert clamped.split_k == 2            # only two windows exist
    # the tensor-core path: slices when the tiles alone leave SMs idle, pieces always in scratch
    tdeep = pkg.make_desc(128, 1024, 131072, 4, 1, 128, path=pkg.PATH_TF32)
    info = pkg.plan(tdeep)
    assert info.tile_n == 256 and info.split_k == 148 // 4 and info.grid == 4 * info.split_k      # four wide tiles, one CTA per SM
    assert pkg.workspace_bytes(tdeep) == (64 << 10) + info.grid * 128 * 256 * 4      # counter block + one slot per slice
    # 512 tiles on 148 one-CTA SMs: three whole waves, the 68 tiles of the last one in two slices each
    tbig = pkg.plan(pkg.make_desc(4096, 4096, 4096, 8, 1, 128, path=pkg.PATH_TF32))
    assert tbig.tile_n == 256 and tbig.n_dp == 444 and tbig.split_k == 2 and tbig.grid == 444 + 2 * 68
    tlow = pkg.plan(pkg.make_desc(4096, 4096, 4096, 16, 0, 128, path=pkg.PATH_TF32))
    assert tlow.tile_n == 256 and tlow.n_dp == 444 and tlow.grid == 444 + 2 * 68   # the wide tile for every ratio once it fills the GPU
    tsmall = pkg.plan(pkg.make_desc(1024, 128, 4096, 16, 0, 128, path=pkg.PATH_TF32))
    assert tsmall.tile_n == 128                                                # B narrower than the wide tile
    texact = pkg.plan(pkg.make_desc(128 * 148, 256, 4096, 8, 1, 128, path=pkg.PATH_TF32))    # exactly one wave: nothing to slice
    assert texact.split_k == 1 and texact.grid == 148 and pkg.workspace_bytes(pkg.make_desc(128 * 148, 256, 4096, 8, 1, 128, path=pkg.PATH_TF32)) == 0
    one = pkg.plan(pkg.make_desc(128, 128, 64, 16, 0, 128, split_k=1))
    assert one.split_k == 1 and pkg.workspace_bytes(pkg.make_desc(128, 128, 64, 16, 0, 128, split_k=1)) == 0


@pytest.mark.parametrize("kw,status", [
    (dict(M=0), 1), (dict(N=100), 1), (dict(K=48), 1), (dict(M=6), 1), (dict(layout_ns=96), 1),
    (dict(n_keep=10), 2), (dict(n_keep=16, fmt=1), 2), (dict(n_keep=4, fmt=0), 2), (dict(path=2), 2), (dict(vec_len=48), 1), (dict(vec_len=64, N=160, layout_ns=32), 1),
    (dict(N=192, layout_ns=128), 1), (dict(K=96, n_keep=8, fmt=1), 1), (dict(split_k=-1), 1),
])
def test_bad_descriptions_are_rejected(pkg, kw, status):
    base = dict(M=128, N=256, K=256, n_keep=16, fmt=0, layout_ns=128, path=0, split_k=0, vec_len=0)
    base.update(kw)
    d = pkg.make_desc(base["M"], base["N"], base["K"], base["n_keep"], base["fmt"], base["layout_ns"],
                      base["path"], base["split_k"], 0, base["vec_len"])
    info = pkg.PlanInfo()
    rc = pkg.load_library().nmspmm_gemm_plan(ctypes.byref(d), ctypes.byref(info))
    assert rc == status, (kw, rc)


def test_sparsity_argument_mapping(pkg):
    assert [pkg.n_keep_of(s) for s in (0.0, 0.5, 0.625, 0.75, 0.875)] == [32, 16, 12, 8, 4]
    assert [pkg.format_of(n) for n in (32, 16, 12, 8, 4)] == [0, 0, 0, 1, 1]
    with pytest.raises(ValueError):
        pkg.n_keep_of(0.3)


def test_partition_columns(pkg_host):
    sh = pkg_host.sharding
    assert sh.partition_columns(28672, 8, 128) == [(i * 3584, (i + 1) * 3584) for i in range(8)]
    parts = sh.partition_columns(11008, 4, 128)          # 86 blocks over 4 ranks: 22, 22, 21, 21
    assert [c1 - c0 for c0, c1 in parts] == [2816, 2816, 2688, 2688]
    assert parts[0][0] == 0 and parts[-1][1] == 11008 and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
    with pytest.raises(ValueError):
        sh.partition_columns(256, 4, 128)
    with pytest.raises(ValueError):
        sh.partition_columns(200, 1, 128)


def test_tuned_plan_table_overrides_the_heuristics_and_only_them(pkg, tmp_path):
    d = pkg.make_desc(256, 2048, 2048, 4, 1, 128)
    base = pkg.plan(d)
    try:
        pkg.set_tuned_plan(d, 2, 4)                                    # tile 64 x 128, four K slices
        tuned = pkg.plan(d)
        assert (tuned.tile_m, tuned.tile_n, tuned.split_k) == (64, 128, 4)
        # a caller that names a tile or a split keeps its own choice
        own = pkg.plan(pkg.make_desc(256, 2048, 2048, 4, 1, 128, tile=1))
        assert (own.tile_m, own.tile_n) == (128, 128)
        assert pkg.plan(pkg.make_desc(256, 2048, 2048, 4, 1, 128, split_k=2)).split_k == 2
        # other shapes are untouched
        other = pkg.plan(pkg.make_desc(512, 2048, 2048, 4, 1, 128))
        assert (other.tile_m, other.tile_n) == (pkg.plan(pkg.make_desc(512, 2048, 2048, 4, 1, 128, tile=0)).tile_m, other.tile_n)
        # the file form
        table = tmp_path / "plans.txt"
        pkg.tuner.write_table(str(table), [((128, 1024, 4096, 8, 1, 0, 32), 3, 2, 1.0, 2.0), ((64, 256, 256, 16, 0, 0, 32), 0, 0, 1.0, 1.0)])
        assert pkg.tuner.read_table(str(table)) == {(128, 1024, 4096, 8, 1, 0, 32): (3, 2)}
        pkg.clear_tuned_plans()
        assert pkg.load_tuned_plans(str(table)) == 1
        got = pkg.plan(pkg.make_desc(128, 1024, 4096, 8, 1, 128))
        assert (got.tile_m, got.split_k) == (32, 2)
    finally:
        pkg.clear_tuned_plans()
    again = pkg.plan(d)
    assert (again.tile_m, again.tile_n, again.split_k) == (base.tile_m, base.tile_n, base.split_k)


def test_tf32_forms_are_selected_by_tile_id(pkg):
    """Tile ids 8 and 9 force the gathering and the expanding form of the TF32 path; the
    expanding one exists for the 32-k formats only and neither exists on the exact path."""
    low = pkg.make_desc(512, 1024, 1024, 16, pkg.FORMAT_LOW, 128, pkg.PATH_TF32)
    for tile, threads in ((pkg.TILE_128x256_GATHER, 256), (pkg.TILE_128x256_EXPAND, 320)):
        d = pkg.make_desc(512, 1024, 1024, 16, pkg.FORMAT_LOW, 128, pkg.PATH_TF32, 0, tile)
        info = pkg.plan(d)
        assert (info.tile_m, info.tile_n, info.threads) == (128, 256, threads)
    assert pkg.plan(low).tile in (pkg.TILE_128x256, pkg.TILE_128x256_EXPAND)
    assert pkg.plan(pkg.make_desc(512, 1024, 1024, 16, pkg.FORMAT_LOW, 128, pkg.PATH_TF32, 0, pkg.TILE_128x128)).tile == pkg.TILE_128x128
    lib = pkg.load_library()
    high = pkg.make_desc(512, 1024, 1024, 8, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32, 0, pkg.TILE_128x256_EXPAND)
    assert lib.nmspmm_gemm_workspace_bytes(ctypes.byref(high)) == 0
    with pytest.raises(pkg.NMSpMMError):
        pkg.plan(high)
    for tile in (pkg.TILE_128x256_GATHER, pkg.TILE_128x256_EXPAND):
        with pytest.raises(pkg.NMSpMMError):
            pkg.plan(pkg.make_desc(512, 1024, 1024, 16, pkg.FORMAT_LOW, 128, pkg.PATH_FP32, 0, tile))


def test_banded_tile_order_visits_every_tile_once(tmp_path):
    """gemm_args.h::tile_coords (shared by host and device): for plain and banded orders, full and
    ragged last bands, every (row, column) of tiles is produced by exactly one tile number, tiles
    of a band are consecutive, and band 0 is the row-by-row order."""
    src = tmp_path / "order.cpp"
    src.write_text(r'''
#include <cstdio>
#include <vector>
#include "gemm_args.h"
using namespace nmspmm;
int main() {
    const int shapes[][3] = {{5, 4, 0}, {5, 4, 2}, {112, 64, 16}, {7, 3, 3}, {8, 1, 4}, {9, 5, 127}, {33, 2, 8}, {224, 64, 32}};
    for (auto& sh : shapes) {
        const int tx_n = sh[0], ty_n = sh[1], band = sh[2];
        if (band >= tx_n && band != 0) continue;               // the planner never packs a band that wide
        const int packed = pack_tiles_x(tx_n, band);
        std::vector<int> seen(tx_n * ty_n, 0);
        int last_band = -1;
        for (int t = 0; t < tx_n * ty_n; ++t) {
            int ty, tx;
            tile_coords(t, packed, ty_n, ty, tx);
            if (ty < 0 || ty >= ty_n || tx < 0 || tx >= tx_n) { std::printf("range %d %d %d: tile %d -> %d %d\n", tx_n, ty_n, band, t, ty, tx); return 1; }
            if (seen[ty * tx_n + tx]++) { std::printf("twice %d %d %d: tile %d\n", tx_n, ty_n, band, t); return 1; }
            if (band == 0 && (ty != t / tx_n || tx != t % tx_n)) { std::printf("plain order broken at %d\n", t); return 1; }
            if (band > 0) {
                const int b = tx / band;
                if (b < last_band) { std::printf("band order %d %d %d: tile %d\n", tx_n, ty_n, band, t); return 1; }
                last_band = b;
            }
        }
    }
    std::printf("ok\n");
    return 0;
}
''')
    exe = tmp_path / "order"
    inc = os.path.join(ROOT, "nm-spmm_b200", "csrc")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-I", inc, str(src), "-o", str(exe)], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stdout + run.stderr


def test_few_rows_plans(pkg):
    """TF32 path, M <= 64: the library takes the 16 / 32 / 64-row tiles by itself, cuts K so that no
    slice has more windows than a CTA's index list holds, and refuses what the form cannot do."""
    for M, rows in ((1, 16), (16, 16), (17, 32), (32, 32), (33, 64), (64, 64)):
        info = pkg.plan(pkg.make_desc(M + (-M) % 4, 11008, 4096, 8, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32))
        assert (info.tile_m, info.tile_n, info.threads) == (rows, 128, 128)
        assert info.tiles_y == 1 and info.tiles_x == 86 and info.grid == 86 * info.split_k
        assert -(-64 // info.split_k) <= 24                       # windows per slice (K / 64 = 64 merged windows)
    assert pkg.plan(pkg.make_desc(68, 11008, 4096, 8, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32)).tile_m == 128
    deep = pkg.plan(pkg.make_desc(64, 1024, 131072, 4, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32))
    assert deep.tile_m == 64 and -(-2048 // deep.split_k) <= 24
    lib = pkg.load_library()
    too_few = pkg.make_desc(16, 1024, 131072, 4, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32, 2, pkg.TILE_16x128)
    assert lib.nmspmm_gemm_workspace_bytes(ctypes.byref(too_few)) == 0   # 1024 windows per slice: refused
    # left to the library, the same split goes to the 128-row tiles instead
    assert pkg.plan(pkg.make_desc(16, 1024, 131072, 4, pkg.FORMAT_HIGH, 128, pkg.PATH_TF32, 2)).tile_m == 128
