"""Measured choice of CTA tile and K split per shape, persisted for the planner.

The reference finds the best of its four tilings x SPLIT_K in {1, 2, 4, 8} for a shape by
sweeping them in a shell script (benchmark/kernel_performance/run_test/nmspmm/
run_nmspmm.sh:16-38) and reports the winner; nothing carries the result back into the
library.  Here the sweep writes a table the library reads at start-up
(``tuned_plans.txt`` beside the shared object, or the file named by NMSPMM_TUNED_PLANS):
``nmspmm_gemm`` with tile = 0 and split_k = 0 then runs the measured winner.

    python -m nm_spmm_b200.tuner                  # (from a script that imported the package)
    tuner.tune(pkg, [(M, N, K, n_keep, fmt, path, vec_len), ...], out_path)

Every candidate is timed with CUDA events over a CUDA-graph replay of several launches on
cycled copies of C (values of the operands do not matter for the timing).
"""
import os
from typing import Iterable, List, Sequence, Tuple

Shape = Tuple[int, int, int, int, int, int, int]       # M, N, K, n_keep, format, path, vec_len

FP32_TILES = (1, 2, 3, 4, 5, 6, 7)    # 128x128, 64x128, 32x128, 16x128, 128x256, 16x256, 32x256
TF32_TILES = (1, 5)
SPLITS = (0, 1, 2, 4, 8, 16)          # 0 = the library's automatic schedule on that tile


def default_table_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "tuned_plans.txt")


def candidates(pkg, M: int, path: int) -> List[Tuple[int, int]]:
    tiles = TF32_TILES if path == pkg.PATH_TF32 else tuple(t for t in FP32_TILES if _tile_rows(t) <= max(16, 2 * M))
    return [(t, s) for t in tiles for s in SPLITS]


def _tile_rows(tile: int) -> int:
    return {1: 128, 2: 64, 3: 32, 4: 16, 5: 128, 6: 16, 7: 32}[tile]


def time_candidate(pkg, torch, op, A, Cs, path: int, tile: int, split_k: int, launches: int = 8) -> float:
    """Milliseconds per launch, or inf when the combination is not supported."""
    try:
        for c in Cs[:2]:
            op.matmul(A, path=path, tile=tile, split_k=split_k, out=c)
        torch.cuda.synchronize()
    except pkg.NMSpMMError:
        return float("inf")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            op.matmul(A, path=path, tile=tile, split_k=split_k, out=Cs[i % len(Cs)])
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(3):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / launches)
    return best


def tune_shape(pkg, shape: Shape, verbose: bool = False):
    """Times every candidate of one shape.  Returns (best_tile, best_split, best_ms, heuristic_ms)."""
    import torch
    M, N, K, n_keep, fmt, path, vec_len = shape
    p = pkg.formats.make_random(4, N, K, n_keep, seed=1, vec_len=vec_len)      # B and indices; A is made on the device
    op = pkg.NMSpMM.from_problem(p, fmt=fmt)
    Mp = M + (-M) % 4
    A = torch.rand((K, Mp), device="cuda") * 2 - 1
    n_c = max(2, min(4, (256 << 20) // max(1, Mp * N * 4)))
    Cs = [torch.empty((Mp, N), device="cuda") for _ in range(n_c)]
    saved = pkg.tuned_plans_snapshot_and_clear()
    try:
        base = time_candidate(pkg, torch, op, A, Cs, path, 0, 0)
        best = (0, 0, base)
        for tile, split in candidates(pkg, M, path):
            ms = time_candidate(pkg, torch, op, A, Cs, path, tile, split)
            if verbose:
                print(f"  {shape} tile {tile} split {split}: {ms:.4f} ms", flush=True)
            if ms < best[2] * 0.98:                      # keep the heuristic unless something is clearly faster
                best = (tile, split, ms)
    finally:
        pkg.tuned_plans_restore(saved)
    assert pkg.device_status() == 0
    return best[0], best[1], best[2], base


def tune(pkg, shapes: Iterable[Shape], out_path: str = "", verbose: bool = False):
    """Tunes ``shapes``, merges the winners that beat the heuristics into the table file and
    registers them in the running library.  Returns the list of result rows."""
    out_path = out_path or default_table_path()
    rows = []
    for shape in shapes:
        tile, split, ms, base = tune_shape(pkg, shape, verbose)
        rows.append((shape, tile, split, ms, base))
        if verbose or True:
            print(f"{shape}: heuristic {base:.4f} ms, best tile {tile} split {split} {ms:.4f} ms ({base / ms:.3f}x)", flush=True)
    write_table(out_path, rows)
    pkg.load_tuned_plans(out_path)
    return rows


def read_table(path: str):
    entries = {}
    if os.path.exists(path):
        for line in open(path):
            f = line.split("#")[0].split()
            if len(f) == 9:
                entries[tuple(int(x) for x in f[:7])] = (int(f[7]), int(f[8]))
    return entries


def write_table(path: str, rows: Sequence) -> None:
    entries = read_table(path)
    for shape, tile, split, ms, base in rows:
        if tile == 0 and split == 0:
            entries.pop(tuple(shape), None)              # the heuristic is the winner: no entry
        else:
            entries[tuple(shape)] = (tile, split)
    with open(path, "w") as f:
        f.write("# M N K n_keep format path vec_len tile split_k   (written by nm-spmm_b200/tuner.py: measured on a B200;\n"
                "# an entry replaces the planner's heuristics for a description with tile = 0 and split_k = 0)\n")
        for key in sorted(entries):
            f.write(" ".join(str(x) for x in key + entries[key]) + "\n")
