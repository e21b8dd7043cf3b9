"""World-size-2 run of the column-sharded path on CPU ranks (gloo): each rank takes
its slab through the package's partition code, the slab product comes from the CPU
checker (the GPU kernel's stand-in here), and the all-gather rebuilds the full C."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    import oracle
    from __graft_entry__ import load_package
    pkg = load_package(native=False)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = oracle.restatement()
        orc.set_num_threads(1)
        M, N, K, n_keep, Ns = 32, 384, 256, 8, 128          # 3 blocks over 2 ranks: uneven slabs (2 + 1)
        p = pkg.formats.make_random(M, N, K, n_keep, seed=9)
        bt, dt, (c0, c1) = pkg.sharding.shard_operands(p.BT, p.DT, rank, world, Ns)
        # pack the slab's indices exactly like a rank would on its GPU, multiply from the packed operands
        DT2, pn, pm = orc.trans_index(dt, n_keep, 32)
        D, ci = orc.preprocess_high(DT2, pm, pn, Ns)
        C_local = torch.from_numpy(orc.nm_gemm_packed(p.A_km, bt, D, ci, pn, Ns))
        assert C_local.shape == (M, c1 - c0)
        C = pkg.sharding.all_gather_columns(C_local, N, world, Ns)
        want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col)
        ok = np.array_equal(C.numpy(), want)
        # a rank's packed indices are the matching blocks of the full problem's packing
        DTf, pnf, pmf = orc.trans_index(p.DT, n_keep, 32)
        Df, cif = orc.preprocess_high(DTf, pmf, pnf, Ns)
        W = p.W
        blk0, blk1 = c0 // Ns, c1 // Ns
        ok = ok and np.array_equal(D, Df[blk0 * W * (Ns // 32):blk1 * W * (Ns // 32)])
        nwin = W // pnf
        ok = ok and np.array_equal(ci[:(blk1 - blk0) * nwin * pmf], cif[blk0 * nwin * pmf:blk1 * nwin * pmf])
        open(os.path.join(out_dir, f"rank{rank}.ok"), "w").write("1" if ok else "0")
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.ok").read() == "1"
