"""Column-sharded multiply on two GPUs with the optional all-gather of C: over NCCL after
the multiply, and fused into the multiply (stores into the peers' symmetric buffers).
Skipped on a single-GPU machine (the CPU ranks of test_sharding_gloo.py cover the
partition logic there).  NVLS is left off: the ranks are short-lived test processes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    import oracle
    from __graft_entry__ import load_package
    pkg = load_package(native=True)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ok = True
        for n_keep, path, tol in ((8, pkg.PATH_FP32, 1e-5), (16, pkg.PATH_FP32, 1e-5), (8, pkg.PATH_TF32, 2e-3)):
            M, N, K = 256, 1152, 512                           # 9 index blocks over 2 ranks: uneven slabs (5 + 4)
            p = pkg.formats.make_random(M, N, K, n_keep, seed=11)
            op = pkg.sharding.ShardedNMSpMM(pkg, p.BT, p.DT, K, n_keep, rank, world)
            A = torch.from_numpy(p.A_km).cuda()
            C = op.matmul(A, gather=True, path=path)
            torch.cuda.synchronize()
            orc = oracle.restatement()
            want = orc.nm_gemm_f32(p.A_km, p.B_col, p.D_col).astype(np.float64)
            err = np.linalg.norm(C.cpu().numpy() - want) / np.linalg.norm(want)
            ok = ok and C.shape == (M, N) and err <= tol
            # the gather fused into the multiply: peers' tiles arrive by their kernels' stores
            for split_k in (0, 3, 8):                      # whole tiles, in-kernel reduction, reduction kernel
                F = op.matmul(A, gather="fused", path=path, split_k=split_k)
                torch.cuda.synchronize()
                same = torch.equal(F, C) if split_k == 0 else float((F - C).norm() / C.norm()) <= 1e-6
                ok = ok and F.shape == (M, N) and same
            ok = ok and pkg.device_status() == 0
        open(os.path.join(out_dir, f"rank{rank}.ok"), "w").write("1" if ok else "0")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_column_sharding_with_all_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.ok").read() == "1"
