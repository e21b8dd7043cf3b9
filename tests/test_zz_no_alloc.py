"""The entry point that allocates nothing (nmspmm_gemm_static_scratch).

It exists for callers that are not allowed to call cudaMalloc at the point where
they multiply -- code running under another framework's allocator, inside a
latency-critical section, or in a process whose device memory was handed
out in full at start-up.  The scratch that split tiles need then comes from a fixed
array inside the library instead of from the caller.

The test drives it through the C-ABI on shapes whose plan splits tiles (so the
scratch is really used), twice in a row on the same array, and checks each result
against the ordinary entry point with caller scratch.  This file is named so that
pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5     # relative Frobenius error, the tolerance of the other multiply tests


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("M,N,K,n_keep,split_k", [(64, 1408, 1024, 8, 0), (128, 256, 2048, 16, 5), (16, 1024, 512, 4, 0)])
def test_static_scratch_matches_caller_scratch_twice(pkg, M, N, K, n_keep, split_k):
    p = pkg.formats.make_random(M, N, K, n_keep, seed=90 + n_keep)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    A2 = (torch.roll(A, 3, dims=1) * 0.25).contiguous()
    desc = op.desc(M, split_k=split_k)
    need = pkg.workspace_bytes(desc)
    assert 0 < need <= pkg.STATIC_SCRATCH_BYTES, "the case must use scratch and fit the built-in array"
    for a in (A, A2):                                   # two calls in a row share the array
        want = op.matmul(a, split_k=split_k)            # existing entry point, caller-owned scratch
        got = torch.full((M, N), float("nan"), device="cuda")
        pkg.gemm_static_scratch(desc, a, op.B, op.D, op.column_info, got)
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        assert _rel(got, want) <= FP32_TOL
        assert torch.equal(got, want), "same kernel, same schedule: the sums are identical"


def test_static_scratch_on_the_tensor_core_path_twice(pkg):
    """The same two-calls-in-a-row check with K slices on the TF32 path (its slots are plain
    row-major tiles added by the reduction kernel)."""
    M, N, K, n_keep, split_k = 128, 512, 2048, 8, 4
    p = pkg.formats.make_random(M, N, K, n_keep, seed=96)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    A2 = (torch.roll(A, 5, dims=1) * 0.5).contiguous()
    desc = op.desc(M, path=pkg.PATH_TF32, split_k=split_k)
    assert 0 < pkg.workspace_bytes(desc) <= pkg.STATIC_SCRATCH_BYTES
    for a in (A, A2):
        want = op.matmul(a, path=pkg.PATH_TF32, split_k=split_k)
        got = torch.full((M, N), float("nan"), device="cuda")
        pkg.gemm_static_scratch(desc, a, op.B, op.D, op.column_info, got)
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        assert torch.equal(got, want), "same kernel, same slices, same order of addition"


@pytest.mark.parametrize("M,path", [(64, 0), (256, 0), (512, 0), (64, 1)])
def test_static_scratch_takes_shapes_whose_automatic_plan_is_too_big(pkg, M, path):
    """An LLM-linear shape with the automatic schedule: nmspmm_gemm would want tens of MB of
    slots here.  The no-allocation entry point must still run it (with a schedule that fits
    its array), allocate nothing, and give the same product, twice in a row."""
    N, K, n_keep = 11008, 4096, 8
    p = pkg.formats.make_random(M, N, K, n_keep, seed=97)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    desc = op.desc(M, path=path)                        # split_k = 0: automatic
    want = op.matmul(A, path=path)
    tol = FP32_TOL if path == 0 else 2e-3               # another order of addition than `want`
    got = torch.full((M, N), float("nan"), device="cuda")
    pkg.gemm_static_scratch(desc, A, op.B, op.D, op.column_info, got)     # warm-up: resolves the array's address
    torch.cuda.synchronize()
    for _ in range(2):
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()      # (nothing of torch's allocates between the two readings)
        pkg.gemm_static_scratch(desc, A, op.B, op.D, op.column_info, got)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the call must not take device memory"
        assert pkg.device_status() == 0
        assert _rel(got, want) <= tol


def test_static_scratch_rejects_sizes_beyond_the_array(pkg):
    p = pkg.formats.make_random(128, 1024, 4096, 8, seed=95)
    op = pkg.NMSpMM.from_problem(p)
    A = torch.from_numpy(p.A_km).cuda()
    desc = op.desc(128, split_k=64)                    # 8 tiles x 64 slices x 64 KB = 32 MB of slots
    assert pkg.workspace_bytes(desc) > pkg.STATIC_SCRATCH_BYTES
    C = torch.zeros((128, 1024), device="cuda")
    with pytest.raises(pkg.NMSpMMError) as e:
        pkg.gemm_static_scratch(desc, A, op.B, op.D, op.column_info, C)
    assert e.value.status == pkg.WORKSPACE_TOO_SMALL
    assert float(C.abs().sum()) == 0.0                 # nothing was launched
