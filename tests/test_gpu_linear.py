"""The sparse linear layer: prune + compress + pack on the device, then the multiply,
against a dense FP32 product with the layer's own pruned weight; the row-major-A entry
point on its own; the torch.library registration (fake kernel, autograd)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [1, 16, 61, 256])
@pytest.mark.parametrize("n_keep", [8, 16])
def test_sparse_linear_matches_dense_product_with_the_pruned_weight(pkg, tokens, n_keep):
    torch.manual_seed(tokens + n_keep)
    in_f, out_f = 1024, 1408
    w = torch.randn(out_f, in_f, device="cuda") * 0.02
    b = torch.randn(out_f, device="cuda")
    layer = pkg.linear.NMSparseLinear(pkg, w, n_keep, bias=b)
    x = torch.randn(2, tokens, in_f, device="cuda") if tokens > 1 else torch.randn(tokens, in_f, device="cuda")
    y = layer(x)
    wp = layer.dense_weight()
    kept = int((wp != 0).sum())                                          # n_keep of every 32 inputs (a kept weight may itself be 0.0)
    assert out_f * in_f * n_keep // 32 - 4 <= kept <= out_f * in_f * n_keep // 32
    assert torch.equal(wp[wp != 0], w[wp != 0])
    want = (x.double() @ wp.double().t() + b.double())
    assert y.shape == want.shape
    err = float((y.double() - want).norm() / want.norm())
    assert err <= 1e-5, err
    assert pkg.device_status() == 0


def test_sparse_linear_tf32_path(pkg):
    torch.manual_seed(5)
    w = torch.randn(1024, 512, device="cuda") * 0.02
    layer = pkg.linear.NMSparseLinear(pkg, w, 8, path=pkg.PATH_TF32)
    x = torch.randn(200, 512, device="cuda")
    want = x.double() @ layer.dense_weight().double().t()
    assert float((layer(x).double() - want).norm() / want.norm()) <= 2e-3


@pytest.mark.parametrize("M", [1, 3, 16, 130, 257])
@pytest.mark.parametrize("n_keep,path", [(16, 0), (8, 0), (4, 0), (8, 1), (12, 1)])
def test_row_major_activations_against_the_checker(pkg, orc, M, n_keep, path):
    """nmspmm_gemm_row_major: A[i*K + k], any M >= 1 (the col-major copy the kernels read is
    padded to 4 rows by the transposing kernel), checked against the CPU checker."""
    p = pkg.formats.make_random(M + (-M) % 4, 384, 512, n_keep, seed=400 + M)
    A_rows = np.ascontiguousarray(p.A_km.T[:M])                          # (M, K) row-major
    op = pkg.NMSpMM.from_problem(p)
    got = op.matmul_rows(torch.from_numpy(A_rows).cuda(), path=path)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and got.shape == (M, 384)
    sub = np.ascontiguousarray(p.A_km[:, :M])
    if path == 0:
        want, tol = orc.nm_gemm_f32(sub, p.B_col, p.D_col), 1e-5
    else:
        want, tol = orc.nm_gemm_f64(sub, p.B_col, p.D_col), 2e-3
    err = float(np.linalg.norm(got.cpu().numpy().astype(np.float64) - want) / np.linalg.norm(want))
    assert err <= tol, err


def test_custom_op_is_registered_with_fake_kernel_and_autograd(pkg):
    torch.manual_seed(7)
    w = torch.randn(256, 128, device="cuda") * 0.1
    layer = pkg.linear.NMSparseLinear(pkg, w, 16)
    op = torch.ops.nmspmm_b200.sparse_linear
    x = torch.randn(8, 128, device="cuda", requires_grad=True)
    layer.values.requires_grad_(True)
    args = (x, layer.values, layer.op.D, layer.op.column_info, layer.raw_indices, 16, layer.op.format, layer.op.layout_ns, 32, 0)
    torch.library.opcheck(op, args, test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))
    # gradients against a dense product with the pruned weight
    y = layer(x)
    y.square().sum().backward()
    gx, gv = x.grad.clone(), layer.values.grad.clone()
    wd = layer.dense_weight().detach().requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    (x2 @ wd.t()).square().sum().backward()
    assert float((gx - x2.grad).norm() / x2.grad.norm()) <= 1e-4
    rows = pkg.linear._dense_rows(layer.raw_indices, 16)
    assert float((gv - wd.grad.t().gather(0, rows)).norm() / gv.norm()) <= 1e-4
    # shape inference without running the kernel
    from torch._subclasses.fake_tensor import FakeTensorMode
    mode = FakeTensorMode()
    fake = [mode.from_tensor(a.detach()) if isinstance(a, torch.Tensor) else a for a in args]
    with mode:
        assert op(*fake).shape == (8, 256)


# ---------------------------------------------------------------------------- 16-bit storage

def _round_to(t, dtype):
    return t.to(dtype).to(torch.float32)


@pytest.mark.parametrize("dtype,out_tol", [(torch.bfloat16, 4e-3), (torch.float16, 5e-4)])
@pytest.mark.parametrize("M", [1, 16, 61, 256])
@pytest.mark.parametrize("n_keep,path", [(8, 0), (8, 1), (16, 1)])
def test_row_major_16_bit_activations_and_result(pkg, orc, dtype, out_tol, M, n_keep, path):
    """nmspmm_gemm_row_major_16 against the CPU checker on the widened operands.  With B's
    values representable in the 16-bit type too, every product is exact on both paths: what is
    left is the FP32 summation and the one rounding of the result (2^-9 for bfloat16, 2^-11
    for half), which the tolerance states."""
    p = pkg.formats.make_random(M + (-M) % 4, 384, 512, n_keep, seed=500 + M)
    p.BT[...] = _round_to(torch.from_numpy(p.BT), dtype).numpy()
    x32 = _round_to(torch.from_numpy(np.ascontiguousarray(p.A_km.T[:M])), dtype)          # (M, K) row-major, representable
    op = pkg.NMSpMM.from_problem(p)
    y = op.matmul_rows(x32.to(dtype).cuda(), path=path)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.dtype == dtype and y.shape == (M, 384)
    want = orc.nm_gemm_f64(np.ascontiguousarray(x32.numpy().T), p.B_col, p.D_col)
    got = y.to(torch.float32).cpu().numpy().astype(np.float64)
    assert float(np.linalg.norm(got - want) / np.linalg.norm(want)) <= out_tol
    # before the final rounding the two paths agree to FP32 summation error: the tensor-core path
    # loses nothing on operands of 16 bits
    exact = op.matmul_rows(x32.cuda(), path=pkg.PATH_FP32)
    tensor = op.matmul_rows(x32.cuda(), path=pkg.PATH_TF32)
    assert float((tensor - exact).norm() / exact.norm()) <= 1e-5


def test_widen_device_is_exact(pkg):
    for dtype in (torch.float16, torch.bfloat16):
        t = (torch.randn(1000, 52, device="cuda") * 3).to(dtype)
        assert torch.equal(pkg.widen_device(t), t.to(torch.float32))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_sparse_linear_with_16_bit_weight_and_activations(pkg, dtype):
    torch.manual_seed(11)
    in_f, out_f = 1024, 1408
    w = (torch.randn(out_f, in_f, device="cuda") * 0.02).to(dtype)
    b = torch.randn(out_f, device="cuda").to(dtype)
    layer = pkg.linear.NMSparseLinear(pkg, w, 8, bias=b, path=pkg.PATH_TF32)
    wp = layer.dense_weight()
    assert torch.equal(wp[wp != 0], w.to(torch.float32)[wp != 0])        # kept weights are the 16-bit values, widened
    x = torch.randn(3, 40, in_f, device="cuda").to(dtype)
    y = layer(x)
    assert y.dtype == dtype and y.shape == (3, 40, out_f)
    want = x.double() @ wp.double().t() + b.double()
    err = float((y.double() - want).norm() / want.norm())
    assert err <= (8e-3 if dtype == torch.bfloat16 else 1e-3), err      # two roundings: the product and the bias add
    assert pkg.device_status() == 0


def test_one_workspace_serves_row_major_calls_of_different_row_counts(pkg, orc):
    """The operator's cached workspace is reused across calls: the multiply's counter block has
    to stay where it is (and zero) whether the call before it had more rows, fewer, or a plan
    that needs no scratch at all."""
    p = pkg.formats.make_random(4096, 1024, 1024, 8, seed=520)
    op = pkg.NMSpMM.from_problem(p)
    x_all = torch.from_numpy(np.ascontiguousarray(p.A_km.T)).cuda()
    exact = op.matmul(torch.from_numpy(p.A_km).cuda())
    for M in (4096, 512, 16, 2048, 128, 4096, 64):
        for dt in (torch.float32, torch.bfloat16):
            x = x_all[:M].contiguous()
            y = op.matmul_rows(x.to(dt))
            ref = exact[:M] if dt == torch.float32 else op.matmul_rows(x.to(dt).to(torch.float32))
            tol = 1e-5 if dt == torch.float32 else 4e-3
            assert float((y.to(torch.float32) - ref).norm() / ref.norm()) <= tol, (M, dt)
    assert pkg.device_status() == 0
