"""The sparse linear layer: prune + compress + pack on the device, then the multiply,
against a dense FP32 product with the layer's own pruned weight."""
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
