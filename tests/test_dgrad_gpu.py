"""GPU parity of the dX GEMM (``forge_dgrad``): dX = dY W with bf16 operands, fp32 accumulation and
bf16 output, against an fp32 CPU matmul of the same bf16 values (the reference computes
``grad_output @ weight``, ``autograd.py:55``)."""

import pytest
import torch

from forge_b200 import kernel as K
from tests.util import assert_one_ulp

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = [(128, 128, 128), (512, 1024, 1024), (200, 392, 1032), (8, 8, 64), (64, 4096, 256), (520, 136, 264)]


@pytest.mark.parametrize("BT,V,H", SHAPES)
def test_dgrad_exact_sums(BT, V, H):
    """Multiples of 1/8: every partial sum is exact in fp32, so the bf16 result is unique."""
    g = torch.Generator().manual_seed(21)
    dy = (torch.randint(-8, 9, (BT, V), generator=g).float() / 8).bfloat16()
    w = (torch.randint(-8, 9, (V, H), generator=g).float() / 8).bfloat16()
    expect = (dy.float() @ w.float()).bfloat16()
    out = K.dgrad(dy.to(DEV), w.to(DEV))
    assert out.shape == (BT, H) and out.dtype == torch.bfloat16
    assert torch.equal(out.cpu().view(torch.int16), expect.view(torch.int16))


@pytest.mark.parametrize("BT,V,H", SHAPES)
def test_dgrad_gaussian(BT, V, H):
    g = torch.Generator().manual_seed(22)
    dy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
    w = (torch.randn(V, H, generator=g) * 0.02).bfloat16()
    expect = dy.double() @ w.double()
    scale = dy.double().abs() @ w.double().abs()
    out = K.dgrad(dy.to(DEV), w.to(DEV))
    assert_one_ulp(expect.float(), out, scale.float(), "dX", noise=4e-6)


def test_dgrad_strided_and_module_path():
    """Row-pitched operands, and the autograd path with the library GEMM switched on."""
    from forge_b200 import FusedLinear, autograd
    BT, V, H = 96, 256, 320
    g = torch.Generator().manual_seed(23)
    dyw = (torch.randn(BT, V + 64, generator=g) * 1e-2).bfloat16().to(DEV)
    ww = (torch.randn(V, H + 64, generator=g) * 0.02).bfloat16().to(DEV)
    dy, w = dyw[:, :V], ww[:, 32:32 + H]
    out = K.dgrad(dy, w)
    assert_one_ulp((dy.double().cpu() @ w.double().cpu()).float(), out,
                   (dy.double().abs().cpu() @ w.double().abs().cpu()).float(), "dX")
    layer = FusedLinear(H, V, optimizer_type="sgd").to(DEV).to(torch.bfloat16).train()
    layer.update_optimizer_config(lr=1e-2, weight_decay=0.0)
    x = torch.randn(4, 24, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w0 = layer.weight.detach().clone()
    old = autograd.use_forge_dgrad
    autograd.use_forge_dgrad = True
    try:
        y = layer(x)
        gy = torch.randn_like(y) * 1e-2
        y.backward(gy)
    finally:
        autograd.use_forge_dgrad = old
    expect = (gy.double().reshape(-1, V) @ w0.double()).reshape(4, 24, H)   # the PRE-update weight
    assert x.grad.shape == x.shape
    assert_one_ulp(expect.float().cpu(), x.grad, (gy.double().abs().reshape(-1, V) @ w0.double().abs()).reshape(4, 24, H).float().cpu(), "x.grad")
    assert not torch.equal(layer.weight.detach(), w0)
