"""``FusedRMSNormLinear`` on the GPU: the norm kernels against the reference's torch arithmetic
(``fused_rmsnorm_linear.py:32-62``), and the folded module against the unfused pair (a separate RMSNorm
in front of ``FusedLinear`` modules) over three training steps of a q / k / v + gate / up block."""

import pytest
import torch
import torch.nn as nn

from forge_b200 import FusedLinear, FusedOptimizerManager
from forge_b200 import rmsnorm_linear as RL
from tests.util import bf16_ulp_distance

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows,H", [(512, 4096), (37, 1032), (8, 8), (64, 14336), (130, 5120)])
def test_norm_kernels_match_torch_arithmetic(rows, H):
    gen = torch.Generator(device=DEV).manual_seed(rows * 7 + H)
    x = (torch.randn(rows, H, device=DEV, generator=gen) * 1.7).bfloat16()
    gamma = (1.0 + 0.2 * torch.randn(H, device=DEV, generator=gen)).bfloat16()
    gy = torch.randn(rows, H, device=DEV, generator=gen).bfloat16()
    y = RL.rmsnorm_forward(x, gamma, 1e-5)
    y_ref = RL._torch_rmsnorm_forward(x, gamma, 1e-5)
    ulps = bf16_ulp_distance(y_ref.float().cpu(), y)
    assert ulps.max().item() <= 1 and (ulps > 0).float().mean().item() < 0.01
    dx, dg = RL.rmsnorm_backward(x, gamma, gy, 1e-5)
    dx_ref, dg_ref = RL._torch_rmsnorm_backward(x, gamma, gy, 1e-5)
    # the two subtract nearly equal terms in different association: compare against the operands' scale
    scale = (gy.float() * gamma.float()).abs() + x.float().abs()
    assert ((dx.float() - dx_ref.float()).abs() <= 2 ** -7 * scale.clamp_min(1e-3)).all()
    assert torch.allclose(dg.float(), dg_ref.float(), rtol=2e-2, atol=2e-2 * rows ** 0.5)
    # twice the same bits: the column sums of grad_gamma are reduced in a fixed order
    dx2, dg2 = RL.rmsnorm_backward(x, gamma, gy, 1e-5)
    assert torch.equal(dg.view(torch.int16), dg2.view(torch.int16)) and torch.equal(dx.view(torch.int16), dx2.view(torch.int16))


class _KernelNorm(torch.autograd.Function):
    """The same norm kernels as a separate autograd node: the unfused pair's norm."""

    @staticmethod
    def forward(ctx, x, gamma, eps):
        ctx.save_for_backward(x, gamma)
        ctx.eps = eps
        return RL.rmsnorm_forward(x, gamma, eps)

    @staticmethod
    def backward(ctx, g):
        x, gamma = ctx.saved_tensors
        dx, dg = RL.rmsnorm_backward(x, gamma, g.contiguous(), ctx.eps)
        return dx, dg, None


class _Pair(nn.Module):
    """norm -> (q, k, v) summed, residual, norm -> silu(gate) * up; `folded` selects the implementation."""

    def __init__(self, folded, state_mode, hid=256, kv=128, ffn=512):
        super().__init__()
        self.folded = folded
        self.g1, self.g2 = nn.Parameter(torch.ones(hid)), nn.Parameter(torch.ones(hid))
        mk = lambda i, o: nn.Linear(i, o, bias=False)  # noqa: E731
        lin = {"q": mk(hid, hid), "k": mk(hid, kv), "v": mk(hid, kv), "gate": mk(hid, ffn), "up": mk(hid, ffn)}
        self.lin = nn.ModuleDict(lin)
        self.state_mode = state_mode

    def fuse(self):
        if self.folded:
            s1, s2 = RL.SharedNorm(self.g1, 1e-5, consumers=3), RL.SharedNorm(self.g2, 1e-5, consumers=2)
            for n in ("q", "k", "v"):
                self.lin[n] = RL.FusedRMSNormLinear(self.lin[n], self.g1, 1e-5, state_mode=self.state_mode, shared=s1, weight_decay=0.01)
            for n in ("gate", "up"):
                self.lin[n] = RL.FusedRMSNormLinear(self.lin[n], self.g2, 1e-5, state_mode=self.state_mode, shared=s2, weight_decay=0.01)
        else:
            for n in list(self.lin):
                self.lin[n] = FusedLinear.from_linear(self.lin[n], state_mode=self.state_mode, weight_decay=0.01)
        return self

    def forward(self, h):
        x1 = h if self.folded else _KernelNorm.apply(h, self.g1, 1e-5)
        kv = torch.cat([self.lin["k"](x1), self.lin["v"](x1)], dim=-1)
        h = h + self.lin["q"](x1) * torch.tanh(kv)
        x2 = h if self.folded else _KernelNorm.apply(h, self.g2, 1e-5)
        return torch.nn.functional.silu(self.lin["gate"](x2)) * self.lin["up"](x2), h


@pytest.mark.parametrize("grouped", [False, True])
@pytest.mark.parametrize("state_mode", ["bf16", "int8"])
def test_folded_norm_equals_unfused_pair(state_mode, grouped):
    torch.manual_seed(0)
    base = _Pair(False, state_mode)
    nets = []
    for folded in (False, True):
        net = _Pair(folded, state_mode)
        net.load_state_dict(base.state_dict())
        net = net.to(DEV).bfloat16().fuse().train()
        mgr = FusedOptimizerManager(net)
        if grouped:
            mgr.group_updates([[net.lin["q"], net.lin["k"], net.lin["v"]], [net.lin["gate"], net.lin["up"]]])
        nets.append((net, mgr))
    gen = torch.Generator(device=DEV).manual_seed(2)
    grads = [[], []]
    for step in range(3):
        h0 = torch.randn(4, 24, 256, device=DEV, generator=gen).bfloat16()
        for i, (net, mgr) in enumerate(nets):
            h = h0.clone().requires_grad_(True)
            mgr.pre_step(lr=1e-2)
            out, hh = net(h)
            (out.float().square().mean() + hh.float().square().mean()).backward()
            mgr.flush_updates()
            grads[i].append((h.grad.clone(), net.g1.grad.clone(), net.g2.grad.clone()))
            net.g1.grad = net.g2.grad = None
    torch.cuda.synchronize()
    (plain, _), (folded, _) = nets
    # weights: both sides feed the fused update the same recomputed activation and the same dY at step 1;
    # later steps see input gradients that were summed in a different order, so compare to a tolerance
    for n in plain.lin:
        a, b = plain.lin[n].weight.data.float(), folded.lin[n].weight.data.float()
        assert (a - b).abs().max().item() <= 2e-2 * a.abs().max().item(), n
        assert ((a - b).abs() > 0).float().mean().item() < 0.05, n
    (gh_p, g1_p, g2_p), (gh_f, g1_f, g2_f) = grads[0][0], grads[1][0]
    # first step (identical weights): the gradient through the norm, summed over the siblings once
    # (folded) or by autograd after three norm backward passes (pair)
    assert torch.allclose(gh_p.float(), gh_f.float(), rtol=3e-2, atol=3e-2 * gh_p.float().abs().max().item())
    assert torch.allclose(g1_p.float(), g1_f.float(), rtol=3e-2, atol=3e-2 * g1_p.float().abs().max().item())
    assert torch.allclose(g2_p.float(), g2_f.float(), rtol=3e-2, atol=3e-2 * g2_p.float().abs().max().item())


def test_norm_output_is_not_kept_for_backward():
    """What autograd holds between forward and backward: hidden states, gamma, weights -- no tensor of the
    normalised activation's content."""
    torch.manual_seed(1)
    lin = nn.Linear(256, 384, bias=False).to(DEV).bfloat16()
    gamma = nn.Parameter((1 + 0.1 * torch.randn(256, device=DEV)).bfloat16())
    fused = RL.FusedRMSNormLinear(lin, gamma, 1e-5).train()
    fused.update_optimizer_config(lr=1e-3)
    h = torch.randn(32, 256, device=DEV).bfloat16().requires_grad_(True)
    normed = RL.rmsnorm_forward(h.detach(), gamma.detach(), 1e-5)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: (saved.append(t), t)[1], lambda t: t):
        y = fused(h)
    assert len(saved) >= 3
    assert not any(t.shape == normed.shape and torch.equal(t, normed) for t in saved)
    w0 = fused.weight.data.clone()
    y.float().sum().backward()
    torch.cuda.synchronize()
    assert h.grad is not None and gamma.grad is not None and not torch.equal(fused.weight.data, w0)
    # eval mode: plain norm + linear
    fused.eval()
    with torch.no_grad():
        ye = fused(h)
    assert torch.allclose(ye.float(), torch.nn.functional.linear(RL.rmsnorm_forward(h.detach(), gamma.detach(), 1e-5), fused.weight).float())
