"""Module-level behaviour on the GPU: multi-step trajectories against torch autograd +
``torch.optim.AdamW`` on the CPU (one 1024 x 1024 linear, fp32 state, ten steps), gradient accumulation, the non-fused
escape hatch, bias handling, checkpoint round trips, every optimizer / state mode under a manager."""

import copy

import numpy as np
import pytest
import torch

from forge_b200 import FusedLinear, FusedOptimizerManager
from oracle import torch_steps as T
from tests.util import assert_w_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_config0_ten_steps_vs_torch_adamw():
    """Linear(1024 -> 1024, no bias), BT=512, X ~ N(0,1) bf16, dY ~ N(0,1e-2) bf16, W ~ N(0,0.02)
    fp32 master, AdamW lr=1e-3 betas=(0.9,0.999) eps=1e-8 wd=0.01, fp32 m/v from zero, 10 steps with
    fresh seeded X/dY; reference = torch autograd + torch.optim.AdamW on the CPU."""
    V = H = 1024
    BT = 512
    w0 = torch.randn(V, H, generator=torch.Generator().manual_seed(0)) * 0.02
    ref = T.TorchAdamWLinear(w0, 1e-3, (0.9, 0.999), 1e-8, 0.01)
    layer = FusedLinear(H, V, optimizer_type="adamw")
    layer.weight.data = w0.clone()
    layer = layer.to(DEV).train()
    for s in range(10):
        g = torch.Generator().manual_seed(1000 + s)
        x = torch.randn(BT, H, generator=g).bfloat16()
        dy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
        ref.step(x, dy)
        layer.update_optimizer_config(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
        # the module computes Y with an fp32 master weight; feed dY directly through autograd
        y = layer(x.float().to(DEV))
        y.backward(dy.float().to(DEV))
    assert layer._state.step == 10 and layer._state.m.dtype == torch.float32
    wf = layer.weight.detach().cpu()
    wr = ref.weight.detach()
    # ten steps of summation-order noise and approximate quotients: still one bf16 ULP, and close in fp32
    from tests.util import assert_one_ulp
    assert_one_ulp(wr, wf, w0.abs() + 1e-2, "W after 10 steps", noise=1e-4)
    np.testing.assert_allclose(wf.numpy(), wr.numpy(), rtol=2e-4, atol=1e-5)
    assert (wf - w0).abs().max() > 1e-3


@pytest.mark.parametrize("mode", ["bf16", "int8", "fp8", "fp8_block"])
def test_bf16_training_tracks_fp32_reference(mode):
    """bf16 weights, each state mode, 6 steps: the loss trajectory follows an fp32 CPU AdamW run."""
    torch.manual_seed(0)
    H, V, BT = 256, 384, 96
    w0 = torch.randn(V, H) * 0.05
    target = torch.randn(V, H) * 0.05
    layer = FusedLinear(H, V, optimizer_type="adamw", state_mode=mode)
    layer.weight.data = w0.clone()
    layer = layer.to(DEV).to(torch.bfloat16).train()
    ref_w = torch.nn.Parameter(w0.clone())
    opt = torch.optim.AdamW([ref_w], lr=2e-3, weight_decay=0.0)
    losses, ref_losses = [], []
    for s in range(6):
        x = torch.randn(BT, H, generator=torch.Generator().manual_seed(s))
        y_t = x @ target.t()
        layer.update_optimizer_config(lr=2e-3, weight_decay=0.0)
        xd = x.to(DEV).bfloat16().requires_grad_(True)
        loss = ((layer(xd).float() - y_t.to(DEV)) ** 2).mean()
        loss.backward()
        losses.append(loss.item())
        opt.zero_grad()
        rl = ((x @ ref_w.t() - y_t) ** 2).mean()
        rl.backward()
        opt.step()
        ref_losses.append(rl.item())
        assert xd.grad is not None and layer.weight.grad is None
    assert losses[-1] < losses[0] * 0.9
    np.testing.assert_allclose(losses, ref_losses, rtol=0.08)


def test_gradient_accumulation_and_escape_hatch():
    torch.manual_seed(1)
    H, V = 128, 192
    base = torch.nn.Linear(H, V, bias=False).to(DEV)
    xs = [torch.randn(16, H, device=DEV) for _ in range(2)]

    fused = FusedLinear.from_linear(copy.deepcopy(base), optimizer_type="adamw").train()
    mgr = FusedOptimizerManager(torch.nn.Sequential(fused), gradient_accumulation_steps=2)
    for x in xs:
        mgr.pre_step(lr=1e-3)
        fused(x).sum().backward()
    assert fused._state.step == 1 and not fused._state.has_accumulated_grad()

    # same total gradient in one shot through the non-fused path
    other = FusedLinear.from_linear(copy.deepcopy(base), optimizer_type="adamw").train()
    other.use_fused_backward = False
    other.update_optimizer_config(lr=1e-3)
    other(torch.cat(xs)).sum().backward()
    torch.testing.assert_close(fused.weight, other.weight, rtol=1e-5, atol=1e-6)

    # and the fused path itself
    third = FusedLinear.from_linear(copy.deepcopy(base), optimizer_type="adamw").train()
    third.update_optimizer_config(lr=1e-3)
    third(torch.cat(xs)).sum().backward()
    torch.testing.assert_close(third.weight, other.weight, rtol=1e-5, atol=1e-6)


def test_bias_gets_a_normal_gradient():
    layer = FusedLinear(64, 32, bias=True, optimizer_type="sgd").to(DEV).train()
    layer.update_optimizer_config(lr=0.1, weight_decay=0.0)
    x = torch.randn(8, 64, device=DEV)
    w0 = layer.weight.detach().clone()
    layer(x).sum().backward()
    assert layer.weight.grad is None
    torch.testing.assert_close(layer.bias.grad, torch.full((32,), 8.0, device=DEV))
    expect = w0 - 0.1 * torch.ones(8, 32, device=DEV).t() @ x
    torch.testing.assert_close(layer.weight.detach(), expect, rtol=1e-4, atol=1e-5)


def test_no_config_behaves_like_a_plain_linear():
    layer = FusedLinear(64, 32).to(DEV).train()
    x = torch.randn(8, 64, device=DEV, requires_grad=True)
    layer(x).sum().backward()
    assert layer.weight.grad is not None and layer.weight.grad.shape == (32, 64)


@pytest.mark.parametrize("opt,mode", [("adamw", "bf16"), ("adamw", "int8"), ("adamw", "fp8"),
                                      ("adamw", "fp8_block"), ("sgdm", "bf16"), ("lion", "bf16"), ("sgd", "bf16")])
def test_checkpoint_round_trip(opt, mode):
    torch.manual_seed(2)

    def make():
        net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU())
        net.add_module("head", FusedLinear(128, 64, optimizer_type=opt, state_mode=mode, momentum=0.9))
        return net.to(DEV).to(torch.bfloat16).train()

    a = make()
    mgr = FusedOptimizerManager(a)
    xs = [torch.randn(32, 64, device=DEV, dtype=torch.bfloat16) for _ in range(4)]
    for x in xs[:2]:
        mgr.pre_step(lr=1e-2, weight_decay=0.0)
        a(x).float().pow(2).mean().backward()
    sd = copy.deepcopy(mgr.optimizer_state_dict())
    weights = copy.deepcopy(a.state_dict())
    assert sd["global_step"] == 2
    b = make()
    b.load_state_dict(weights)
    mgr_b = FusedOptimizerManager(b)
    mgr_b.load_optimizer_state_dict(sd)
    for net, mg in ((a, mgr), (b, mgr_b)):
        for x in xs[2:]:
            mg.pre_step(lr=1e-2, weight_decay=0.0)
            net(x).float().pow(2).mean().backward()
    assert torch.equal(a.head.weight, b.head.weight)
    assert a.head._state.step == b.head._state.step == (4 if True else 0)


def test_manager_quantize_override_and_counts():
    net = torch.nn.Sequential(FusedLinear(64, 64), torch.nn.ReLU(), FusedLinear(64, 64)).to(DEV).train()
    mgr = FusedOptimizerManager(net, quantize_state=True)
    assert mgr.num_fused_modules == 2 and mgr.num_fused_params == 2
    mgr.pre_step(lr=1e-3)
    net(torch.randn(8, 64, device=DEV)).sum().backward()
    assert net[0]._state.state_mode == "int8" and net[0]._state.m_q.dtype == torch.int8
    assert net[0]._config is net[2]._config


def test_device_hyper_ring_survives_a_host_far_ahead_of_the_gpu():
    """40 updates queued behind a busy GPU without a single synchronisation: every step must run with
    its own bias corrections although the pinned staging ring has only 16 slots (a slot is rewritten
    only after the copy that read it has run)."""
    from forge_b200 import kernel as K
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(3)
    BT, V, H = 64, 128, 256
    dy = (torch.randn(BT, V, device=dev, generator=gen) * 1e-2).bfloat16()
    x = torch.randn(BT, H, device=dev, generator=gen).bfloat16()
    w0 = (torch.randn(V, H, device=dev, generator=gen) * 0.02).bfloat16()
    ref, snaps_ref = [w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)], []
    for step in range(1, 41):
        K.fused_grad_adamw(dy, x, *ref, lr=1e-3 * step, weight_decay=0.01, step=step)
        snaps_ref.append(ref[0].clone())
    torch.cuda.synchronize()
    hd = K.DeviceHyper(dev)
    got, snaps = [w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)], []
    torch.cuda._sleep(int(4e8))                 # keeps the GPU busy while the host queues everything
    for step in range(1, 41):
        hd.update(lr=1e-3 * step, weight_decay=0.01, step=step)
        K.fused_grad_adamw(dy, x, *got, hyper_device=hd)
        snaps.append(got[0].clone())
    torch.cuda.synchronize()
    for step, (a, b) in enumerate(zip(snaps_ref, snaps), 1):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), f"step {step} ran with another step's hyper-parameters"


def test_device_hyper_blocks_follow_constructor_keywords():
    """Two AdamW groups that differ in weight_decay must not share a device block."""
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)

    def build():
        torch.manual_seed(0)
        net = torch.nn.Sequential(torch.nn.Linear(128, 128, bias=False), torch.nn.Linear(128, 128, bias=False)).to(dev).bfloat16()
        net[0] = FusedLinear.from_linear(net[0], weight_decay=0.0)
        net[1] = FusedLinear.from_linear(net[1], weight_decay=0.5)
        return net

    direct, blocks = build(), build()
    m_direct = FusedOptimizerManager(direct)
    m_blocks = FusedOptimizerManager(blocks).enable_device_hyper()
    assert len(m_blocks._device_hyper) == 2
    x = torch.randn(32, 128, device=dev).bfloat16()
    for _ in range(3):
        for net, mgr in ((direct, m_direct), (blocks, m_blocks)):
            mgr.pre_step(lr=1e-2)
            net(x).float().square().mean().backward()
    torch.cuda.synchronize()
    for a, b in zip(direct.parameters(), blocks.parameters()):
        assert torch.equal(a.data.view(torch.int16), b.data.view(torch.int16))
