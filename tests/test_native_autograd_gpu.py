"""The C++ autograd node (``forge_b200/_forge_autograd.so``) against the Python autograd function: both
issue the same library calls, so three training steps of a small network must leave bit-identical
weights, optimizer states and step counts, for every optimizer / moment storage, with and without
grouped launches; input and bias gradients must flow; what the node does not cover (gradient
accumulation) must fall back to the Python function without a trace."""

import pytest
import torch
import torch.nn as nn

from forge_b200 import FusedLinear, FusedOptimizerManager, native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bits(t):
    return t.view(torch.int16) if t.dtype == torch.bfloat16 else (t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.uint8))


class _Net(nn.Module):
    def __init__(self, **kw):
        super().__init__()
        self.layers = nn.ModuleList([nn.ModuleDict({"a": FusedLinear(256, 384, bias=True, **kw), "b": FusedLinear(384, 256, **kw)})
                                     for _ in range(2)])
        self.head = FusedLinear(256, 128, **kw)

    def forward(self, x):
        for blk in self.layers:
            x = x + blk["b"](torch.tanh(blk["a"](x)))
        return self.head(x)


def _train(use_native, kw, grouped, steps=3):
    native.reset()
    if not use_native:
        native._tried, native._mod = True, None
    assert (native.module() is not None) == use_native
    torch.manual_seed(0)
    net = _Net(**kw).to(DEV).bfloat16()
    mgr = FusedOptimizerManager(net)
    if grouped:
        mgr.group_updates("layer")
    gen = torch.Generator(device=DEV).manual_seed(1)
    xs = []
    for _ in range(steps):
        x = torch.randn(8, 16, 256, device=DEV, generator=gen).bfloat16().requires_grad_(True)
        mgr.pre_step(lr=1e-2)
        y = net(x)
        y.float().square().mean().backward()
        xs.append(x.grad.clone())
    mgr.flush_updates()
    torch.cuda.synchronize()
    native.reset()
    return net, mgr, xs, y


CASES = [dict(optimizer_type="adamw", state_mode="bf16"), dict(optimizer_type="adamw", state_mode="int8"),
         dict(optimizer_type="adamw", state_mode="fp8"), dict(optimizer_type="adamw", state_mode="fp8_block"),
         dict(optimizer_type="sgd"), dict(optimizer_type="sgdm", momentum=0.9), dict(optimizer_type="lion")]


@pytest.mark.parametrize("grouped", [False, True])
@pytest.mark.parametrize("kw", CASES, ids=[c.get("state_mode", c["optimizer_type"]) for c in CASES])
def test_native_node_equals_python_function(kw, grouped):
    if native.module() is None:
        pytest.skip("C++ autograd node not built")
    n_py, m_py, gx_py, _ = _train(False, kw, grouped)
    n_cc, m_cc, gx_cc, y = _train(True, kw, grouped)
    assert "CppNode" in y.grad_fn.name() and "FusedLinearFn" in y.grad_fn.name()      # the C++ node
    for (name, a), (_, b) in zip(n_py.named_parameters(), n_cc.named_parameters()):
        assert torch.equal(_bits(a.data), _bits(b.data)), name
        assert (a.grad is None) == (b.grad is None), name
        if a.grad is not None:      # biases go through autograd to the user's optimizer
            assert torch.equal(_bits(a.grad), _bits(b.grad)), name + ".grad"
    for a, b in zip(gx_py, gx_cc):
        assert torch.equal(_bits(a), _bits(b))
    sd_py, sd_cc = m_py.optimizer_state_dict()["modules"], m_cc.optimizer_state_dict()["modules"]
    assert sd_py.keys() == sd_cc.keys()
    for name in sd_py:
        for key, val in sd_py[name].items():
            if torch.is_tensor(val):
                assert torch.equal(_bits(val), _bits(sd_cc[name][key])), f"{name}.{key}"
            else:
                assert val == sd_cc[name][key], f"{name}.{key}"     # includes the step count (3)
    assert all(m._state.step == 3 for m in m_cc._fused_modules)


def test_node_follows_a_loaded_checkpoint_and_falls_back_where_it_must():
    if native.module() is None:
        pytest.skip("C++ autograd node not built")
    native.reset()
    torch.manual_seed(0)
    lin = FusedLinear(128, 128).to(DEV).bfloat16()
    x = torch.randn(16, 128, device=DEV).bfloat16()
    lin.update_optimizer_config(lr=1e-2)
    lin(x).float().sum().backward()
    sd = lin.get_optimizer_state_dict()
    assert sd["step"] == 1
    w1 = lin.weight.data.clone()
    lin(x).float().sum().backward()
    assert lin._state.step == 2
    # restore step 1: the node must pick up the replaced moment buffers and the restored step count
    lin.weight.data.copy_(w1)
    lin.load_optimizer_state_dict(sd)
    lin(x).float().sum().backward()
    w_again = lin.weight.data.clone()
    assert lin._state.step == 2
    ref = FusedLinear(128, 128).to(DEV).bfloat16()
    ref.weight.data.copy_(w1)
    ref.load_optimizer_state_dict(sd)
    ref.update_optimizer_config(lr=1e-2)
    native._tried, native._mod = True, None          # Python function
    ref(x).float().sum().backward()
    native.reset()
    torch.cuda.synchronize()
    assert torch.equal(_bits(w_again), _bits(ref.weight.data))
    # gradient accumulation is outside the node: same module, Python function
    y = lin(x)
    assert "CppNode" in y.grad_fn.name()
    lin.set_accumulating(True)
    y = lin(x)
    assert "CppNode" not in y.grad_fn.name() and "FusedLinearFunction" in y.grad_fn.name()
    y.float().sum().backward()
    lin.set_accumulating(False)
    y = lin(x)
    assert "CppNode" not in y.grad_fn.name() and "FusedLinearFunction" in y.grad_fn.name()     # a pending accumulated gradient
    y.float().sum().backward()
    assert lin._state.step == 3
    torch.cuda.synchronize()
