"""Grouped launches (``forge_wgrad_update_group``): several weights updated by one kernel launch must
come out with exactly the bits of one launch per weight, for every state mode, for weights of
different shapes, token counts and hyper-parameters inside one group, and through the module-level
``FusedOptimizerManager.group_updates``.  Everything goes through the C ABI."""

import pytest
import torch
import torch.nn as nn

from forge_b200 import FusedLinear, FusedOptimizerManager
from forge_b200 import kernel as K
from tests.util import ADAMW

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (BT, V, H) of the members of one group: a multi-tile weight, a single 128-row tile (only one CTA of
# a pair has rows), ragged shapes, a different token count, a weight with a half-tile tail
GROUP = [(256, 1024, 1024), (256, 128, 1024), (256, 392, 1088), (64, 264, 512), (256, 2048, 512), (8, 8, 64)]


def _bits(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t.view(torch.uint8)


def _assert_same(a, b, what):
    for i, (x, y) in enumerate(zip(a, b)):
        assert torch.equal(_bits(x), _bits(y)), f"{what}: tensor {i}: {(_bits(x) != _bits(y)).sum().item()} elements differ"


def _make(mode, gen, BT, V, H):
    dy = (torch.randn(BT, V, device=DEV, generator=gen) * 1e-2).bfloat16()
    x = torch.randn(BT, H, device=DEV, generator=gen).bfloat16()
    w = (torch.randn(V, H, device=DEV, generator=gen) * 0.02).bfloat16()
    if mode in ("bf16", "f32"):
        dt = torch.bfloat16 if mode == "bf16" else torch.float32
        st = [(torch.randn(V, H, device=DEV, generator=gen) * 1e-3).to(dt),
              (torch.randn(V, H, device=DEV, generator=gen).abs() * 1e-5).to(dt)]
    elif mode in ("int8", "fp8_block"):
        if mode == "int8":
            mq = torch.randint(-127, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
            vq = torch.randint(0, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
        else:
            mq = torch.randint(0, 120, (V, H), device=DEV, generator=gen, dtype=torch.uint8)
            vq = torch.randint(0, 120, (V, H), device=DEV, generator=gen, dtype=torch.uint8)
        st = [mq, vq, torch.rand(V, H // 64, device=DEV, generator=gen) * 1e-5 + 1e-6,
              torch.rand(V, H // 64, device=DEV, generator=gen) * 1e-9 + 1e-10]
    elif mode == "fp8":
        st = [torch.randint(0, 120, (V, H), device=DEV, generator=gen, dtype=torch.uint8),
              torch.randint(0, 120, (V, H), device=DEV, generator=gen, dtype=torch.uint8),
              torch.tensor(2e-5, device=DEV), torch.tensor(3e-9, device=DEV),
              torch.tensor(0.25, device=DEV), torch.tensor(0.0, device=DEV)]
    else:   # sgd, sgdm, lion
        st = [] if mode == "sgd" else [(torch.randn(V, H, device=DEV, generator=gen) * 1e-3).bfloat16()]
    return dy, x, w, st


class _Fp8State:
    def __init__(self, st):
        self.m_fp8 = st[0].view(torch.float8_e4m3fn)
        self.v_fp8 = st[1].view(torch.float8_e5m2)
        self.m_scale, self.v_scale, self.m_absmax_next, self.v_absmax_next = st[2:6]


def _update(mode, dy, x, w, st, step):
    hp = dict(ADAMW, step=step, lr=1e-3 * step)
    if mode in ("bf16", "f32"):
        K.fused_grad_adamw(dy, x, w, st[0], st[1], **hp)
    elif mode == "int8":
        K.fused_grad_adamw_int8state(dy, x, w, *st, qblock=64, **hp)
    elif mode == "fp8_block":
        K.fused_grad_adamw_fp8block(dy, x, w, *st, qblock=64, **hp)
    elif mode == "fp8":
        K.fused_grad_adamw_fp8state(dy, x, w, _Fp8State(st), **hp)
    elif mode == "sgd":
        K.fused_grad_sgd(dy, x, w, lr=0.01 * step, weight_decay=0.1)
    elif mode == "sgdm":
        K.fused_grad_sgd_momentum(dy, x, w, st[0], lr=0.01 * step, momentum=0.9, weight_decay=0.1)
    else:
        K.fused_grad_lion(dy, x, w, st[0], lr=1e-3 * step, weight_decay=0.1)


@pytest.mark.parametrize("mode", ["bf16", "f32", "int8", "fp8_block", "fp8", "sgd", "sgdm", "lion"])
def test_group_equals_single_launches_bitwise(mode):
    gen = torch.Generator(device=DEV).manual_seed(21)
    shapes = [s for s in GROUP if mode not in ("int8", "fp8_block") or s[2] % 64 == 0]
    probs = [_make(mode, gen, *s) for s in shapes]
    single = [(w.clone(), [t.clone() for t in st]) for _, _, w, st in probs]
    grouped = [(w.clone(), [t.clone() for t in st]) for _, _, w, st in probs]
    for i, (dy, x, _, _) in enumerate(probs):
        _update(mode, dy, x, single[i][0], single[i][1], step=i + 1)     # every member its own step and lr
    with K.UpdateGroup() as g:
        for i, (dy, x, _, _) in enumerate(probs):
            _update(mode, dy, x, grouped[i][0], grouped[i][1], step=i + 1)
        assert len(g) == len(probs)
        assert all(torch.equal(grouped[i][0], probs[i][2]) for i in range(len(probs))), "recorded calls must not launch"
    torch.cuda.synchronize()
    for i in range(len(probs)):
        assert not torch.equal(grouped[i][0], probs[i][2]), "weight did not change"
        _assert_same([single[i][0]] + single[i][1], [grouped[i][0]] + grouped[i][1], f"{mode} member {i} {shapes[i]}")


def test_group_of_mixed_configurations_splits_into_launches():
    """Entries of different kernel configurations in one call: consecutive runs share a launch."""
    gen = torch.Generator(device=DEV).manual_seed(22)
    order = ["bf16", "bf16", "int8", "sgd", "bf16"]
    probs = [_make(m, gen, 128, 256, 512) for m in order]
    single = [(w.clone(), [t.clone() for t in st]) for _, _, w, st in probs]
    grouped = [(w.clone(), [t.clone() for t in st]) for _, _, w, st in probs]
    for i, (m, (dy, x, _, _)) in enumerate(zip(order, probs)):
        _update(m, dy, x, single[i][0], single[i][1], step=2)
    with K.UpdateGroup():
        for i, (m, (dy, x, _, _)) in enumerate(zip(order, probs)):
            _update(m, dy, x, grouped[i][0], grouped[i][1], step=2)
    torch.cuda.synchronize()
    for i in range(len(probs)):
        _assert_same([single[i][0]] + single[i][1], [grouped[i][0]] + grouped[i][1], f"member {i}")


def test_group_larger_than_one_launch_and_fp32_operands():
    """Nineteen members (more than one launch holds) with fp32 dY / X: every member gets a split area
    of its own for the time the group is pending."""
    gen = torch.Generator(device=DEV).manual_seed(23)
    probs = []
    for i in range(19):
        V, H = 128 + 8 * i, 256
        probs.append((torch.randn(48, V, device=DEV, generator=gen), torch.randn(48, H, device=DEV, generator=gen),
                      torch.randn(V, H, device=DEV, generator=gen), torch.zeros(V, H, device=DEV), torch.zeros(V, H, device=DEV)))
    single = [(w.clone(), m.clone(), v.clone()) for _, _, w, m, v in probs]
    grouped = [(w.clone(), m.clone(), v.clone()) for _, _, w, m, v in probs]
    for i, (dy, x, *_r) in enumerate(probs):
        K.fused_grad_adamw(dy, x, *single[i], **ADAMW)
    with K.UpdateGroup():
        for i, (dy, x, *_r) in enumerate(probs):
            K.fused_grad_adamw(dy, x, *grouped[i], **ADAMW)
    torch.cuda.synchronize()
    for i in range(19):
        _assert_same(single[i], grouped[i], f"member {i}")


def test_group_rejects_a_bad_entry_before_launching_anything():
    gen = torch.Generator(device=DEV).manual_seed(24)
    dy, x, w, st = _make("bf16", gen, 64, 128, 256)
    w0 = w.clone()
    with pytest.raises(ValueError):
        with K.UpdateGroup():
            K.fused_grad_adamw(dy, x, w, st[0], st[1], **ADAMW)
            K.fused_grad_adamw(dy, x, w.clone(), st[0].clone(), st[1].clone(), **dict(ADAMW, step=0))
    torch.cuda.synchronize()
    assert torch.equal(w, w0), "a rejected group must leave every weight untouched"


class _Block(nn.Module):
    def __init__(self, hid, kv, ffn):
        super().__init__()
        self.q, self.k, self.v = nn.Linear(hid, hid, bias=False), nn.Linear(hid, kv, bias=False), nn.Linear(hid, kv, bias=False)
        self.o = nn.Linear(hid, hid, bias=False)
        self.gate, self.up, self.down = nn.Linear(hid, ffn, bias=False), nn.Linear(hid, ffn, bias=False), nn.Linear(ffn, hid, bias=False)

    def forward(self, x):
        a = self.o(torch.tanh(self.q(x)) * torch.cat([self.k(x), self.v(x)] * 2, dim=-1)[..., : x.shape[-1]])
        x = x + a
        return x + self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))


class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.layers = nn.ModuleList([_Block(256, 128, 512) for _ in range(2)])
        self.head = nn.Linear(256, 384, bias=False)

    def forward(self, x):
        for blk in self.layers:
            x = blk(x)
        return self.head(x)


def _fuse(model, state_mode):
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear):
                setattr(parent, name, FusedLinear.from_linear(child, state_mode=state_mode, weight_decay=0.01))
    return model


@pytest.mark.parametrize("state_mode", ["bf16", "int8", "fp8"])
def test_manager_layer_groups_train_bit_identically(state_mode):
    """Three training steps of a two-block toy model: one launch per block (seven projections) gives
    the weights and states of one launch per linear, bit for bit; the ungrouped head is unaffected."""
    torch.manual_seed(0)
    base = _Toy().to(DEV).bfloat16()
    models = []
    for grouped in (False, True):
        m = _Toy().to(DEV).bfloat16()
        m.load_state_dict(base.state_dict())
        m = _fuse(m, state_mode)
        mgr = FusedOptimizerManager(m)
        if grouped:
            mgr.group_updates("layer")
            assert len(mgr._update_groups) == 2 and all(len(g) == 7 for g in mgr._update_groups)
        models.append((m, mgr))
    gen = torch.Generator(device=DEV).manual_seed(1)
    for step in range(3):
        x = torch.randn(4, 32, 256, device=DEV, generator=gen).bfloat16()
        for m, mgr in models:
            mgr.pre_step(lr=1e-3)
            m(x).float().square().mean().backward()
    torch.cuda.synchronize()
    (m0, g0), (m1, g1) = models
    for (n0, p0), (n1, p1) in zip(m0.named_parameters(), m1.named_parameters()):
        assert torch.equal(_bits(p0.data), _bits(p1.data)), n0
    sd0, sd1 = g0.optimizer_state_dict()["modules"], g1.optimizer_state_dict()["modules"]
    assert sd0.keys() == sd1.keys() and len(sd0) == 15
    for name in sd0:
        for key, val in sd0[name].items():
            if torch.is_tensor(val):
                assert torch.equal(_bits(val), _bits(sd1[name][key])), f"{name}.{key}"
            else:
                assert val == sd1[name][key], f"{name}.{key}"


def test_incomplete_group_is_flushed_by_the_next_pre_step():
    """A member that takes no part in a backward pass must not hold the others' updates back."""
    torch.manual_seed(0)
    a, b = nn.Linear(128, 128, bias=False), nn.Linear(128, 128, bias=False)
    model = nn.ModuleDict({"a": a, "b": b}).to(DEV).bfloat16()
    model = _fuse(model, "bf16")
    mgr = FusedOptimizerManager(model).group_updates([[model["a"], model["b"]]])
    w_a = model["a"].weight.data.clone()
    mgr.pre_step(lr=1e-2)
    x = torch.randn(16, 128, device=DEV).bfloat16()
    model["a"](x).float().square().mean().backward()     # only one of the two members runs
    torch.cuda.synchronize()
    assert torch.equal(model["a"].weight.data, w_a), "the update waits for the rest of its group"
    mgr.pre_step(lr=1e-2)                                # flushes what the last pass left
    torch.cuda.synchronize()
    assert not torch.equal(model["a"].weight.data, w_a)


def test_group_with_members_on_both_autograd_paths_launches_inside_the_backward():
    """One member of a group runs its backward in the Python autograd function (here: called directly,
    as the tensor-parallel layers with a fused scatter do) and the others in the C++ node: the group
    still goes out as soon as its last member has reported -- nothing is left for ``pre_step`` -- and
    the weights equal those of ungrouped launches bit for bit."""
    from forge_b200 import native
    from forge_b200.autograd import FusedLinearFunction
    torch.manual_seed(0)
    base = nn.ModuleDict({k: nn.Linear(128, 192, bias=False) for k in ("a", "b", "c")}).to(DEV).bfloat16()
    runs = []
    for grouped in (False, True):
        m = nn.ModuleDict({k: nn.Linear(128, 192, bias=False) for k in ("a", "b", "c")}).to(DEV).bfloat16()
        m.load_state_dict(base.state_dict())
        m = _fuse(m, "int8").train()
        mgr = FusedOptimizerManager(m)
        if grouped:
            mgr.group_updates([[m["a"], m["b"], m["c"]]])
        runs.append((m, mgr))
    gen = torch.Generator(device=DEV).manual_seed(2)
    for step in range(3):
        x = torch.randn(64, 128, device=DEV, generator=gen).bfloat16()
        for m, mgr in runs:
            mgr.pre_step(lr=1e-2)
            b = m["b"]
            b._ensure_state()
            yb = FusedLinearFunction.apply(x, b.weight, None, b._state, b._config, False, None, True, b._update_group)
            ya, yc = m["a"](x), m["c"](x)
            if native.module() is not None:
                assert "CppNode" in ya.grad_fn.name() and "CppNode" not in yb.grad_fn.name()
            (ya + yb + yc).float().square().mean().backward()
            for g in mgr._update_groups:
                assert g.pending() == 0, "the group was complete at the end of the backward pass"
    torch.cuda.synchronize()
    (m0, _), (m1, _) = runs
    for k in ("a", "b", "c"):
        assert torch.equal(_bits(m0[k].weight.data), _bits(m1[k].weight.data)), k
        s0, s1 = m0[k].get_optimizer_state_dict(), m1[k].get_optimizer_state_dict()
        for key, val in s0.items():
            if torch.is_tensor(val):
                assert torch.equal(_bits(val), _bits(s1[key])), f"{k}.{key}"
