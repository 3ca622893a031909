"""CPU-only checks of the host side: the shared library loads and exports every symbol the public
header declares, host-only entry points behave, the state allocator reproduces the reference's
buffer layout (golden ``state_layout.json``), manager / config logic, error conventions."""

import ctypes
import json
import os
import re

import pytest
import torch

from forge_b200 import FusedLinear, FusedOptimizerManager, FusedOptimizerState, OptimizerConfig, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "forge_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(forge_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/forge_b200.h but not exported"
    assert sorted(_lib.EXPORTED_SYMBOLS) == declared
    assert lib.forge_abi_version() == 3
    assert isinstance(_lib.last_error(), str)


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.forge_wgrad_scratch_bytes(512, 1024, 1024, _lib.DT_BF16) == 0
    assert lib.forge_wgrad_scratch_bytes(100, 256, 128, _lib.DT_F32) == 3 * 128 * (256 + 128) * 2
    mb, sb, nm = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_int32()
    for opt, mode, exp in [(_lib.OPT_ADAMW, _lib.ST_BF16, (2 * 4096 * 1024, 0, 2)),
                           (_lib.OPT_ADAMW, _lib.ST_INT8, (4096 * 1024, 4096 * 16 * 4, 2)),
                           (_lib.OPT_ADAMW, _lib.ST_FP8_TENSOR, (4096 * 1024, 4, 2)),
                           (_lib.OPT_LION, _lib.ST_F32, (4 * 4096 * 1024, 0, 1)),
                           (_lib.OPT_SGD, _lib.ST_NONE, (0, 0, 0))]:
        assert lib.forge_state_bytes(opt, mode, 4096, 1024, 64, ctypes.byref(mb), ctypes.byref(sb), ctypes.byref(nm)) == 0
        assert (mb.value, sb.value, nm.value) == exp
    rc = lib.forge_state_bytes(_lib.OPT_ADAMW, _lib.ST_INT8, 16, 100, 64, ctypes.byref(mb), ctypes.byref(sb), ctypes.byref(nm))
    assert rc == _lib.FORGE_ERR_SHAPE and "divisible" in _lib.last_error()
    assert lib.forge_wgrad_update(None, None) == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_optimizer_update(None, None) == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_fp8_prestep(None, None, None, None, None) == _lib.FORGE_ERR_INVALID_ARG
    with pytest.raises(ValueError):
        _lib.check(_lib.FORGE_ERR_SHAPE, "x")
    with pytest.raises(_lib.ForgeLibraryError):
        _lib.check(_lib.FORGE_ERR_CUDA, "x")


def test_operators_refuse_cpu_tensors():
    from forge_b200 import kernel as K
    with pytest.raises(_lib.ForgeLibraryError):
        K.fused_grad_sgd(torch.zeros(8, 8), torch.zeros(8, 8), torch.zeros(8, 8))
    with pytest.raises(_lib.ForgeLibraryError):
        K.optimizer_only_adamw(torch.zeros(8, 16), torch.zeros(8, 16), torch.zeros(8, 16), torch.zeros(8, 16))


def test_state_layout_matches_reference(golden_dir):
    layout = json.load(open(os.path.join(golden_dir, "state_layout.json")))
    w = torch.zeros(256, 128, dtype=torch.bfloat16)
    for mode in ("bf16", "int8", "fp8"):
        st = FusedOptimizerState(w, "adamw", state_mode=mode)
        assert st.step == layout[mode]["step"] and st.qblock_size == layout[mode]["qblock"]
        assert st.quantize_state == layout[mode]["quantize_state"]
        for name in st._buffer_names():
            assert getattr(st, name) is None     # lazy
        st.ensure_buffers()
        ref = layout[mode]["buffers"]
        # the reference's per-tile absmax scratch arrays have no counterpart here
        ref = {k: v for k, v in ref.items() if "scratch" not in k}
        assert set(st._buffer_names()) == set(ref)
        for name, spec in ref.items():
            t = getattr(st, name)
            assert list(t.shape) == spec["shape"] and str(t.dtype) == spec["dtype"]
            assert bool((t.float() == spec["init"]).all())
    assert FusedOptimizerState(w, "sgd")._buffer_names() == ()
    assert layout["sgd"]["buffers"] == {}


def test_state_modes_and_errors():
    w = torch.zeros(64, 128)
    assert FusedOptimizerState(w, quantize_state=True).state_mode == "int8"
    with pytest.raises(ValueError):
        FusedOptimizerState(w, "adagrad")
    with pytest.raises(ValueError):
        FusedOptimizerState(w, "adamw", state_mode="fp4")
    with pytest.raises(ValueError):
        FusedOptimizerState(w, "lion", state_mode="int8")
    st = FusedOptimizerState(torch.zeros(64, 100), "adamw", state_mode="int8")
    with pytest.raises(ValueError):
        st.ensure_buffers()
    st = FusedOptimizerState(w, "adamw", state_mode="fp8_block")
    st.ensure_buffers()
    assert st.m_q.dtype == torch.float8_e4m3fn and st.m_scale.shape == (64, 2)
    st = FusedOptimizerState(w.bfloat16(), "lion")
    st.ensure_buffers()
    assert st.m.dtype == torch.bfloat16 and not hasattr(st, "v")
    assert FusedOptimizerState(w.bfloat16(), "adamw", state_dtype=torch.float32)._state_dtype == torch.float32


def test_state_dict_round_trip_all_modes():
    w = torch.zeros(64, 128)
    for opt, mode in [("adamw", "bf16"), ("adamw", "int8"), ("adamw", "fp8"), ("adamw", "fp8_block"),
                      ("sgdm", "bf16"), ("sgd", "bf16")]:
        a = FusedOptimizerState(w, opt, state_mode=mode)
        a.ensure_buffers()
        a.step = 7
        for n in a._buffer_names():
            t = getattr(a, n)
            if t.dtype in (torch.float32, torch.bfloat16):
                t.add_(0.25)
        sd = a.state_dict()
        assert sd["step"] == 7 and sd["optimizer_type"] == opt and sd["state_mode"] == mode
        b = FusedOptimizerState(w, opt, state_mode=mode)
        b.load_state_dict(sd)
        assert b.step == 7
        for n in a._buffer_names():
            assert torch.equal(getattr(a, n).reshape(-1).view(torch.uint8), getattr(b, n).reshape(-1).view(torch.uint8))
            assert getattr(a, n).data_ptr() != getattr(b, n).data_ptr()
    other = FusedOptimizerState(w, "adamw", state_mode="int8")
    other.ensure_buffers()
    with pytest.raises(ValueError):
        FusedOptimizerState(w, "adamw", state_mode="bf16").load_state_dict(other.state_dict())
    # a reference-format dict (no state_mode key) still loads
    legacy = {"optimizer_type": "adamw", "step": 3, "quantize_state": False, "m": torch.ones(64, 128), "v": torch.ones(64, 128)}
    c = FusedOptimizerState(w, "adamw")
    c.load_state_dict(legacy)
    assert c.step == 3 and bool((c.m == 1).all())


def test_accumulation_buffer():
    st = FusedOptimizerState(torch.zeros(4, 4), "adamw")
    assert not st.has_accumulated_grad() and st.pop_accumulated_grad() is None
    st.accumulate_grad(torch.ones(4, 4, dtype=torch.bfloat16))
    st.accumulate_grad(torch.ones(4, 4) * 2)
    g = st.pop_accumulated_grad()
    assert g.dtype == torch.float32 and bool((g == 3).all()) and not st.has_accumulated_grad()


def test_optimizer_config():
    c = OptimizerConfig(lr=3e-4, step=12, foo="bar")
    assert (c.optimizer_type, c.lr, c.beta1, c.beta2, c.eps, c.weight_decay) == ("adamw", 3e-4, 0.9, 0.999, 1e-8, 0.01)
    assert not hasattr(c, "foo") and c.momentum == 0.0 and c.nesterov is False
    assert OptimizerConfig(lr=1.0) == OptimizerConfig(lr=1.0) and OptimizerConfig(lr=1.0) != OptimizerConfig(lr=2.0)


def test_fused_linear_surface():
    lin = torch.nn.Linear(32, 16, bias=True)
    f = FusedLinear.from_linear(lin, optimizer_type="adamw", state_mode="int8", weight_decay=0.1)
    assert f.weight.data_ptr() == lin.weight.data_ptr() and f.bias.data_ptr() == lin.bias.data_ptr()
    assert (f.in_features, f.out_features, f.state_mode, f.use_fused_backward) == (32, 16, "int8", True)
    assert "state_mode=int8" in repr(f) and f.get_optimizer_state_dict() is None
    f.update_optimizer_config(lr=5e-4, step=3)
    assert f._config.lr == 5e-4 and f._config.weight_decay == 0.1
    shared = OptimizerConfig(lr=1.0)
    f.update_optimizer_config(shared)
    assert f._config is shared
    f.set_accumulating(True)
    assert f._is_accumulating
    f.eval()
    assert f(torch.randn(4, 32)).shape == (4, 16) and f._state is None
    g = FusedLinear(8, 4, bias=False, quantize_state=True)
    assert g.state_mode == "int8" and g.bias is None and g.weight.shape == (4, 8)


def test_manager_logic():
    net = torch.nn.Sequential(torch.nn.Linear(8, 8), FusedLinear(8, 8, bias=True),
                              FusedLinear(8, 8, optimizer_type="sgdm", momentum=0.5))
    mgr = FusedOptimizerManager(net, gradient_accumulation_steps=2)
    non_fused = {id(p) for p in mgr.get_non_fused_params()}
    assert id(net[1].weight) not in non_fused and id(net[1].bias) in non_fused and id(net[0].weight) in non_fused
    assert mgr.num_fused_modules == 2 and mgr.num_fused_params == 2 and mgr.l2_manager is None
    mgr.pre_step(lr=1e-3)
    assert net[1]._is_accumulating and mgr._global_step == 0 and mgr._micro_step == 1
    mgr.pre_step(lr=2e-3, weight_decay=0.2)
    assert not net[1]._is_accumulating and mgr._global_step == 1
    assert net[1]._config.optimizer_type == "adamw" and net[1]._config.lr == 2e-3 and net[1]._config.weight_decay == 0.2
    assert net[2]._config.optimizer_type == "sgdm" and net[2]._config.momentum == 0.5
    mgr.pre_step()
    assert net[1]._config.lr == 1e-4
    mgr.pre_step(lr=1.0, is_accumulating=True)
    assert net[2]._is_accumulating
    sd = mgr.optimizer_state_dict()
    assert sd["micro_step"] == 4 and sd["modules"] == {}
    net[1]._ensure_state()
    assert set(mgr.optimizer_state_dict()["modules"]) == {"1"}
    mgr2 = FusedOptimizerManager(net)
    mgr2.load_optimizer_state_dict(mgr.optimizer_state_dict())
    assert mgr2._micro_step == 4 and mgr2._global_step == mgr._global_step


def test_alias_package():
    import fused_grad_optimizer
    from fused_grad_optimizer.kernel import fused_grad_adamw, fused_grad_adamw_int8state, fused_grad_sgd  # noqa: F401
    from fused_grad_optimizer.kernel_fp8_state import fused_grad_adamw_fp8state  # noqa: F401
    from fused_grad_optimizer.module import FusedLinear as FL, FusedOptimizerManager as FM  # noqa: F401
    from fused_grad_optimizer.state import FusedOptimizerState as FS, OptimizerConfig as OC  # noqa: F401
    assert fused_grad_optimizer.FusedLinear is FusedLinear and FL is FusedLinear


def test_unsupported_shapes_are_refused_at_the_first_forward():
    """Row pitches the copy engine cannot take raise a clear ValueError before any kernel is involved."""
    lin = FusedLinear(100, 64).train()                     # fp32 weights: in_features % 4 is fine ...
    lin = lin.bfloat16()                                   # ... bf16 needs in_features % 8
    with pytest.raises(ValueError, match="multiple of 8"):
        lin(torch.zeros(4, 100, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="divisible by 64"):
        FusedLinear(96, 64, state_mode="int8").train()(torch.zeros(4, 96))
    FusedLinear(96, 64).eval()(torch.zeros(4, 96))          # eval mode is a plain linear: anything goes


def test_layer_groups_are_formed_by_name_prefix():
    """``group_updates("layer")``: modules under the same numbered block share a launch, largest weights
    first, at most eight per group; modules outside numbered blocks stay on their own."""
    import torch.nn as nn

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = nn.ModuleDict({n: FusedLinear(64, o) for n, o in (("q", 64), ("k", 16), ("v", 16), ("o", 64))})
            self.mlp = nn.ModuleDict({"gate": FusedLinear(64, 128), "up": FusedLinear(64, 128), "down": FusedLinear(128, 64)})

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Blk(), Blk()])
            self.lm_head = FusedLinear(64, 256)

    net = Net()
    mgr = FusedOptimizerManager(net).group_updates("layer")
    assert len(mgr._update_groups) == 2 and all(len(g) == 7 for g in mgr._update_groups)
    assert net.lm_head._update_group is None
    assert net.layers[0].attn["q"]._update_group is net.layers[0].mlp["down"]._update_group
    assert net.layers[0].attn["q"]._update_group is not net.layers[1].attn["q"]._update_group
    mgr.group_updates([[net.layers[0].attn["q"], net.layers[0].attn["k"]]])      # regrouping replaces the old groups
    assert len(mgr._update_groups) == 1 and net.layers[1].attn["q"]._update_group is None
    with pytest.raises(ValueError):
        mgr.group_updates([[net.lm_head, FusedLinear(8, 8)]])                     # not a module of this model
    mixed = Net()
    mixed.layers[0].attn["k"] = FusedLinear(64, 16, state_mode="int8")
    g = FusedOptimizerManager(mixed).group_updates("layer")._update_groups
    assert sorted(len(x) for x in g) == [6, 7]          # the int8 module cannot share a launch with bf16 ones


def test_peer_helpers_work_without_a_process_group():
    """A single-GPU process never initialises torch.distributed: the peer-memory classes then run their
    one-rank forms."""
    import torch.distributed as dist
    from forge_b200 import peer
    if not dist.is_initialized():
        assert peer._world_and_rank() == (1, 0)
        t = torch.zeros(4)
        assert peer._share(t)[0] is t
