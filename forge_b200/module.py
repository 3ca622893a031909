"""``FusedLinear`` and ``FusedOptimizerManager`` -- the module-level surface.

Mirror of ``src/fused_grad_optimizer/module.py`` (``FusedLinear`` :35-154, ``FusedOptimizerManager``
:157-266): same constructor arguments, methods and attributes, so a training loop written for the
reference runs unchanged:

    model.proj = FusedLinear.from_linear(model.proj, optimizer_type="adamw", state_mode="int8")
    manager = FusedOptimizerManager(model)
    other = torch.optim.AdamW(manager.get_non_fused_params(), lr=1e-4)
    for batch in data:
        manager.pre_step(lr=lr)
        model(**batch).loss.backward()      # fused layers update their weights here
        other.step(); other.zero_grad()

Deliberate differences from the reference:
* ``pre_step`` builds the step's config with each module's own ``optimizer_type`` and constructor
  keywords (the reference hard-codes ``"adamw"`` and drops the module's keywords,
  ``module.py:229``, which breaks SGD modules under a manager).
* a manager-level ``quantize_state`` override also switches ``state_mode`` (in the reference it only
  sets ``module.quantize_state``, which ``_ensure_state`` then ignores, ``module.py:189-190,93-96``).
* ``from_linear`` adopts the source layer's storage without first materialising and initialising a
  throw-away fp32 weight of the same shape (``module.py:50-51,86``).
* there is no L2-pinning manager; ``use_l2_pinning`` is accepted and ignored (the kernel keeps the
  activation panels L2-resident with per-load cache policies instead).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from forge_b200 import autograd as fa
from forge_b200 import native
from forge_b200.autograd import FusedLinearFunction, LayerUpdateGroup
from forge_b200.state import FusedOptimizerState, OptimizerConfig


class FusedLinear(nn.Module):
    """Drop-in ``nn.Linear`` whose backward computes the weight gradient tile by tile on chip and
    feeds it straight to the optimizer; the (out_features, in_features) gradient is never allocated."""

    _native_dgrad = False    # the use_forge_dgrad switch as last told to the C++ autograd node

    def __init__(self, in_features, out_features, bias=False, optimizer_type="adamw",
                 quantize_state=False, state_mode=None, _adopt: nn.Linear | None = None,
                 **optimizer_kwargs):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        if _adopt is not None:
            # share the existing parameters' storage (fresh Parameter objects, same data)
            self.weight = nn.Parameter(_adopt.weight.data, requires_grad=_adopt.weight.requires_grad)
            self.bias = (nn.Parameter(_adopt.bias.data, requires_grad=_adopt.bias.requires_grad)
                         if _adopt.bias is not None else None)
        else:
            self.weight = nn.Parameter(torch.empty(out_features, in_features))
            nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
            if bias:
                bound = 1 / math.sqrt(in_features) if in_features > 0 else 0
                self.bias = nn.Parameter(torch.empty(out_features).uniform_(-bound, bound))
            else:
                self.bias = None
        self.optimizer_type = optimizer_type
        self.quantize_state = quantize_state
        self.state_mode = state_mode if state_mode is not None else ("int8" if quantize_state else "bf16")
        self.optimizer_kwargs = optimizer_kwargs
        self._state: FusedOptimizerState | None = None
        self._config: OptimizerConfig | None = None
        self._is_accumulating = False
        self._l2_manager = None
        # False: materialise grad_W with a library GEMM and run the optimizer-only kernel
        self.use_fused_backward = True
        # set by FusedOptimizerManager.group_updates: the launch this module's update is issued with
        self._update_group = None
        # handle of the C++ autograd node (forge_b200.native), created on first use
        self._native = None
        self._native_key = None

    @classmethod
    def from_linear(cls, linear: nn.Linear, optimizer_type="adamw", quantize_state=False,
                    state_mode=None, **optimizer_kwargs):
        """Create from an existing ``nn.Linear``, sharing its weight (and bias) storage."""
        return cls(linear.in_features, linear.out_features, bias=linear.bias is not None,
                   optimizer_type=optimizer_type, quantize_state=quantize_state,
                   state_mode=state_mode, _adopt=linear, **optimizer_kwargs)

    def _check_shape(self):
        """The kernels move rows with the copy engine, which needs 16-byte row pitches: say so here, at the
        first training forward, not from inside a backward pass (the reference masks ragged shapes in
        its Triton kernels, ``kernel.py:261-265``)."""
        per16 = 16 // self.weight.element_size()
        if self.in_features % per16 or self.out_features % 8:
            raise ValueError(
                f"FusedLinear({self.in_features}, {self.out_features}) with {self.weight.dtype} weights: in_features must be a "
                f"multiple of {per16} and out_features a multiple of 8 (16-byte rows of W, X and dY); pad the layer or keep it "
                f"a plain nn.Linear")
        if self.state_mode in ("int8", "fp8_block") and self.in_features % 64:
            raise ValueError(f"state_mode={self.state_mode!r} needs in_features ({self.in_features}) divisible by 64, the "
                             f"quantisation block (as in the reference, kernel.py:1513)")
        if self.state_mode == "fp8" and self.in_features % 16:
            raise ValueError(f"state_mode='fp8' needs in_features ({self.in_features}) divisible by 16")

    def _ensure_state(self):
        if self._state is None:
            self._check_shape()
            self._state = FusedOptimizerState(self.weight, self.optimizer_type,
                                              quantize_state=self.quantize_state,
                                              state_mode=self.state_mode)

    def update_optimizer_config(self, config=None, **kwargs):
        """Set the hyper-parameters of the coming step: a shared ``OptimizerConfig`` or keywords
        merged over the constructor's ``optimizer_kwargs``."""
        if config is not None:
            self._config = config
        else:
            self._config = OptimizerConfig(optimizer_type=self.optimizer_type,
                                           **{**self.optimizer_kwargs, **kwargs})

    def set_accumulating(self, is_accumulating: bool):
        self._is_accumulating = is_accumulating

    def set_l2_manager(self, l2_manager):
        self._l2_manager = l2_manager

    def _native_handle(self, nat):
        """The C++ node's per-module handle, rebuilt whenever the weight or a state buffer moved."""
        st = self._state
        key = (self.weight.data_ptr(), st._version, self.weight.stride(0))
        if self._native is None or self._native_key != key:
            st.ensure_buffers()
            key = (self.weight.data_ptr(), st._version, self.weight.stride(0))
            from forge_b200.autograd import native_proto
            h = self._native if self._native is not None else nat.Linear()
            h.set_proto(bytes(native_proto(self.weight, st)))
            if st._native is not h:
                h.step = st.step
                st._native = h
            self._native, self._native_key = h, key
        g = self._update_group
        self._native.set_group(g.native if g is not None else None)
        return self._native

    def forward(self, x):
        if not self.training:
            return F.linear(x, self.weight, self.bias)
        self._ensure_state()
        cfg = self._config
        if (cfg is not None and not self._is_accumulating and self.use_fused_backward and x.is_cuda
                and x.dtype == torch.bfloat16 and self._state._pending_grad is None):
            nat = native.module()
            if nat is not None:
                if cfg.optimizer_type != self._state.optimizer_type:
                    raise ValueError(f"config asks for {cfg.optimizer_type!r} but the state was built for "
                                     f"{self._state.optimizer_type!r}")
                h = self._native_handle(nat)
                hd = cfg.hyper_device
                h.set_hyper(cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.momentum, bool(cfg.nesterov),
                            hd.data_ptr() if hd is not None else 0)
                if fa.use_forge_dgrad != FusedLinear._native_dgrad:
                    nat.set_use_forge_dgrad(bool(fa.use_forge_dgrad))
                    FusedLinear._native_dgrad = fa.use_forge_dgrad
                return nat.fused_linear(x, self.weight, self.bias, h)
        return FusedLinearFunction.apply(x, self.weight, self.bias, self._state, self._config,
                                         self._is_accumulating, self._l2_manager,
                                         self.use_fused_backward, self._update_group)

    def get_optimizer_state_dict(self):
        return None if self._state is None else self._state.state_dict()

    def load_optimizer_state_dict(self, d):
        self._ensure_state()
        self._state.load_state_dict(d)

    def extra_repr(self):
        s = (f"in_features={self.in_features}, out_features={self.out_features}, "
             f"bias={self.bias is not None}, optimizer={self.optimizer_type}")
        if self.state_mode != "bf16":
            s += f", state_mode={self.state_mode}"
        return s


class FusedOptimizerManager:
    """Coordinates every ``FusedLinear`` of a model: per-step configs, accumulation phase, the list
    of parameters left to the user's own optimizer, and checkpointing of the fused state."""

    def __init__(self, model: nn.Module, gradient_accumulation_steps: int = 1,
                 use_l2_pinning: bool = False, quantize_state: bool | None = None):
        self.model = model
        self.gradient_accumulation_steps = gradient_accumulation_steps
        self._global_step = 0
        self._micro_step = 0
        self._l2_manager = None  # accepted for signature compatibility; see the module docstring
        self._update_groups: list[LayerUpdateGroup] = []   # see group_updates
        self._device_hyper = {}   # _group_key -> DeviceHyper, see enable_device_hyper
        self._use_device_hyper = False
        self._fused_modules: list[FusedLinear] = []
        self._fused_module_names: dict[int, str] = {}
        self._fused_param_ids: set[int] = set()
        for name, module in model.named_modules():
            if not isinstance(module, FusedLinear):
                continue
            if quantize_state is not None and module._state is None:
                module.quantize_state = quantize_state
                module.state_mode = "int8" if quantize_state else "bf16"
            self._fused_modules.append(module)
            self._fused_module_names[id(module)] = name
            # only the weight is fused; a bias keeps flowing through autograd to the user's optimizer
            self._fused_param_ids.add(id(module.weight))

    def get_non_fused_params(self) -> list[nn.Parameter]:
        """Parameters NOT updated by the fused kernels -- hand these to your own optimizer."""
        return [p for p in self.model.parameters()
                if p.requires_grad and id(p) not in self._fused_param_ids]

    def pre_step(self, lr: float | None = None, step: int | None = None,
                 is_accumulating: bool | None = None, **kwargs):
        """Call before each forward pass.  ``step`` is accepted for compatibility; the bias
        correction uses each parameter's own update count, as in the reference."""
        self._micro_step += 1
        if is_accumulating is None:
            is_accumulating = (self._micro_step % self.gradient_accumulation_steps) != 0
        if not is_accumulating:
            self._global_step += 1
        if lr is None:
            lr = 1e-4
        for g in self._update_groups:      # nothing recorded in an earlier pass may wait any longer
            g.flush()
        for m in self._fused_modules:      # norms shared by sibling linears: forget passes that never finished
            shared = getattr(m, "_shared", None)
            if shared is not None:
                shared.reset()
        # one shared config per distinct (optimizer, constructor keywords, device) instead of one per module
        configs: dict[tuple, OptimizerConfig] = {}
        for m in self._fused_modules:
            key = self._group_key(m)
            cfg = configs.get(key)
            if cfg is None:
                cfg = OptimizerConfig(optimizer_type=m.optimizer_type,
                                      **{**m.optimizer_kwargs, **kwargs, "lr": lr})
                if self._use_device_hyper and not is_accumulating:
                    hd = self._device_hyper.get(key)
                    if hd is None:      # a group that appeared after enable_device_hyper()
                        from forge_b200.kernel import DeviceHyper
                        hd = self._device_hyper[key] = DeviceHyper(m.weight.device)
                    hd.update(lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.eps,
                              weight_decay=cfg.weight_decay, step=max(self._global_step, 1),
                              momentum=cfg.momentum, nesterov=cfg.nesterov)
                    cfg.hyper_device = hd
                configs[key] = cfg
            m._config = cfg
            m._is_accumulating = is_accumulating

    @staticmethod
    def _group_key(m: "FusedLinear") -> tuple:
        """Modules that share this key train with the same hyper-parameters on the same device."""
        return (m.optimizer_type, tuple(sorted(m.optimizer_kwargs.items())), str(m.weight.device))

    def enable_device_hyper(self, device=None):
        """Keep the step's hyper-parameters in device memory -- one 64-byte block per distinct
        (optimizer type, constructor keywords, device) of the fused modules, rewritten by
        ``pre_step`` -- so that a CUDA graph holding the backward pass can be replayed with a new lr
        and step count.  Modules built with different keywords (say ``weight_decay=0`` on some
        layers) or living on different GPUs get blocks of their own.  The step count is the manager's
        global step; every fused parameter is assumed to be updated on every non-accumulating step.
        ``device`` is accepted for compatibility and ignored: a block lives where its modules do.
        No reference counterpart."""
        from forge_b200.kernel import DeviceHyper
        self._use_device_hyper = True
        for m in self._fused_modules:
            key = self._group_key(m)
            if key not in self._device_hyper:
                self._device_hyper[key] = DeviceHyper(m.weight.device)
        return self

    def group_updates(self, groups="layer", max_group: int = 16, layers_per_group: int = 1):
        """Issue the fused updates of several linears as ONE launch each (``forge_wgrad_update_group``):
        the start-up and ragged end of a launch are then paid once per group instead of once per
        weight, which is most of what the small projections (k, v; every row shard in tensor-parallel
        mode) cost.  ``groups`` is a list of lists of ``FusedLinear`` modules, or ``"layer"``: modules
        whose names share the prefix up to their last numeric component (``model.layers.17.`` ...)
        form a group, largest weights first, at most ``max_group`` (<= 16) per launch;
        ``layers_per_group=2`` puts two consecutive numbered blocks into one launch (smaller shards in
        tensor-parallel mode: fewer, larger launches).  Members must
        share optimizer type, state mode, weight dtype and device.  A group launches when its last
        member's backward has run; ``pre_step`` (and ``flush_updates``) issue anything left over.
        Results are bit-identical to ungrouped launches.  No reference counterpart."""
        if self._update_groups:
            self.flush_updates()
            for m in self._fused_modules:
                m._update_group = None
            self._update_groups = []
        if groups == "layer":
            by_prefix: dict[tuple, list[FusedLinear]] = {}
            for m in self._fused_modules:
                parts = self._fused_module_names[id(m)].split(".")
                idx = [i for i, p in enumerate(parts) if p.isdigit()]
                if not idx:
                    continue
                block = parts[: idx[-1]] + [str(int(parts[idx[-1]]) // max(1, layers_per_group))]
                key = (".".join(block), self._group_key(m), m.state_mode, m.weight.dtype)
                by_prefix.setdefault(key, []).append(m)
            groups = []
            for members in by_prefix.values():
                members = sorted(members, key=lambda m: -m.weight.numel())
                groups += [members[i:i + max_group] for i in range(0, len(members), max_group)]
        for members in groups:
            members = list(members)
            if len(members) < 2:
                continue
            if len(members) > 16:
                raise ValueError("a group holds at most 16 linears")
            first = members[0]
            for m in members:
                if not isinstance(m, FusedLinear) or id(m) not in self._fused_module_names:
                    raise ValueError("group members must be FusedLinear modules of this manager's model")
                if (m.optimizer_type, m.state_mode, m.weight.dtype, m.weight.device) != (
                        first.optimizer_type, first.state_mode, first.weight.dtype, first.weight.device):
                    raise ValueError("members of a group must share optimizer type, state mode, weight dtype and device")
            g = LayerUpdateGroup([m.weight for m in members])
            for m in members:
                m._update_group = g
            self._update_groups.append(g)
        return self

    def flush_updates(self):
        """Issue every recorded, not yet launched fused update (see ``group_updates``)."""
        for g in self._update_groups:
            g.flush()

    def optimizer_state_dict(self) -> dict:
        modules = {}
        for m in self._fused_modules:
            sd = m.get_optimizer_state_dict()
            if sd is not None:
                modules[self._fused_module_names[id(m)]] = sd
        return {"global_step": self._global_step, "micro_step": self._micro_step, "modules": modules}

    def load_optimizer_state_dict(self, state: dict):
        self._global_step = state["global_step"]
        self._micro_step = state["micro_step"]
        for m in self._fused_modules:
            sd = state["modules"].get(self._fused_module_names[id(m)])
            if sd is not None:
                m.load_optimizer_state_dict(sd)

    @property
    def l2_manager(self):
        return self._l2_manager

    @property
    def num_fused_params(self) -> int:
        return len(self._fused_param_ids)

    @property
    def num_fused_modules(self) -> int:
        return len(self._fused_modules)
