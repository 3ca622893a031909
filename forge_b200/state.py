"""Per-parameter optimizer state and the per-step hyper-parameter snapshot.

Host-side mirror of ``src/fused_grad_optimizer/state.py`` (``OptimizerConfig`` :10-30,
``FusedOptimizerState`` :33-205) with the same attribute names, lazy allocation and state-dict keys.
Differences, all additive:

* ``optimizer_type`` also accepts ``"sgdm"`` (SGD with momentum) and ``"lion"``; ``OptimizerConfig``
  carries ``momentum`` and ``nesterov``.
* ``state_mode="fp8_block"``: e4m3 codes for both moments with one fp32 absmax scale per
  (row, 64 columns) -- the int8 layout with a different code book.
* ``state_mode="fp8"`` keeps the reference layout (e4m3 m, e5m2 v, one scale per tensor, delayed
  scaling) but the scale promotion runs on the device (no ``float(tensor)`` host syncs) and the
  next-step absmax is produced by the update kernel, so the per-tile scratch arrays are gone.
* ``state_dict`` / ``load_state_dict`` cover every mode (the reference drops fp8 state).
"""

from __future__ import annotations

from typing import Optional

import torch

_ADAM_LIKE = ("adamw",)
_ONE_MOMENT = ("sgdm", "lion")
_STATELESS = ("sgd",)
OPTIMIZER_TYPES = _ADAM_LIKE + _ONE_MOMENT + _STATELESS
STATE_MODES = ("bf16", "int8", "fp8", "fp8_block")


class OptimizerConfig:
    """Hyper-parameters of one step; build a fresh one per step so schedulers act naturally.
    Unknown keyword arguments are ignored, as in the reference (``state.py:23-24``)."""

    __slots__ = ("optimizer_type", "lr", "beta1", "beta2", "eps", "weight_decay", "momentum", "nesterov",
                 "hyper_device")

    def __init__(self, optimizer_type="adamw", lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8,
                 weight_decay=0.01, momentum=0.0, nesterov=False, hyper_device=None, **_ignored):
        self.optimizer_type = optimizer_type
        self.lr = lr
        self.beta1 = beta1
        self.beta2 = beta2
        self.eps = eps
        self.weight_decay = weight_decay
        self.momentum = momentum
        self.nesterov = nesterov
        # optional forge_b200.kernel.DeviceHyper: the fused kernels then read lr / betas / step from
        # device memory (CUDA-graph replay); the scalar fields above are ignored by them
        self.hyper_device = hyper_device

    def __repr__(self):
        return ("OptimizerConfig(" + ", ".join(f"{k}={getattr(self, k)!r}" for k in self.__slots__) + ")")

    def __eq__(self, other):
        return isinstance(other, OptimizerConfig) and all(
            getattr(self, k) == getattr(other, k) for k in self.__slots__)


class FusedOptimizerState:
    """Moment buffers of one (V, H) weight, allocated on first use next to the weight.

    Layouts (``state.py:95-130`` of the reference):
      bf16 mode   ``m``, ``v``: (V, H) in ``state_dtype`` (default: the weight's dtype)
      int8 mode   ``m_q``, ``v_q``: (V, H) int8; ``m_scale``, ``v_scale``: (V, H // qblock) fp32,
                  initial codes 0 and scales 1
      fp8 mode    ``m_fp8`` e4m3fn, ``v_fp8`` e5m2: (V, H); scalars ``m_scale``, ``v_scale`` (init 1)
                  and ``m_absmax_next``, ``v_absmax_next`` (init 0)
      fp8_block   ``m_q``, ``v_q``: (V, H) e4m3fn; scales as in int8 mode
    One-moment optimizers (``sgdm``, ``lion``) only allocate ``m``; plain ``sgd`` allocates nothing.
    """

    def __init__(self, weight: torch.Tensor, optimizer_type: str = "adamw",
                 state_dtype: Optional[torch.dtype] = None, quantize_state: bool = False,
                 qblock_size: int = 64, state_mode: Optional[str] = None):
        if optimizer_type not in OPTIMIZER_TYPES:
            raise ValueError(f"Unknown optimizer: {optimizer_type}. Use one of {OPTIMIZER_TYPES}.")
        if state_mode is None:
            state_mode = "int8" if quantize_state else "bf16"
        if state_mode not in STATE_MODES:
            raise ValueError(f"Unknown state_mode: {state_mode}")
        if optimizer_type not in _ADAM_LIKE and state_mode != "bf16":
            raise ValueError(f"state_mode={state_mode!r} is only available for adamw")
        self.optimizer_type = optimizer_type
        self.state_mode = state_mode
        self.quantize_state = state_mode == "int8"
        self.qblock_size = qblock_size
        self._step = 0
        self._native = None      # C++ autograd node's handle, which then owns the step count (see module.py)
        self._version = 0        # bumped whenever a buffer is (re)allocated or replaced
        self._weight_ref = weight
        self._state_dtype = state_dtype if state_dtype is not None else weight.dtype
        self._pending_grad: Optional[torch.Tensor] = None
        for name in self._buffer_names():
            setattr(self, name, None)

    @property
    def step(self) -> int:
        """Per-parameter count of updates (``state.py:159-160`` of the reference)."""
        return self._native.step if self._native is not None else self._step

    @step.setter
    def step(self, value: int):
        self._step = int(value)
        if self._native is not None:
            self._native.step = int(value)

    # ------------------------------------------------------------------ layout
    def _buffer_names(self):
        if self.optimizer_type in _STATELESS:
            return ()
        if self.optimizer_type in _ONE_MOMENT:
            return ("m",)
        return {
            "bf16": ("m", "v"),
            "int8": ("m_q", "v_q", "m_scale", "v_scale"),
            "fp8_block": ("m_q", "v_q", "m_scale", "v_scale"),
            "fp8": ("m_fp8", "v_fp8", "m_scale", "v_scale", "m_absmax_next", "v_absmax_next"),
        }[self.state_mode]

    def ensure_buffers(self):
        """Allocate the moments on first use (called right before the first update)."""
        names = self._buffer_names()
        if not names or getattr(self, names[0]) is not None:
            return
        w = self._weight_ref
        V, H = w.shape
        dev = w.device
        self._version += 1
        if self.optimizer_type in _ONE_MOMENT:
            self.m = torch.zeros(V, H, dtype=self._state_dtype, device=dev)
        elif self.state_mode == "bf16":
            self.m = torch.zeros(V, H, dtype=self._state_dtype, device=dev)
            self.v = torch.zeros(V, H, dtype=self._state_dtype, device=dev)
        elif self.state_mode in ("int8", "fp8_block"):
            if H % self.qblock_size != 0:
                raise ValueError(f"H ({H}) must be divisible by qblock ({self.qblock_size})")
            code = torch.int8 if self.state_mode == "int8" else torch.float8_e4m3fn
            self.m_q = torch.zeros(V, H, dtype=code, device=dev)
            self.v_q = torch.zeros(V, H, dtype=code, device=dev)
            self.m_scale = torch.ones(V, H // self.qblock_size, dtype=torch.float32, device=dev)
            self.v_scale = torch.ones(V, H // self.qblock_size, dtype=torch.float32, device=dev)
        else:  # fp8 per tensor
            self.m_fp8 = torch.zeros(V, H, dtype=torch.float8_e4m3fn, device=dev)
            self.v_fp8 = torch.zeros(V, H, dtype=torch.float8_e5m2, device=dev)
            self.m_scale = torch.ones((), dtype=torch.float32, device=dev)
            self.v_scale = torch.ones((), dtype=torch.float32, device=dev)
            self.m_absmax_next = torch.zeros((), dtype=torch.float32, device=dev)
            self.v_absmax_next = torch.zeros((), dtype=torch.float32, device=dev)

    def state_nbytes(self) -> int:
        """Bytes currently held by the moment and scale buffers."""
        return sum(t.nbytes for t in (getattr(self, n) for n in self._buffer_names()) if t is not None)

    # ------------------------------------------------------------------ stepping
    def increment_step(self):
        self.step += 1

    def pre_step_fp8(self):
        """fp8 mode: promote last step's absmax to this step's scale (capped at 2x the previous
        scale) and reset the accumulator.  Runs as one tiny kernel; no host synchronisation."""
        if self.state_mode != "fp8" or self.m_fp8 is None:
            return
        from forge_b200.kernel import fp8_prestep
        fp8_prestep(self.m_scale, self.v_scale, self.m_absmax_next, self.v_absmax_next)

    # ------------------------------------------------------------------ gradient accumulation
    def accumulate_grad(self, grad: torch.Tensor):
        g = grad.detach().float()
        if self._pending_grad is None:
            self._pending_grad = g.clone()
        else:
            self._pending_grad.add_(g)

    def pop_accumulated_grad(self) -> Optional[torch.Tensor]:
        g, self._pending_grad = self._pending_grad, None
        return g

    def has_accumulated_grad(self) -> bool:
        return self._pending_grad is not None

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        d = {"optimizer_type": self.optimizer_type, "step": self.step,
             "quantize_state": self.quantize_state, "state_mode": self.state_mode}
        for name in self._buffer_names():
            t = getattr(self, name)
            if t is not None:
                d[name] = t.clone()
        return d

    def load_state_dict(self, d: dict):
        mode = d.get("state_mode", "int8" if d.get("quantize_state") else "bf16")
        if mode != self.state_mode:
            has_buffers = any(n in d for n in ("m", "m_q", "m_fp8"))
            if has_buffers:
                raise ValueError(f"checkpoint holds {mode!r} state but this parameter uses {self.state_mode!r}")
        self.step = d["step"]
        self._version += 1
        for name in self._buffer_names():
            if name in d:
                setattr(self, name, d[name].clone().to(self._weight_ref.device))
