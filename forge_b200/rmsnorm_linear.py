"""``FusedRMSNormLinear``: a fused linear that folds the RMSNorm in front of it.

Mirror of the reference's prototype (``src/fused_grad_optimizer/fused_rmsnorm_linear.py``:
``FusedRMSNormLinearFunction`` :65-135, ``FusedRMSNormLinear`` :138-175, ``fuse_rmsnorm_linear_pairs``
:178-242): forward saves the PRE-norm hidden states and gamma instead of the norm's output; backward
recomputes the normalised activation right before the fused weight-gradient + optimizer update that
consumes it, then chains the input gradient through the norm.  Same constructor, same helper, same
branch table as ``FusedLinear``.

What is done differently here:

* the norm's forward (recompute) and backward are CUDA kernels behind the C ABI
  (``forge_rmsnorm_forward`` / ``forge_rmsnorm_backward``, bf16 activations) instead of ~10 elementwise
  torch kernels each; other dtypes use the reference's torch arithmetic;
* linears that share one norm (q / k / v; gate / up) share ONE recomputation and ONE norm backward per
  step: the siblings register with a ``SharedNorm``; in backward the first to arrive recomputes the
  normalised activation for all, every sibling adds its ``dY W`` to a common buffer, and the last one
  runs the norm's backward once on the sum (the reference recomputes and back-propagates the norm once
  per linear, three times for q / k / v);
* with ``FusedOptimizerManager.group_updates`` the siblings' updates go out as one kernel launch.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from forge_b200 import _lib
from forge_b200.autograd import _apply_fused, _apply_precomputed, _grad_input
from forge_b200.module import FusedLinear


# --------------------------------------------------------------------------------------------
# the norm itself
# --------------------------------------------------------------------------------------------
def _torch_rmsnorm_forward(x, gamma, eps):
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (gamma.float() * xf).to(x.dtype)


def _torch_rmsnorm_backward(x, gamma, g, eps):
    xf, gf, gm = x.float(), g.float(), gamma.float()
    H = xf.shape[-1]
    rrms = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    s = (gf * gm * xf).sum(-1, keepdim=True)
    dx = gf * gm * rrms - xf * s * rrms ** 3 / H
    dgamma = (gf * (xf * rrms)).reshape(-1, H).sum(0)
    return dx.to(x.dtype), dgamma.to(gamma.dtype)


def _native_ok(x, gamma):
    return (x.is_cuda and x.dtype == torch.bfloat16 and gamma.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.shape[-1] <= 16384 and gamma.is_contiguous())


def rmsnorm_forward(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """``bf16(gamma * (x * rsqrt(mean(x^2) + eps)))`` with fp32 arithmetic (``fused_rmsnorm_linear.py:32-41``)."""
    if not _native_ok(x, gamma):
        return _torch_rmsnorm_forward(x, gamma, eps)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    y = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().forge_rmsnorm_forward(x2.data_ptr(), gamma.data_ptr(), y.data_ptr(), x2.shape[0], x2.shape[1],
                                               x2.stride(0), y.stride(0), float(eps), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "forge_rmsnorm_forward")
    return y.view(x.shape)


def rmsnorm_backward(x: torch.Tensor, gamma: torch.Tensor, grad_y: torch.Tensor, eps: float):
    """Returns ``(grad_x, grad_gamma)`` (``fused_rmsnorm_linear.py:44-62``); ``grad_gamma`` in gamma's dtype."""
    if not (_native_ok(x, gamma) and grad_y.dtype == torch.bfloat16):
        return _torch_rmsnorm_backward(x, gamma, grad_y, eps)
    H = x.shape[-1]
    x2 = x.reshape(-1, H)
    g2 = grad_y.reshape(-1, H)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    if g2.stride(1) != 1:
        g2 = g2.contiguous()
    lib = _lib.load()
    dx = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    dgamma = torch.empty(H, dtype=gamma.dtype, device=x.device)
    scratch = torch.empty(lib.forge_rmsnorm_backward_scratch_bytes(x2.shape[0], H), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.forge_rmsnorm_backward(x2.data_ptr(), gamma.data_ptr(), g2.data_ptr(), dx.data_ptr(), dgamma.data_ptr(),
                                        _lib.dtype_id(gamma.dtype), 0, x2.shape[0], H, x2.stride(0), g2.stride(0),
                                        dx.stride(0), float(eps), scratch.data_ptr(), scratch.numel(),
                                        _lib.current_stream_ptr(x.device))
    _lib.check(rc, "forge_rmsnorm_backward")
    return dx.view(x.shape), dgamma


class SharedNorm:
    """One RMSNorm feeding several ``FusedRMSNormLinear`` modules.  Per forward pass it counts the
    consumers of each hidden-state tensor; in backward the first consumer recomputes the normalised
    activation, every consumer adds its partial input gradient, and the last one back-propagates the
    sum through the norm once."""

    def __init__(self, gamma: nn.Parameter, eps: float, consumers: int | None = None):
        self.gamma = gamma
        self.eps = eps
        self.consumers = consumers           # when known, the forward pass shares one normalisation too
        self._open: dict[tuple, dict] = {}
        self._fwd = None                     # (key, normalised activation, forwards still to come)

    @staticmethod
    def _key(hidden):
        return (hidden.data_ptr(), hidden._version, tuple(hidden.shape))

    def forward_normed(self, hidden):
        """The normalised activation for a forward pass; computed once for all siblings when their
        number is known, and dropped as soon as the last of them has taken it."""
        if not self.consumers or self.consumers < 2:
            return rmsnorm_forward(hidden, self.gamma, self.eps)
        key = self._key(hidden)
        if self._fwd is None or self._fwd[0] != key:
            self._fwd = [key, rmsnorm_forward(hidden, self.gamma, self.eps), self.consumers]
        y = self._fwd[1]
        self._fwd[2] -= 1
        if self._fwd[2] <= 0:
            self._fwd = None
        return y

    def register_forward(self, hidden):
        rec = self._open.setdefault(self._key(hidden), {"consumers": 0, "normed": None, "dnorm": None})
        rec["consumers"] += 1

    def normed(self, hidden):
        rec = self._open.get(self._key(hidden))
        if rec is None:                       # backward without a registered forward (e.g. double backward): no sharing
            return rmsnorm_forward(hidden, self.gamma, self.eps), None
        if rec["normed"] is None:
            rec["normed"] = rmsnorm_forward(hidden, self.gamma, self.eps)
        return rec["normed"], rec

    def finish(self, hidden, rec, dnorm):
        """Add this consumer's dY W; returns (grad_hidden, grad_gamma) from the last consumer, (None, None) before."""
        if rec is None:
            return rmsnorm_backward(hidden, self.gamma, dnorm, self.eps)
        rec["dnorm"] = dnorm if rec["dnorm"] is None else rec["dnorm"].add_(dnorm)
        rec["consumers"] -= 1
        if rec["consumers"] > 0:
            return None, None
        self._open.pop(self._key(hidden), None)
        return rmsnorm_backward(hidden, self.gamma, rec["dnorm"], self.eps)

    def reset(self):
        """Forget unfinished passes (a forward whose backward never ran)."""
        self._open.clear()
        self._fwd = None


class FusedRMSNormLinearFunction(torch.autograd.Function):
    """forward: ``linear(rmsnorm(h))`` saving ``h`` and gamma, not the norm's output; backward: the
    branch table of ``FusedLinearFunction`` on the recomputed activation, then the norm's backward."""

    @staticmethod
    def forward(ctx, hidden_states, gamma, eps, weight, bias, optimizer_state, optimizer_config, is_accumulating,
                l2_manager, use_fused_backward=True, shared=None, update_group=None):
        norm_output = (shared.forward_normed(hidden_states) if shared is not None
                       else rmsnorm_forward(hidden_states, gamma, eps))
        output = F.linear(norm_output, weight, bias)
        ctx.save_for_backward(hidden_states, gamma, weight, bias)
        ctx.eps = eps
        ctx.optimizer_state = optimizer_state
        ctx.optimizer_config = optimizer_config
        ctx.is_accumulating = is_accumulating
        ctx.l2_manager = l2_manager
        ctx.use_fused_backward = use_fused_backward
        ctx.shared = shared
        ctx.update_group = update_group
        if shared is not None and any(ctx.needs_input_grad):      # not under no_grad: a backward will come
            shared.register_forward(hidden_states)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        hidden_states, gamma, weight, bias = ctx.saved_tensors
        state, config, shared = ctx.optimizer_state, ctx.optimizer_config, ctx.shared
        # transient: recomputed here (once per group of siblings), never kept across the backward pass
        if shared is not None:
            norm_output, rec = shared.normed(hidden_states)
        else:
            norm_output, rec = rmsnorm_forward(hidden_states, gamma, ctx.eps), None
        grad_norm_output = _grad_input(grad_output, weight)       # before any in-place update of `weight`
        norm_2d = norm_output.reshape(-1, norm_output.shape[-1])
        dy2d = grad_output.reshape(-1, grad_output.shape[-1])
        grad_weight = None
        if config is None:
            grad_weight = dy2d.t() @ norm_2d
        elif ctx.is_accumulating:
            state.accumulate_grad(dy2d.t() @ norm_2d)
        else:
            pending = state.pop_accumulated_grad()
            if pending is not None:
                total = (dy2d.t() @ norm_2d).float()
                total.add_(pending)
                _apply_precomputed(total, weight, state, config)
            elif not ctx.use_fused_backward:
                _apply_precomputed((dy2d.t() @ norm_2d).float(), weight, state, config)
            elif ctx.update_group is not None:
                ctx.update_group.add(weight, lambda: _apply_fused(dy2d, norm_2d, weight, state, config, ctx.l2_manager))
            else:
                _apply_fused(dy2d, norm_2d, weight, state, config, ctx.l2_manager)
        grad_bias = dy2d.sum(0) if bias is not None else None
        if shared is not None:
            grad_hidden, grad_gamma = shared.finish(hidden_states, rec, grad_norm_output)
        else:
            grad_hidden, grad_gamma = rmsnorm_backward(hidden_states, gamma, grad_norm_output, ctx.eps)
        return grad_hidden, grad_gamma, None, grad_weight, grad_bias, None, None, None, None, None, None, None


class FusedRMSNormLinear(FusedLinear):
    """``FusedLinear`` that additionally applies the RMSNorm in front of it.  ``gamma`` stays owned by the
    original norm module (and by the user's optimizer); this class holds it by reference.  Found by
    ``FusedOptimizerManager`` like any ``FusedLinear``.  ``shared``: the ``SharedNorm`` of the siblings
    that consume the same normalised activation (optional)."""

    def __init__(self, linear: nn.Linear, gamma: nn.Parameter, eps: float, optimizer_type: str = "adamw",
                 state_mode: str = "bf16", shared: SharedNorm | None = None, **optimizer_kwargs):
        super().__init__(linear.in_features, linear.out_features, bias=linear.bias is not None,
                         optimizer_type=optimizer_type, state_mode=state_mode, _adopt=linear, **optimizer_kwargs)
        self._gamma_ref = [gamma]          # in a list: not registered a second time as this module's parameter
        self._eps = eps
        self._shared = shared

    @property
    def _gamma(self):
        return self._gamma_ref[0]

    def forward(self, hidden_states):
        if not self.training:
            return F.linear(rmsnorm_forward(hidden_states, self._gamma, self._eps), self.weight, self.bias)
        self._ensure_state()
        return FusedRMSNormLinearFunction.apply(hidden_states, self._gamma, self._eps, self.weight, self.bias, self._state,
                                                self._config, self._is_accumulating, self._l2_manager,
                                                self.use_fused_backward, self._shared, self._update_group)

    def extra_repr(self):
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}, shared_gamma=True, "
                f"eps={self._eps}, state_mode={self.state_mode}")


def fuse_rmsnorm_linear_pairs(model, optimizer_type: str = "adamw", state_mode: str = "bf16", **optimizer_kwargs):
    """Replace the (RMSNorm, consuming linears) pairs of a Llama-style model -- ``input_layernorm`` with
    q / k / v, ``post_attention_layernorm`` with gate / up -- by ``FusedRMSNormLinear`` modules that share a
    ``SharedNorm``; the norm modules' own forward becomes the identity.  Accepts ``nn.Linear`` or
    ``FusedLinear`` children.  Returns a callable that restores the original modules."""
    undo = []

    def _identity(self, x):
        return x

    for layer in model.model.layers:
        for norm, parent, names in ((layer.input_layernorm, layer.self_attn, ("q_proj", "k_proj", "v_proj")),
                                    (layer.post_attention_layernorm, layer.mlp, ("gate_proj", "up_proj"))):
            eps = getattr(norm, "variance_epsilon", getattr(norm, "eps", 1e-6))
            shared = SharedNorm(norm.weight, eps, consumers=sum(
                isinstance(getattr(parent, n, None), (nn.Linear, FusedLinear)) for n in names))
            undo.append(("norm_fwd", norm, norm.forward))
            norm.forward = _identity.__get__(norm, type(norm))
            for name in names:
                orig = getattr(parent, name)
                if isinstance(orig, FusedRMSNormLinear) or not isinstance(orig, (nn.Linear, FusedLinear)):
                    continue
                kw = dict(optimizer_kwargs)
                if isinstance(orig, FusedLinear):
                    kw = {**orig.optimizer_kwargs, **kw}
                fused = FusedRMSNormLinear(orig, norm.weight, eps, optimizer_type=optimizer_type, state_mode=state_mode,
                                           shared=shared, **kw)
                setattr(parent, name, fused)
                undo.append(("submod", parent, name, orig))

    def _restore():
        for entry in reversed(undo):
            if entry[0] == "norm_fwd":
                entry[1].forward = entry[2]
            else:
                setattr(entry[1], entry[2], entry[3])

    return _restore


__all__ = ["FusedRMSNormLinear", "FusedRMSNormLinearFunction", "SharedNorm", "fuse_rmsnorm_linear_pairs",
           "rmsnorm_forward", "rmsnorm_backward"]
