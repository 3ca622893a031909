"""Autograd boundary: a linear whose backward updates its own weight.

Mirror of ``src/fused_grad_optimizer/autograd.py`` (``FusedLinearFunction`` :26-91, ``_apply_fused``
:94-144, ``_apply_precomputed`` :147-178) with the same argument list and branch table:

    forward   Y = X W^T (+ b)
    backward  dX = dY W                       enqueued first: it must read the pre-update W
              then, by case --
                no config            -> return dW = dY^T X like a plain linear
                accumulating         -> add dW to the fp32 pending buffer
                pending accumulation -> dW + pending, optimizer-only kernel
                use_fused_backward=False -> materialise dW, optimizer-only kernel
                otherwise            -> fused wgrad + optimizer kernel, dW never exists
              weight.grad stays None; the bias gradient is returned to autograd.

All optimizer work goes through the C ABI (``forge_b200.kernel``); there is no PyTorch fallback.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from forge_b200 import kernel as K
from forge_b200.state import FusedOptimizerState, OptimizerConfig  # noqa: F401  (re-exported)

# dX through the library's own GEMM (bf16 CUDA operands); plain `grad_output @ weight` otherwise
use_forge_dgrad = False


def _grad_input(grad_output: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if (use_forge_dgrad and grad_output.is_cuda and grad_output.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16 and weight.stride(1) == 1):
        go2d = grad_output.reshape(-1, grad_output.shape[-1])
        if not go2d.is_contiguous():
            go2d = go2d.contiguous()
        return K.dgrad(go2d, weight).reshape(*grad_output.shape[:-1], weight.shape[1])
    return grad_output @ weight


class FusedLinearFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, input, weight, bias, optimizer_state, optimizer_config, is_accumulating,
                l2_manager, use_fused_backward=True, update_group=None):
        # update_group (no reference counterpart): a LayerUpdateGroup that collects the fused updates of
        # several linears and issues them as one launch once every member has reported
        ctx.update_group = update_group
        ctx.save_for_backward(input, weight, bias)
        ctx.optimizer_state = optimizer_state
        ctx.optimizer_config = optimizer_config
        ctx.is_accumulating = is_accumulating
        ctx.l2_manager = l2_manager
        ctx.use_fused_backward = use_fused_backward
        return F.linear(input, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        input, weight, bias = ctx.saved_tensors
        state, config = ctx.optimizer_state, ctx.optimizer_config

        # before any in-place update of `weight` on this stream
        grad_input = _grad_input(grad_output, weight) if ctx.needs_input_grad[0] else None

        x2d = input.reshape(-1, input.shape[-1])
        dy2d = grad_output.reshape(-1, grad_output.shape[-1])
        grad_weight = None
        if config is None:
            grad_weight = dy2d.t() @ x2d
        elif ctx.is_accumulating:
            state.accumulate_grad(dy2d.t() @ x2d)
        else:
            pending = state.pop_accumulated_grad()
            if pending is not None:
                total = (dy2d.t() @ x2d).float()
                total.add_(pending)
                _apply_precomputed(total, weight, state, config)
            elif not ctx.use_fused_backward:
                _apply_precomputed((dy2d.t() @ x2d).float(), weight, state, config)
            elif ctx.update_group is not None:
                ctx.update_group.add(weight, lambda: _apply_fused(dy2d, x2d, weight, state, config, ctx.l2_manager))
            else:
                _apply_fused(dy2d, x2d, weight, state, config, ctx.l2_manager)

        grad_bias = dy2d.sum(0) if bias is not None else None
        return grad_input, grad_weight, grad_bias, None, None, None, None, None, None


def native_proto(weight, state):
    """The argument block of one weight's fused update with everything that stays the same from step
    to step filled in (W, moments, scales, dtypes, optimizer), for the C++ autograd node."""
    from forge_b200 import _lib
    w = weight.data
    K._require_cuda(w)
    K._row_major_2d(w, "weight")
    opt = state.optimizer_type
    if opt == "sgd":
        st = K._state()
    elif opt in ("sgdm", "lion"):
        st = K._moment_state(state.m)
    elif state.state_mode == "int8":
        st = K._int8_state(w, state.m_q, state.v_q, state.m_scale, state.v_scale, state.qblock_size)
    elif state.state_mode == "fp8_block":
        st = K._int8_state(w, state.m_q, state.v_q, state.m_scale, state.v_scale, state.qblock_size, mode=_lib.ST_FP8_BLOCK)
    elif state.state_mode == "fp8":
        st = K._fp8_tensor_state(state)
    else:
        st = K._moment_state(state.m, state.v)
    a = _lib.ForgeWgradArgs()
    a.W = w.data_ptr()
    a.V, a.H = w.shape
    a.ld_w = w.stride(0)
    a.operand_dtype = _lib.DT_BF16
    a.w_dtype = _lib.dtype_id(w.dtype)
    a.optimizer = _lib.OPTIMIZER_IDS[opt]
    a.flags = 0
    a.state = st
    a.status = _lib.status_word(w.device).data_ptr()
    return a


class LayerUpdateGroup:
    """The fused updates of a fixed set of linears (the projections of a decoder layer, or q / k / v)
    issued as one launch.  Each member's backward records its update instead of launching it; when the
    last member has reported, the group enqueues ``forge_wgrad_update_group`` on the current stream.
    Deferring is safe because a weight is read by nothing between its own backward and the end of the
    layer's backward: every dX GEMM of the members has been enqueued, on the same stream, before the
    launch that rewrites the weights.  ``flush()`` issues whatever has been recorded (a member that
    took no part in this backward pass would otherwise hold the others back);
    ``FusedOptimizerManager.pre_step`` calls it.  No reference counterpart."""

    def __init__(self, weights):
        self._members = {w.data_ptr() for w in weights}
        self._seen: set[int] = set()
        self._group = K.UpdateGroup()
        # With the C++ autograd node built, ITS group object is the one that counts the members and
        # launches: members whose backward runs in Python hand their recorded update to it, so a
        # layer whose linears are split between the two paths still goes out as one launch, inside
        # the backward pass (and therefore inside a captured graph of it).
        from forge_b200 import native
        nat = native.module()
        self.native = None
        self._keep: list = []
        if nat is not None:
            self.native = nat.Group()
            self.native.set_members(sorted(self._members))

    def __len__(self):
        return len(self._members)

    def add(self, weight, launch):
        wid = weight.data_ptr()
        if self.native is not None:
            with self._group.record():
                launch()
            blocks, keep, device = self._group.take()
            if self.native.pending() == 0:
                self._keep.clear()     # everything recorded before has been enqueued
            self._keep.extend(keep)
            for a in blocks:           # the native group flushes itself on a repeated or on the last member
                self.native.add_recorded(bytes(a), torch.device(device).index)
            if self.native.pending() == 0:
                self._keep.clear()
            return
        if wid in self._seen:          # the same linear twice in one pass: issue what is there first
            self.flush()
        with self._group.record():
            launch()
        self._seen.add(wid)
        if self._seen >= self._members:
            self.flush()

    def pending(self) -> int:
        """Updates recorded and not yet enqueued."""
        return len(self._group) + (self.native.pending() if self.native is not None else 0)

    def flush(self):
        self._seen.clear()
        self._group.flush()
        if self.native is not None:
            self.native.flush()
        self._keep.clear()


def _begin_update(state, config):
    if config.optimizer_type != state.optimizer_type:
        raise ValueError(f"config asks for {config.optimizer_type!r} but the state was built for "
                         f"{state.optimizer_type!r}")
    state.ensure_buffers()
    state.increment_step()


def _apply_fused(grad_output_2d, input_2d, weight, state, config, l2_manager=None):
    """Tile-wise fused gradient + optimizer; ``grad_W`` never exists in memory."""
    _begin_update(state, config)
    go = grad_output_2d if grad_output_2d.is_contiguous() else grad_output_2d.contiguous()
    inp = input_2d if input_2d.is_contiguous() else input_2d.contiguous()
    w = weight.data
    opt = config.optimizer_type
    hd = getattr(config, "hyper_device", None)
    if opt == "sgd":
        K.fused_grad_sgd(go, inp, w, lr=config.lr, weight_decay=config.weight_decay, hyper_device=hd)
    elif opt == "sgdm":
        K.fused_grad_sgd_momentum(go, inp, w, state.m, lr=config.lr, momentum=config.momentum,
                                  weight_decay=config.weight_decay, nesterov=config.nesterov, hyper_device=hd)
    elif opt == "lion":
        K.fused_grad_lion(go, inp, w, state.m, lr=config.lr, beta1=config.beta1, beta2=config.beta2,
                          weight_decay=config.weight_decay, hyper_device=hd)
    elif opt == "adamw":
        kw = dict(lr=config.lr, beta1=config.beta1, beta2=config.beta2, eps=config.eps,
                  weight_decay=config.weight_decay, step=state.step, hyper_device=hd)
        if state.state_mode == "int8":
            K.fused_grad_adamw_int8state(go, inp, w, state.m_q, state.v_q, state.m_scale, state.v_scale,
                                         qblock=state.qblock_size, **kw)
        elif state.state_mode == "fp8_block":
            K.fused_grad_adamw_fp8block(go, inp, w, state.m_q, state.v_q, state.m_scale, state.v_scale,
                                        qblock=state.qblock_size, **kw)
        elif state.state_mode == "fp8":
            state.pre_step_fp8()
            K.fused_grad_adamw_fp8state(go, inp, w, state, **kw)
        else:
            K.fused_grad_adamw(go, inp, w, state.m, state.v, **kw)
    else:
        raise ValueError(f"Unknown optimizer: {opt}")


def _apply_precomputed(grad_weight, weight, state, config):
    """Optimizer on a materialised gradient (gradient accumulation, non-fused layers)."""
    _begin_update(state, config)
    g = grad_weight if grad_weight.is_contiguous() else grad_weight.contiguous()
    w = weight.data
    opt = config.optimizer_type
    if opt == "sgd":
        K.optimizer_only_sgd(g, w, lr=config.lr, weight_decay=config.weight_decay)
    elif opt == "sgdm":
        K.optimizer_only_sgd_momentum(g, w, state.m, lr=config.lr, momentum=config.momentum,
                                      weight_decay=config.weight_decay, nesterov=config.nesterov)
    elif opt == "lion":
        K.optimizer_only_lion(g, w, state.m, lr=config.lr, beta1=config.beta1, beta2=config.beta2,
                              weight_decay=config.weight_decay)
    elif opt == "adamw":
        kw = dict(lr=config.lr, beta1=config.beta1, beta2=config.beta2, eps=config.eps,
                  weight_decay=config.weight_decay, step=state.step)
        if state.state_mode == "int8":
            K.optimizer_only_adamw_int8state(g, w, state.m_q, state.v_q, state.m_scale, state.v_scale,
                                             qblock=state.qblock_size, **kw)
        elif state.state_mode == "fp8_block":
            K.optimizer_only_adamw_fp8block(g, w, state.m_q, state.v_q, state.m_scale, state.v_scale,
                                            qblock=state.qblock_size, **kw)
        elif state.state_mode == "fp8":
            state.pre_step_fp8()
            K.optimizer_only_adamw_fp8state(g, w, state, **kw)
        else:
            K.optimizer_only_adamw(g, w, state.m, state.v, **kw)
    else:
        raise ValueError(f"Unknown optimizer: {opt}")
