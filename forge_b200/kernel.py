"""Operator wrappers with the reference's signatures, marshalling tensors into the C ABI.

Mirrors ``src/fused_grad_optimizer/kernel.py:1319-1575`` (``fused_grad_sgd``, ``fused_grad_adamw``,
``optimizer_only_adamw``, ``fused_grad_adamw_int8state``, ``optimizer_only_adamw_int8state``) and
``src/fused_grad_optimizer/kernel_fp8_state.py:343-392`` (``fused_grad_adamw_fp8state``).  Shapes:
``grad_output`` (BT, V), ``input`` (BT, H), ``weight`` and moments (V, H).  Every function updates
its tensors in place on the current CUDA stream, returns ``None`` and never materialises ``grad_W``.

Additions with no reference counterpart: SGD with momentum, Lion, e4m3 moments with per-block scales.
"""

from __future__ import annotations

import ctypes
import threading

import torch

from forge_b200 import _lib
from forge_b200._lib import (
    ForgeHyper, ForgeOptimArgs, ForgeState, ForgeWgradArgs,
    OPT_ADAMW, OPT_LION, OPT_SGD, OPT_SGDM,
    ST_FP8_BLOCK, ST_FP8_TENSOR, ST_INT8, ST_NONE,
)

FP8_E4M3_MAX = 448.0
FP8_E5M2_MAX = 57344.0

# Scratch for fp32 operands (the library itself allocates nothing on this path): one growing buffer per
# (device, stream).  Updates on different streams may overlap on the GPU, so they must not share the
# split area; on one stream launches are ordered, and the caching allocator only hands a dropped
# buffer's memory to later work of the stream that allocated it.
_scratch: dict[tuple, torch.Tensor] = {}


def _get_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def _require_cuda(*tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.ForgeLibraryError(
                "forge_b200 operators run on CUDA tensors only (sm_100a); there is no CPU path")


def _row_major_2d(t: torch.Tensor, what: str):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{what} must be 2-D with a contiguous last dimension (got strides {tuple(t.stride())})")


def _hyper(lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, momentum=0.0, nesterov=False):
    return ForgeHyper(float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
                      float(momentum), int(bool(nesterov)), int(step))


def _state(mode=ST_NONE, m=None, v=None, m_scale=None, v_scale=None, m_absmax=None, v_absmax=None, qblock=64):
    st = ForgeState()
    st.mode = mode
    st.qblock = qblock
    st.m = m.data_ptr() if m is not None else None
    st.v = v.data_ptr() if v is not None else None
    st.ld_state = m.stride(0) if m is not None else 0
    st.m_scale = m_scale.data_ptr() if m_scale is not None else None
    st.v_scale = v_scale.data_ptr() if v_scale is not None else None
    st.ld_scale = m_scale.stride(0) if (m_scale is not None and m_scale.dim() == 2) else 0
    st.m_absmax_next = m_absmax.data_ptr() if m_absmax is not None else None
    st.v_absmax_next = v_absmax.data_ptr() if v_absmax is not None else None
    return st


# Marshalled argument blocks are cached per weight: W / moment pointers, shapes and dtypes do not change
# between steps, so a call only refreshes the activation pointers, the token count, the hyper-parameters
# and the stream.  (225 launches per Llama-8B step: the per-call host cost matters once the GPU time per
# launch drops below ~50 us, e.g. in the row-sharded mode.)
_wgrad_cache: dict[tuple, ForgeWgradArgs] = {}
_WGRAD_CACHE_MAX = 4096


class DeviceHyper:
    """Hyper-parameters kept in device memory so that captured CUDA graphs can be replayed with a
    new lr / step: ``update(...)`` packs them on the host (same narrowing as the direct path) and
    enqueues one 64-byte copy on the current stream; pass the object as ``hyper_device=`` to the
    fused operators.  The pinned staging area is a ring of ``RING`` slots; an event recorded after
    each copy guards its slot, and ``update`` waits for that event before it rewrites the slot, so a
    host that runs many steps ahead of the GPU never overwrites bytes a queued copy has not read."""

    NBYTES = 64
    RING = 16

    def __init__(self, device):
        self.host = torch.zeros(self.RING, self.NBYTES, dtype=torch.uint8).pin_memory()
        self.dev = torch.zeros(self.NBYTES, dtype=torch.uint8, device=device)
        self._copied = [None] * self.RING     # event after the last copy that read each slot
        self._n = 0

    def update(self, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, momentum=0.0, nesterov=False):
        h = _hyper(lr, beta1, beta2, eps, weight_decay, step, momentum, nesterov)
        i = self._n % self.RING
        self._n += 1
        capturing = torch.cuda.is_current_stream_capturing()
        ev = self._copied[i]
        if ev is not None and not capturing:
            ev.synchronize()                  # the copy that last read this slot has run
        slot = self.host[i]
        _lib.check(_lib.load().forge_hyper_pack(ctypes.byref(h), slot.data_ptr()), "forge_hyper_pack")
        with torch.cuda.device(self.dev.device):
            self.dev.copy_(slot, non_blocking=True)
            if not capturing:
                if ev is None:
                    ev = self._copied[i] = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(self.dev.device))
        return self

    def data_ptr(self):
        return self.dev.data_ptr()


class UpdateGroup:
    """Fused updates of several weights issued together (``forge_wgrad_update_group``): consecutive
    entries of one kernel configuration share a launch, sixteen at most, so the fixed start-up and the
    ragged end of a launch are paid once per group.  No reference counterpart: the reference launches
    one kernel per linear (``autograd.py:94-144``).

        with UpdateGroup() as g:                       # calls inside are recorded, not launched
            fused_grad_adamw(dy_q, x, w_q, m_q, v_q, lr=lr, step=t)
            fused_grad_adamw(dy_k, x, w_k, m_k, v_k, lr=lr, step=t)
        # leaving the block enqueues one launch on the current stream

    ``record()`` / ``flush()`` give the same in two steps for callers (the autograd function of
    ``FusedLinear``) that collect entries over several backward nodes.  The group keeps the recorded
    activations alive until ``flush`` has enqueued the launch.  Each weight's result is bit-identical
    to its own single launch.  Put the largest weights first: work units follow the recorded order.
    """

    def __init__(self):
        self._args: list[ForgeWgradArgs] = []
        self._keep: list = []
        self._device = None

    def __len__(self):
        return len(self._args)

    def record(self):
        """Context manager: fused_grad_* calls made by this thread inside it are added to the group."""
        return _Recording(self)

    def __enter__(self):
        self._rec = _Recording(self)
        self._rec.__enter__()
        return self

    def __exit__(self, exc_type, exc, tb):
        self._rec.__exit__(exc_type, exc, tb)
        if exc_type is None:
            self.flush()
        else:
            self.clear()
        return False

    def _add(self, a: ForgeWgradArgs, device, keep):
        if self._device is not None and device != self._device:
            raise ValueError("an UpdateGroup holds weights of one device")
        self._device = device
        c = ForgeWgradArgs()
        ctypes.memmove(ctypes.byref(c), ctypes.byref(a), ctypes.sizeof(ForgeWgradArgs))
        self._args.append(c)
        self._keep.append(keep)

    def clear(self):
        self._args.clear()
        self._keep.clear()
        self._device = None

    def take(self):
        """Hand the recorded entries to the caller: ``(argument blocks, kept tensors, device)``; the
        group is empty afterwards and the caller answers for the launch."""
        out = (list(self._args), list(self._keep), self._device)
        self.clear()
        return out

    def flush(self):
        """Enqueue the recorded updates on the current stream of their device and forget them."""
        n = len(self._args)
        if n == 0:
            return
        arr = (ForgeWgradArgs * n)(*self._args)
        dev = self._device
        lib = _lib.load()
        try:
            with torch.cuda.device(dev):
                rc = lib.forge_wgrad_update_group(arr, n, _lib.current_stream_ptr(dev))
        finally:
            self.clear()
        if rc:
            _lib.check(rc, "forge_wgrad_update_group")


_recording = threading.local()


class _Recording:
    def __init__(self, group):
        self.group = group

    def __enter__(self):
        self.prev = getattr(_recording, "group", None)
        _recording.group = self.group
        return self.group

    def __exit__(self, *exc):
        _recording.group = self.prev
        return False


def _wgrad(grad_output, input, weight, optimizer, state, hyper, hyper_device=None):
    if not (grad_output.is_cuda and input.is_cuda and weight.is_cuda):
        _require_cuda(grad_output, input, weight)
    if not (grad_output.is_contiguous() and input.is_contiguous()):
        # AssertionError as in the reference (kernel.py:1363), raised explicitly so that it survives `python -O`
        raise AssertionError("grad_output and input must be contiguous (row pitches V and H)")
    BT, V = grad_output.shape
    H = input.shape[1]
    odt = grad_output.dtype
    key = (weight.data_ptr(), state.m, state.v, state.m_scale, optimizer, state.mode, V, H, weight.stride(0),
           weight.dtype, odt)
    a = _wgrad_cache.get(key)
    lib = _lib.load()
    if a is None:
        _row_major_2d(weight, "weight")
        if input.shape[0] != BT or tuple(weight.shape) != (V, H):
            raise ValueError(f"shape mismatch: grad_output {tuple(grad_output.shape)}, input {tuple(input.shape)}, "
                             f"weight {tuple(weight.shape)}")
        if odt != input.dtype:
            raise ValueError("grad_output and input must have the same dtype")
        a = ForgeWgradArgs()
        a.W = weight.data_ptr()
        a.V, a.H = V, H
        a.ld_dy, a.ld_x, a.ld_w = V, H, weight.stride(0)
        a.operand_dtype = _lib.dtype_id(odt)
        a.w_dtype = _lib.dtype_id(weight.dtype)
        a.optimizer = optimizer
        a.flags = 0
        a.status = _lib.status_word(weight.device).data_ptr()
        if len(_wgrad_cache) >= _WGRAD_CACHE_MAX:
            _wgrad_cache.clear()
        _wgrad_cache[key] = a
    elif input.shape[0] != BT or weight.shape[0] != V or weight.shape[1] != H or input.dtype != odt:
        raise ValueError(f"shape mismatch: grad_output {tuple(grad_output.shape)}, input {tuple(input.shape)}, "
                         f"weight {tuple(weight.shape)}")
    a.dY, a.X, a.BT = grad_output.data_ptr(), input.data_ptr(), BT
    a.state = state
    a.hyper = hyper
    a.hyper_device = hyper_device.data_ptr() if hyper_device is not None else None
    group = getattr(_recording, "group", None)
    scratch = None
    if odt != torch.bfloat16:
        nbytes = lib.forge_wgrad_scratch_bytes(BT, V, H, a.operand_dtype)
        # a recorded entry keeps a split area of its own until the group's launch has been enqueued
        scratch = (torch.empty(nbytes, dtype=torch.uint8, device=weight.device) if group is not None
                   else _get_scratch(weight.device, nbytes))
        a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    dev = weight.device
    if group is not None:
        group._add(a, dev, (grad_output, input, weight, scratch, hyper_device))
        return
    if dev.index == torch.cuda.current_device():
        rc = lib.forge_wgrad_update(ctypes.byref(a), torch.cuda.current_stream().cuda_stream)
    else:
        with torch.cuda.device(dev):
            rc = lib.forge_wgrad_update(ctypes.byref(a), _lib.current_stream_ptr(dev))
    if rc:
        _lib.check(rc, "forge_wgrad_update")


def _optim(grad, weight, optimizer, state, hyper):
    _require_cuda(grad, weight)
    if not grad.is_contiguous():
        raise AssertionError("grad must be contiguous")
    _row_major_2d(weight, "weight")
    V, H = weight.shape
    if tuple(grad.shape) != (V, H):
        raise ValueError(f"grad shape {tuple(grad.shape)} does not match weight {tuple(weight.shape)}")
    lib = _lib.load()
    a = ForgeOptimArgs()
    a.grad, a.W = grad.data_ptr(), weight.data_ptr()
    a.V, a.H = V, H
    a.ld_grad, a.ld_w = grad.stride(0), weight.stride(0)
    a.grad_dtype = _lib.dtype_id(grad.dtype)
    a.w_dtype = _lib.dtype_id(weight.dtype)
    a.optimizer = optimizer
    a.flags = 0
    a.state = state
    a.hyper = hyper
    with torch.cuda.device(weight.device):
        rc = lib.forge_optimizer_update(ctypes.byref(a), _lib.current_stream_ptr(weight.device))
    _lib.check(rc, "forge_optimizer_update")


def _moment_state(m, v=None):
    if m.dtype != (v.dtype if v is not None else m.dtype):
        raise ValueError("m and v must share a dtype")
    _row_major_2d(m, "m")
    if v is not None:
        _row_major_2d(v, "v")
        if v.stride(0) != m.stride(0):
            raise ValueError("m and v must share a row pitch")
    return _state(_lib.state_mode_id(m.dtype), m, v)


# --------------------------------------------------------------------------------------------
# reference signatures
# --------------------------------------------------------------------------------------------
def fused_grad_sgd(grad_output, input, weight, lr: float = 1e-3, weight_decay: float = 0.0, hyper_device=None):
    """Fused weight gradient + SGD update (``kernel.py:1319-1339``): ``W = W(1 - lr wd) - lr dW``."""
    _wgrad(grad_output, input, weight, OPT_SGD, _state(), _hyper(lr, weight_decay=weight_decay), hyper_device)


def fused_grad_adamw(grad_output, input, weight, m, v, lr: float = 1e-4, beta1: float = 0.9,
                     beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01, step: int = 1,
                     hyper_device: "DeviceHyper | None" = None):
    """Fused weight gradient + AdamW update (``kernel.py:1342-1455``); m, v bf16 or fp32, in place.
    ``hyper_device`` (no reference counterpart): read the hyper-parameters from a ``DeviceHyper`` block
    at run time instead of the keyword values, for replay inside a captured CUDA graph."""
    _require_cuda(m, v)
    _wgrad(grad_output, input, weight, OPT_ADAMW, _moment_state(m, v),
           _hyper(lr, beta1, beta2, eps, weight_decay, step), hyper_device)


def optimizer_only_adamw(grad, weight, m, v, lr: float = 1e-4, beta1: float = 0.9, beta2: float = 0.999,
                         eps: float = 1e-8, weight_decay: float = 0.01, step: int = 1):
    """AdamW on a pre-computed gradient (``kernel.py:1458-1484``)."""
    _require_cuda(m, v)
    _optim(grad, weight, OPT_ADAMW, _moment_state(m, v), _hyper(lr, beta1, beta2, eps, weight_decay, step))


def _int8_state(weight, m_q, v_q, m_scale, v_scale, qblock, mode=ST_INT8):
    H = weight.shape[1]
    if H % qblock != 0:
        raise AssertionError(f"H ({H}) must be divisible by qblock ({qblock})")   # kernel.py:1513
    _require_cuda(m_q, v_q, m_scale, v_scale)
    _row_major_2d(m_q, "m_q")
    _row_major_2d(v_q, "v_q")
    _row_major_2d(m_scale, "m_scale")
    _row_major_2d(v_scale, "v_scale")
    if m_q.stride(0) != v_q.stride(0) or m_scale.stride(0) != v_scale.stride(0):
        raise ValueError("m_q/v_q and m_scale/v_scale must share row pitches")
    return _state(mode, m_q, v_q, m_scale, v_scale, qblock=qblock)


def fused_grad_adamw_int8state(grad_output, input, weight, m_q, v_q, m_scale, v_scale, lr: float = 1e-4,
                               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                               weight_decay: float = 0.01, step: int = 1, qblock: int = 64, hyper_device=None):
    """Fused weight gradient + AdamW with int8 moments and per-(row, qblock) fp32 absmax scales
    (``kernel.py:1487-1539``)."""
    st = _int8_state(weight, m_q, v_q, m_scale, v_scale, qblock)
    _wgrad(grad_output, input, weight, OPT_ADAMW, st, _hyper(lr, beta1, beta2, eps, weight_decay, step), hyper_device)


def optimizer_only_adamw_int8state(grad, weight, m_q, v_q, m_scale, v_scale, lr: float = 1e-4,
                                   beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                                   weight_decay: float = 0.01, step: int = 1, qblock: int = 64):
    """AdamW on a pre-computed gradient with int8 moments (``kernel.py:1542-1575``)."""
    st = _int8_state(weight, m_q, v_q, m_scale, v_scale, qblock)
    _optim(grad, weight, OPT_ADAMW, st, _hyper(lr, beta1, beta2, eps, weight_decay, step))


def _fp8_tensor_state(state):
    _require_cuda(state.m_fp8, state.v_fp8)
    return _state(ST_FP8_TENSOR, state.m_fp8, state.v_fp8, state.m_scale, state.v_scale,
                  state.m_absmax_next, state.v_absmax_next)


def fused_grad_adamw_fp8state(grad_output, input, weight, state, lr: float = 1e-4, beta1: float = 0.9,
                              beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
                              step: int = 1, hyper_device=None):
    """Fused weight gradient + AdamW with e4m3 m / e5m2 v and one delayed scale per tensor
    (``kernel_fp8_state.py:343-392``).  ``state`` is a ``FusedOptimizerState`` in fp8 mode; the
    next-step absmax is accumulated by the kernel itself (no scratch arrays, no reduce launches)."""
    _wgrad(grad_output, input, weight, OPT_ADAMW, _fp8_tensor_state(state),
           _hyper(lr, beta1, beta2, eps, weight_decay, step), hyper_device)


def optimizer_only_adamw_fp8state(grad, weight, state, lr: float = 1e-4, beta1: float = 0.9,
                                  beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.01,
                                  step: int = 1):
    """AdamW on a pre-computed gradient with per-tensor fp8 moments (the reference has no such path:
    ``autograd.py:158-176`` reaches for ``state.m``, which does not exist in fp8 mode)."""
    _optim(grad, weight, OPT_ADAMW, _fp8_tensor_state(state), _hyper(lr, beta1, beta2, eps, weight_decay, step))


def fp8_prestep(m_scale, v_scale, m_absmax_next, v_absmax_next):
    """Device-side ``FusedOptimizerState.pre_step_fp8`` (``state.py:132-157``) without host syncs."""
    _require_cuda(m_scale, v_scale, m_absmax_next, v_absmax_next)
    lib = _lib.load()
    with torch.cuda.device(m_scale.device):
        rc = lib.forge_fp8_prestep(m_scale.data_ptr(), v_scale.data_ptr(), m_absmax_next.data_ptr(),
                                   v_absmax_next.data_ptr(), _lib.current_stream_ptr(m_scale.device))
    _lib.check(rc, "forge_fp8_prestep")


# --------------------------------------------------------------------------------------------
# additions without a reference counterpart
# --------------------------------------------------------------------------------------------
def fused_grad_adamw_fp8block(grad_output, input, weight, m_q, v_q, m_scale, v_scale, lr: float = 1e-4,
                              beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                              weight_decay: float = 0.01, step: int = 1, qblock: int = 64, hyper_device=None):
    """AdamW with e4m3 codes for both moments and one fp32 absmax scale per (row, 64 columns):
    the int8 scheme with ``scale = absmax / 448 + 1e-12``.  ``m_q``/``v_q`` are uint8 or float8 views."""
    st = _int8_state(weight, m_q, v_q, m_scale, v_scale, qblock, mode=ST_FP8_BLOCK)
    _wgrad(grad_output, input, weight, OPT_ADAMW, st, _hyper(lr, beta1, beta2, eps, weight_decay, step), hyper_device)


def optimizer_only_adamw_fp8block(grad, weight, m_q, v_q, m_scale, v_scale, lr: float = 1e-4,
                                  beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8,
                                  weight_decay: float = 0.01, step: int = 1, qblock: int = 64):
    st = _int8_state(weight, m_q, v_q, m_scale, v_scale, qblock, mode=ST_FP8_BLOCK)
    _optim(grad, weight, OPT_ADAMW, st, _hyper(lr, beta1, beta2, eps, weight_decay, step))


def fused_grad_sgd_momentum(grad_output, input, weight, buf, lr: float = 1e-3, momentum: float = 0.9,
                            weight_decay: float = 0.0, nesterov: bool = False, hyper_device=None):
    """SGD with momentum: ``buf = mu buf + dW``; ``u = dW + mu buf`` (Nesterov) or ``buf``;
    ``W = W(1 - lr wd) - lr u``.  Buffer semantics of ``torch.optim.SGD`` with dampening 0."""
    _require_cuda(buf)
    _wgrad(grad_output, input, weight, OPT_SGDM, _moment_state(buf),
           _hyper(lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov), hyper_device)


def optimizer_only_sgd(grad, weight, lr: float = 1e-3, weight_decay: float = 0.0):
    _optim(grad, weight, OPT_SGD, _state(), _hyper(lr, weight_decay=weight_decay))


def optimizer_only_sgd_momentum(grad, weight, buf, lr: float = 1e-3, momentum: float = 0.9,
                                weight_decay: float = 0.0, nesterov: bool = False):
    _require_cuda(buf)
    _optim(grad, weight, OPT_SGDM, _moment_state(buf),
           _hyper(lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov))


def fused_grad_lion(grad_output, input, weight, m, lr: float = 1e-4, beta1: float = 0.9,
                    beta2: float = 0.99, weight_decay: float = 0.0, hyper_device=None):
    """Lion: ``u = sign(b1 m + (1-b1) dW)``; ``W = W(1 - lr wd) - lr u``; ``m = b2 m + (1-b2) dW``."""
    _require_cuda(m)
    _wgrad(grad_output, input, weight, OPT_LION, _moment_state(m),
           _hyper(lr, beta1, beta2, weight_decay=weight_decay), hyper_device)


def optimizer_only_lion(grad, weight, m, lr: float = 1e-4, beta1: float = 0.9, beta2: float = 0.99,
                        weight_decay: float = 0.0):
    _require_cuda(m)
    _optim(grad, weight, OPT_LION, _moment_state(m), _hyper(lr, beta1, beta2, weight_decay=weight_decay))


def dgrad_sum(members) -> torch.Tensor:
    """``dX = sum_i dY_i @ W_i`` over one to four bf16 pairs in ONE launch (the input gradient of linears
    that share their input: q / k / v, gate / up); the accumulator never leaves tensor memory."""
    members = list(members)
    if not 1 <= len(members) <= 4:
        raise ValueError("one to four (dY, W) pairs")
    dy0, w0 = members[0]
    _require_cuda(dy0, w0)
    BT, H = dy0.shape[0], w0.shape[1]
    segs = (_lib.ForgeDgradSegment * len(members))()
    for k, (dy, w) in enumerate(members):
        _require_cuda(dy, w)
        if dy.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise ValueError("dgrad_sum takes bfloat16 operands")
        if dy.shape[0] != BT or w.shape[1] != H or dy.shape[1] != w.shape[0]:
            raise ValueError(f"member {k}: shapes {tuple(dy.shape)} x {tuple(w.shape)} do not fit ({BT}, V) x (V, {H})")
        _row_major_2d(dy, "dY")
        _row_major_2d(w, "W")
        segs[k].dY, segs[k].W, segs[k].V = dy.data_ptr(), w.data_ptr(), dy.shape[1]
        segs[k].ld_dy, segs[k].ld_w = dy.stride(0), w.stride(0)
    out = torch.empty(BT, H, dtype=torch.bfloat16, device=dy0.device)
    lib = _lib.load()
    with torch.cuda.device(w0.device):
        rc = lib.forge_dgrad_sum(segs, len(members), out.data_ptr(), BT, H, out.stride(0),
                                 _lib.status_word(w0.device).data_ptr(), _lib.current_stream_ptr(w0.device))
    _lib.check(rc, "forge_dgrad_sum")
    return out


def dgrad(grad_output_2d: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``dX = dY @ W`` for bf16 operands through the library's own GEMM (``autograd.py:55``)."""
    _require_cuda(grad_output_2d, weight)
    BT, V = grad_output_2d.shape
    H = weight.shape[1]
    out = torch.empty(BT, H, dtype=grad_output_2d.dtype, device=grad_output_2d.device)
    lib = _lib.load()
    with torch.cuda.device(weight.device):
        rc = lib.forge_dgrad(grad_output_2d.data_ptr(), weight.data_ptr(), out.data_ptr(), BT, V, H,
                             grad_output_2d.stride(0), weight.stride(0), out.stride(0),
                             _lib.status_word(weight.device).data_ptr(), _lib.current_stream_ptr(weight.device))
    _lib.check(rc, "forge_dgrad")
    return out
