"""The allocation-free entry point ``forge_wgrad_update_static_scratch`` (fp32 dY / X, scratch held in
an array inside the library) against ``forge_wgrad_update`` with caller scratch.

It serves callers that cannot allocate device memory at the point of the call -- a plug-in inside a
host framework's allocator callback, a job whose memory is fully committed to a static plan.  The
test goes through the C ABI with ctypes, runs the new entry point twice in a row (the array keeps
the first call's contents, which must not leak into the second) and demands bit-identical W, m and v.
It is collected last so that a run stopping at the first failure has already run everything else.
"""

import ctypes

import pytest
import torch

from forge_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(dy, x, w, m, v, step, scratch=None):
    a = _lib.ForgeWgradArgs()
    a.dY, a.X, a.W = dy.data_ptr(), x.data_ptr(), w.data_ptr()
    a.BT, a.V = dy.shape
    a.H = x.shape[1]
    a.ld_dy, a.ld_x, a.ld_w = dy.stride(0), x.stride(0), w.stride(0)
    a.operand_dtype = _lib.dtype_id(dy.dtype)
    a.w_dtype = _lib.dtype_id(w.dtype)
    a.optimizer = _lib.OPT_ADAMW
    a.state.mode = _lib.state_mode_id(m.dtype)
    a.state.qblock = 64
    a.state.m, a.state.v, a.state.ld_state = m.data_ptr(), v.data_ptr(), m.stride(0)
    a.hyper = _lib.ForgeHyper(1e-3, 0.9, 0.999, 1e-8, 0.01, 0.0, 0, step)
    if scratch is not None:
        a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    a.status = _lib.status_word(w.device).data_ptr()
    return a


def test_static_scratch_matches_caller_scratch_twice():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two problems of different shape, so the second call finds stale data of another layout in the array
    cases = [(200, 392, 264), (96, 1024, 512)]
    for i, (BT, V, H) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        dy = torch.randn(BT, V, generator=g).to(DEV)
        x = torch.randn(BT, H, generator=g).to(DEV)
        w0 = (torch.randn(V, H, generator=g) * 0.02).to(DEV)
        m0 = (torch.randn(V, H, generator=g) * 1e-3).to(DEV)
        v0 = (torch.randn(V, H, generator=g).abs() * 1e-5).to(DEV)

        need = lib.forge_wgrad_scratch_bytes(BT, V, H, _lib.DT_F32)
        assert 0 < need <= (32 << 20)
        scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
        w1, m1, v1 = w0.clone(), m0.clone(), v0.clone()
        rc = lib.forge_wgrad_update(ctypes.byref(_args(dy, x, w1, m1, v1, 3, scratch)), stream)
        assert rc == 0, _lib.last_error()

        w2, m2, v2 = w0.clone(), m0.clone(), v0.clone()
        rc = lib.forge_wgrad_update_static_scratch(ctypes.byref(_args(dy, x, w2, m2, v2, 3)), stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        for name, a, b in (("W", w1, w2), ("m", m1, m2), ("v", v1, v2)):
            assert torch.equal(a.view(torch.int32), b.view(torch.int32)), f"case {i}: {name} differs"
        assert not torch.equal(w2, w0)
    assert _lib.read_status(torch.device(DEV, torch.cuda.current_device())) == 0


def test_static_scratch_limits():
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # too large for the built-in array: 3 * 512 * (8192 + 8192) * 2 bytes = 48 MiB
    BT, V, H = 512, 8192, 8192
    dy = torch.zeros(BT, V, device=DEV)
    x = torch.zeros(BT, H, device=DEV)
    w = torch.zeros(V, H, device=DEV, dtype=torch.bfloat16)
    m, v = torch.zeros_like(w), torch.zeros_like(w)
    rc = lib.forge_wgrad_update_static_scratch(ctypes.byref(_args(dy, x, w, m, v, 1)), stream)
    assert rc == _lib.FORGE_ERR_SCRATCH and "built-in array" in _lib.last_error()
    # bf16 operands have no business here
    rc = lib.forge_wgrad_update_static_scratch(
        ctypes.byref(_args(dy[:64, :128].bfloat16().contiguous(), x[:64, :128].bfloat16().contiguous(),
                           w[:128, :128].contiguous(), m[:128, :128].contiguous(), v[:128, :128].contiguous(), 1)), stream)
    assert rc == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_wgrad_update_static_scratch(None, stream) == _lib.FORGE_ERR_INVALID_ARG
    torch.cuda.synchronize()
