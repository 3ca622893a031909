"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once in a container that has the reference checkout (its directory is taken from the
``REFERENCE_ROOT`` environment variable); the tests only read the ``.npz`` / ``.json`` files it writes, so nothing at test
time needs the reference.  Sources of truth, in order of strength:

A. ``interp_*.npz`` -- the bodies of the reference's Triton kernels executed by Triton's CPU
   interpreter (``TRITON_INTERPRET=1``), called past the autotuner with explicit tile sizes:
   ``_fused_grad_adamw_kernel`` and ``_fused_grad_sgd_kernel`` (``kernel.py:212-317, 122-205``),
   ``_fused_grad_adamw_int8state_kernel`` (``kernel.py:324-478``) and
   ``_fused_grad_adamw_persistent_tma_fp8state_nows`` (``kernel_fp8_state.py:204-295``).  Inputs are
   multiples of 1/8 so that every partial sum of the gradient is exact in fp32 and the tile /
   summation order cannot matter; the update arithmetic is then compared bit for bit.  One
   intrinsic is substituted: ``libdevice.rint`` (not interpretable) by the equivalent
   add-and-subtract-1.5*2^23 rounding, exact for |x| < 2^22.  Known interpreter defect: its
   float -> fp8 cast is not a faithful round-to-nearest-even.  It drops the carry when rounding
   bumps the mantissa into the next binade (126.125 becomes 64 instead of 128 in e4m3; torch's cast
   and the hardware give 128), rounds exact ties away from zero and flushes some subnormals, so a
   few percent of the fp8 codes in ``interp_fp8.npz`` are off; the test that reads it excuses
   exactly those patterns (W and the absmax values are unaffected and compared bit for bit).
B. ``helper_*.npz`` -- ``_reference_sgd_step`` / ``_reference_adamw_step`` from the reference's
   ``tests/test_correctness.py:27-55`` on its three shapes with its seed (42) and hyper-parameters,
   on CPU.  Outputs are stored for every 13th row together with a checksum of the seeded inputs.
C. ``fp8_prestep.json`` -- ``FusedOptimizerState.pre_step_fp8`` (``state.py:132-157``) driven on CPU
   with a fixed absmax sequence.
D. ``state_layout.json`` -- buffer names, shapes, dtypes and initial values that
   ``FusedOptimizerState.ensure_buffers`` (``state.py:95-130``) allocates for each mode.
"""

import json
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
REF = os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("set REFERENCE_ROOT to the reference checkout")
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

import fused_grad_optimizer.kernel as K  # noqa: E402
import fused_grad_optimizer.kernel_fp8_state as F8  # noqa: E402
from fused_grad_optimizer.state import FusedOptimizerState  # noqa: E402
from tests.test_correctness import _reference_adamw_step, _reference_sgd_step  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


@triton.jit
def _rint_exact(x):
    return (x + 12582912.0) - 12582912.0


tl.extra.cuda.libdevice.rint = _rint_exact

HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=5)


def _exact_inputs(seed, BT, V, H):
    g = torch.Generator().manual_seed(seed)
    dy = torch.randint(-16, 17, (BT, V), generator=g).float() / 8
    x = torch.randint(-16, 17, (BT, H), generator=g).float() / 8
    w = torch.randn(V, H, generator=g)
    m = torch.randn(V, H, generator=g) * 0.01
    v = torch.randn(V, H, generator=g).abs() * 0.01
    return dy, x, w, m, v


def _quantise_like_reference_test(t, qblock):
    """The quantiser of tests/test_correctness.py:170-180, verbatim semantics."""
    V, H = t.shape
    q = torch.zeros(V, H, dtype=torch.int8)
    s = torch.ones(V, H // qblock)
    for b in range(H // qblock):
        blk = t[:, b * qblock:(b + 1) * qblock]
        sc = blk.abs().amax(dim=1) / 127.0 + 1e-12
        s[:, b] = sc
        q[:, b * qblock:(b + 1) * qblock] = (blk / sc[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q, s


def make_interp():
    BT, V, H = 64, 128, 128
    h = HYPER
    bc1, bc2 = 1.0 - h["beta1"] ** h["step"], 1.0 - h["beta2"] ** h["step"]
    tiles = dict(BLOCK_V=64, BLOCK_H=64, BLOCK_BT=32, GROUP_SIZE_V=8)
    grid = (triton.cdiv(V, 64) * triton.cdiv(H, 64),)
    dy, x, w, m, v = _exact_inputs(7, BT, V, H)
    strides = (dy.stride(0), dy.stride(1), x.stride(0), x.stride(1), w.stride(0), w.stride(1))

    # AdamW fp32
    w1, m1, v1 = w.clone(), m.clone(), v.clone()
    K._fused_grad_adamw_kernel.fn[grid](dy, x, w1, m1, v1, BT, V, H, *strides, h["lr"], h["beta1"], h["beta2"],
                                        h["eps"], h["weight_decay"], bc1, bc2, **tiles)
    # SGD
    w2 = w.clone()
    K._fused_grad_sgd_kernel.fn[grid](dy, x, w2, BT, V, H, *strides, 0.01, 0.1, **tiles)
    np.savez_compressed(os.path.join(HERE, "interp_adamw_sgd.npz"), dy=dy.numpy(), x=x.numpy(), w=w.numpy(),
                        m=m.numpy(), v=v.numpy(), w_adamw=w1.numpy(), m_adamw=m1.numpy(), v_adamw=v1.numpy(),
                        w_sgd=w2.numpy(), sgd_lr=0.01, sgd_wd=0.1, **{k: np.float64(val) for k, val in h.items()})

    # int8 moments: start from the reference test's quantisation of (m, v)
    mq, ms = _quantise_like_reference_test(m, 64)
    vq, vs = _quantise_like_reference_test(v, 64)
    mq0, ms0, vq0, vs0 = mq.clone(), ms.clone(), vq.clone(), vs.clone()
    w3 = w.clone()
    K._fused_grad_adamw_int8state_kernel.fn[grid](dy, x, w3, mq, vq, ms, vs, BT, V, H, *strides, mq.stride(0),
                                                  mq.stride(1), ms.stride(0), ms.stride(1), h["lr"], h["beta1"],
                                                  h["beta2"], h["eps"], h["weight_decay"], bc1, bc2, QBLOCK=64, **tiles)
    np.savez_compressed(os.path.join(HERE, "interp_int8.npz"), mq0=mq0.numpy(), ms0=ms0.numpy(), vq0=vq0.numpy(),
                        vs0=vs0.numpy(), w_out=w3.numpy(), mq=mq.numpy(), vq=vq.numpy(), ms=ms.numpy(), vs=vs.numpy())

    # fp8 moments, one scale per tensor
    s_m, s_v = torch.tensor(0.02), torch.tensor(5.5e-5)
    m8 = (m / s_m).clamp(-448, 448).to(torch.float8_e4m3fn)
    v8 = (v / s_v).clamp(-57344, 57344).to(torch.float8_e5m2)
    m8_0, v8_0 = m8.clone(), v8.clone()
    scr_m, scr_v = torch.zeros(4), torch.zeros(4)
    w4 = w.clone()
    F8._fused_grad_adamw_persistent_tma_fp8state_nows.fn[(2,)](
        dy, x, w4, m8, v8, s_m, s_v, scr_m, scr_v, BT, V, H, *strides, m8.stride(0), m8.stride(1), h["lr"],
        h["beta1"], h["beta2"], h["eps"], h["weight_decay"], bc1, bc2, FP8_E4M3_MAX=448.0, FP8_E5M2_MAX=57344.0,
        NUM_SMS=2, BLOCK_V=128, BLOCK_H=128, BLOCK_BT=32, GROUP_SIZE_V=8)
    np.savez_compressed(os.path.join(HERE, "interp_fp8.npz"), m8_0=m8_0.view(torch.uint8).numpy(),
                        v8_0=v8_0.view(torch.uint8).numpy(), s_m=np.float32(s_m.item()), s_v=np.float32(s_v.item()),
                        w_out=w4.numpy(), m8=m8.view(torch.uint8).numpy(), v8=v8.view(torch.uint8).numpy(),
                        amax_m=np.float32(scr_m.max().item()), amax_v=np.float32(scr_v.max().item()))


def _checksum(*tensors):
    return [float(t.double().sum().item()) for t in tensors] + [float(t.double().abs().sum().item()) for t in tensors]


def make_helper():
    out = {}
    for BT, V, H in [(128, 256, 128), (64, 512, 256), (256, 1024, 512)]:
        torch.manual_seed(42)
        go = torch.randn(BT, V)
        inp = torch.randn(BT, H)
        w = torch.randn(V, H)
        w_sgd = _reference_sgd_step(go, inp, w, 0.01, 0.1)
        torch.manual_seed(42)
        go = torch.randn(BT, V)
        inp = torch.randn(BT, H)
        w = torch.randn(V, H)
        m = torch.randn(V, H) * 0.01
        v = torch.randn(V, H).abs() * 0.01
        w_a, m_a, v_a = _reference_adamw_step(go, inp, w, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 5)
        key = f"{BT}x{V}x{H}"
        out[key + "_check"] = np.array(_checksum(go, inp, w, m, v))
        out[key + "_w_sgd"] = w_sgd[::13].numpy()
        out[key + "_w"] = w_a[::13].numpy()
        out[key + "_m"] = m_a[::13].numpy()
        out[key + "_v"] = v_a[::13].numpy()
    np.savez_compressed(os.path.join(HERE, "helper_steps.npz"), **out)


def make_prestep():
    w = torch.zeros(128, 128)
    st = FusedOptimizerState(w, "adamw", state_mode="fp8")
    st.ensure_buffers()
    amax_m = [0.0, 3e-3, 2.5e-3, 2.6e-3, 1e-2, 5e-2, 4e-2, 1e-1, 1e-1, 9e-2, 0.0, 1e-9] + [0.05] * 20
    amax_v = [0.0, 6e-4, 7e-4, 7e-4, 1e-3, 2e-3, 2e-3, 3e-3, 3e-3, 2e-3, 0.0, 1e-12] + [0.002] * 20
    rows = []
    for am, av in zip(amax_m, amax_v):
        st.m_absmax_next.fill_(am)
        st.v_absmax_next.fill_(av)
        st.pre_step_fp8()
        rows.append(dict(amax_m=am, amax_v=av, m_scale=float(st.m_scale), v_scale=float(st.v_scale),
                         m_next=float(st.m_absmax_next), v_next=float(st.v_absmax_next)))
    with open(os.path.join(HERE, "fp8_prestep.json"), "w") as f:
        json.dump(rows, f, indent=1)


def make_layout():
    layout = {}
    w = torch.zeros(256, 128, dtype=torch.bfloat16)
    for mode in ("bf16", "int8", "fp8"):
        st = FusedOptimizerState(w, "adamw", state_mode=mode)
        st.ensure_buffers()
        bufs = {}
        for name, t in vars(st).items():
            if isinstance(t, torch.Tensor) and not name.startswith("_"):
                bufs[name] = dict(shape=list(t.shape), dtype=str(t.dtype), init=float(t.float().flatten()[0]) if t.numel() else 0.0,
                                  uniform=bool((t.float() == t.float().flatten()[0]).all()) if t.numel() else True)
        layout[mode] = dict(buffers=bufs, quantize_state=st.quantize_state, qblock=st.qblock_size, step=st.step)
    st = FusedOptimizerState(w, "sgd")
    st.ensure_buffers()
    layout["sgd"] = dict(buffers={n: 0 for n, t in vars(st).items() if isinstance(t, torch.Tensor) and not n.startswith("_")})
    with open(os.path.join(HERE, "state_layout.json"), "w") as f:
        json.dump(layout, f, indent=1)


if __name__ == "__main__":
    make_interp()
    make_helper()
    make_prestep()
    make_layout()
    for fn in sorted(os.listdir(HERE)):
        print(fn, os.path.getsize(os.path.join(HERE, fn)))
