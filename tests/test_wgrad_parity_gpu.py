"""GPU parity of the fused weight-gradient + optimizer kernel against the CPU oracle.

Every call goes through the Python wrappers -> ctypes -> C ABI (``forge_wgrad_update`` /
``forge_optimizer_update``).  Three kinds of checks:

* exact: inputs whose gradient sums are exact in fp32 (multiples of 1/8), so the tensor-core
  summation order is immaterial and moments / codes / scales (and the SGD / momentum / Lion weights)
  must equal the oracle BIT FOR BIT, for every optimizer, state mode and weight dtype; the AdamW
  weight, whose quotient the device evaluates with approximate reciprocal and square root, must sit
  within ONE bf16 ULP of the oracle;
* tolerance: Gaussian inputs, W / m / v within ONE bf16 ULP of the oracle (the oracle sums the token
  axis sequentially in fp32; the device sums it in tensor-core order);
* the optimizer-only kernels fed the oracle's fp32 gradient: bit for bit, Gaussian inputs included.
"""

import numpy as np
import pytest
import torch

import oracle
from forge_b200 import kernel as K
from tests.util import (ADAMW, as_dtype, assert_bits_equal, assert_one_ulp, assert_w_close,
                        bf16_ulp_distance, gen_inputs, np32, oracle_adamw)

pytestmark = pytest.mark.gpu
DEV = "cuda"

# (BT, V, H): a full tile, several tiles, ragged in every dimension (multiples of 8), tiny
SHAPES = [(64, 128, 256), (512, 1024, 1024), (192, 256, 512), (72, 136, 264), (8, 8, 64), (200, 392, 1032)]


def _dt(name):
    return torch.bfloat16 if name == "bf16" else torch.float32


@pytest.mark.parametrize("BT,V,H", SHAPES)
@pytest.mark.parametrize("wdt,sdt", [("bf16", "bf16"), ("f32", "f32"), ("bf16", "f32")])
def test_adamw_exact(BT, V, H, wdt, sdt):
    dy, x, w, m, v = gen_inputs(1, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    ms, mf = as_dtype(m, _dt(sdt))
    vs, vf = as_dtype(v, _dt(sdt))
    wn, mn, vn, _ = oracle_adamw(dy, x, wf, mf, vf, ADAMW, wdt == "bf16", sdt == "bf16")
    wd, md, vd = ws.to(DEV), ms.to(DEV), vs.to(DEV)
    K.fused_grad_adamw(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, md, vd, **ADAMW)
    assert_w_close(wn, wd, wf)
    assert_bits_equal(mn, md, "m")
    assert_bits_equal(vn, vd, "v")


@pytest.mark.parametrize("BT,V,H", SHAPES)
def test_adamw_bf16_within_one_ulp(BT, V, H):
    dy, x, w, m, v = gen_inputs(2, BT, V, H)
    dyb, xb = dy.bfloat16(), x.bfloat16()
    ws, wf = as_dtype(w, torch.bfloat16)
    ms, mf = as_dtype(m, torch.bfloat16)
    vs, vf = as_dtype(v, torch.bfloat16)
    wn, mn, vn, g = oracle_adamw(dyb, xb, wf, mf, vf, ADAMW, True, True)
    wd, md, vd = ws.to(DEV), ms.to(DEV), vs.to(DEV)
    K.fused_grad_adamw(dyb.to(DEV), xb.to(DEV), wd, md, vd, **ADAMW)
    # fp32 summation noise scales with sum |dY||X| (the terms that were added), not with |g|
    gabs = torch.from_numpy(oracle.wgrad(np32(dyb.abs()), np32(xb.abs())))
    assert_w_close(wn, wd, wf)
    assert_one_ulp(mn, md, 0.9 * mf.abs() + 0.1 * gabs, "m", noise=2e-6)
    assert_one_ulp(vn, vd, torch.from_numpy(vn), "v")
    for name, e, a in (("W", wn, wd), ("m", mn, md), ("v", vn, vd)):
        assert (bf16_ulp_distance(e, a) > 0).float().mean().item() < 0.02, f"{name}: too many roundings differ"
    assert not torch.equal(wd.cpu(), ws)


def test_adamw_fp32_state_close():
    """fp32 W/m/v (fp32 master weights and moments): fp32 agreement up to summation order."""
    BT, V, H = 512, 1024, 1024
    dy, x, w, m, v = gen_inputs(3, BT, V, H)
    dyb, xb = dy.bfloat16(), x.bfloat16()
    wn, mn, vn, _ = oracle_adamw(dyb, xb, w, m, v, ADAMW, False, False)
    wd, md, vd = w.to(DEV), m.to(DEV), v.to(DEV)
    K.fused_grad_adamw(dyb.to(DEV), xb.to(DEV), wd, md, vd, **ADAMW)
    g = oracle.wgrad(np32(dyb), np32(xb))
    np.testing.assert_allclose(np32(md), mn, rtol=2e-5, atol=4e-7 * float(np.abs(g).max()))
    np.testing.assert_allclose(np32(vd), vn, rtol=4e-5, atol=1e-12)
    assert_w_close(wn, wd, w)


@pytest.mark.parametrize("BT,V,H", [(64, 128, 256), (200, 392, 1032)])
@pytest.mark.parametrize("wdt", ["bf16", "f32"])
def test_sgd_exact(BT, V, H, wdt):
    dy, x, w, _, _ = gen_inputs(4, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    g = oracle.wgrad(np32(dy), np32(x))
    wn = np32(wf).copy()
    oracle.sgd(wn, g, oracle.Hyper(lr=0.01, weight_decay=0.1), w_bf16=wdt == "bf16")
    wd = ws.to(DEV)
    K.fused_grad_sgd(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, lr=0.01, weight_decay=0.1)
    assert_bits_equal(wn, wd, "W")


@pytest.mark.parametrize("nesterov", [False, True])
@pytest.mark.parametrize("wdt,sdt", [("bf16", "bf16"), ("f32", "f32")])
def test_sgd_momentum_exact(nesterov, wdt, sdt):
    BT, V, H = 136, 264, 520
    dy, x, w, m, _ = gen_inputs(5, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    ms, mf = as_dtype(m, _dt(sdt))
    g = oracle.wgrad(np32(dy), np32(x))
    wn, bn = np32(wf).copy(), np32(mf).copy()
    oracle.sgdm(wn, bn, g, oracle.Hyper(lr=0.01, weight_decay=0.1, momentum=0.9, nesterov=nesterov),
                w_bf16=wdt == "bf16", s_bf16=sdt == "bf16")
    wd, bd = ws.to(DEV), ms.to(DEV)
    K.fused_grad_sgd_momentum(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, bd, lr=0.01, momentum=0.9,
                              weight_decay=0.1, nesterov=nesterov)
    assert_bits_equal(wn, wd, "W")
    assert_bits_equal(bn, bd, "buf")


@pytest.mark.parametrize("wdt,sdt", [("bf16", "bf16"), ("f32", "f32")])
def test_lion_exact(wdt, sdt):
    BT, V, H = 136, 264, 520
    dy, x, w, m, _ = gen_inputs(6, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    ms, mf = as_dtype(m, _dt(sdt))
    g = oracle.wgrad(np32(dy), np32(x))
    wn, mn = np32(wf).copy(), np32(mf).copy()
    oracle.lion(wn, mn, g, oracle.Hyper(lr=1e-3, beta1=0.9, beta2=0.99, weight_decay=0.1),
                w_bf16=wdt == "bf16", s_bf16=sdt == "bf16")
    wd, md = ws.to(DEV), ms.to(DEV)
    K.fused_grad_lion(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, md, lr=1e-3, beta1=0.9, beta2=0.99,
                      weight_decay=0.1)
    assert_bits_equal(wn, wd, "W")
    assert_bits_equal(mn, md, "m")


# ------------------------------------------------------------------ quantised moments
def _blockq_start(m, v, kind):
    """Initial codes/scales: quantise the seeded m, v with the oracle's own quantiser."""
    if kind == "int8":
        mq, ms = oracle.int8_quantise(np32(m))
        vq, vs = oracle.int8_quantise(np32(v))
        return mq, vq, ms, vs
    # e4m3 per block: scale = absmax/448 + 1e-12
    V, H = m.shape
    out = []
    for t in (m, v):
        tb = np32(t).reshape(V, H // 64, 64)
        s = (np.abs(tb).max(axis=2) / np.float32(448.0) + np.float32(1e-12)).astype(np.float32)
        q = oracle.e4m3_encode((tb / s[:, :, None]).astype(np.float32)).reshape(V, H)
        out.append((q, s))
    return out[0][0], out[1][0], out[0][1], out[1][1]


@pytest.mark.parametrize("BT,V,H", [(64, 128, 256), (192, 256, 512), (72, 136, 320), (200, 392, 1088)])
@pytest.mark.parametrize("kind", ["int8", "e4m3"])
@pytest.mark.parametrize("wdt", ["bf16", "f32"])
def test_blockq_exact(BT, V, H, kind, wdt):
    dy, x, w, m, v = gen_inputs(7, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    mq, vq, ms, vs = _blockq_start(m, v, kind)
    g = oracle.wgrad(np32(dy), np32(x))
    wn = np32(wf).copy()
    emq, evq, ems, evs = mq.copy(), vq.copy(), ms.copy(), vs.copy()
    oracle.adamw_blockq(wn, emq, evq, ems, evs, g, oracle.Hyper(**ADAMW), w_bf16=wdt == "bf16", kind=kind)
    wd = ws.to(DEV)
    code_dt = torch.int8 if kind == "int8" else torch.uint8
    dmq = torch.from_numpy(mq.view(np.int8) if kind == "int8" else mq).to(code_dt).to(DEV)
    dvq = torch.from_numpy(vq.view(np.int8) if kind == "int8" else vq).to(code_dt).to(DEV)
    dms, dvs = torch.from_numpy(ms).to(DEV), torch.from_numpy(vs).to(DEV)
    fn = K.fused_grad_adamw_int8state if kind == "int8" else K.fused_grad_adamw_fp8block
    fn(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, dmq, dvq, dms, dvs, qblock=64, **ADAMW)
    assert_w_close(wn, wd, wf)
    assert_bits_equal(ems, dms, "m_scale")
    assert_bits_equal(evs, dvs, "v_scale")
    assert_bits_equal(emq.view(np.uint8), dmq, "m codes")
    assert_bits_equal(evq.view(np.uint8), dvq, "v codes")


def test_int8_from_initial_state_gaussian():
    """Fresh state (codes 0, scales 1; reference init, state.py:103-107) and Gaussian inputs: codes
    may differ by one unit where x/scale lands within summation noise of .5."""
    BT, V, H = 256, 512, 1024
    dy, x, w, _, _ = gen_inputs(8, BT, V, H)
    dyb, xb = dy.bfloat16(), x.bfloat16()
    ws, wf = as_dtype(w, torch.bfloat16)
    g = oracle.wgrad(np32(dyb), np32(xb))
    wn = np32(wf).copy()
    emq, evq = np.zeros((V, H), np.int8), np.zeros((V, H), np.int8)
    ems, evs = np.ones((V, H // 64), np.float32), np.ones((V, H // 64), np.float32)
    hp = dict(ADAMW, step=1)
    oracle.adamw_blockq(wn, emq, evq, ems, evs, g, oracle.Hyper(**hp), w_bf16=True, kind="int8")
    wd = ws.to(DEV)
    dmq, dvq = torch.zeros(V, H, dtype=torch.int8, device=DEV), torch.zeros(V, H, dtype=torch.int8, device=DEV)
    dms, dvs = torch.ones(V, H // 64, device=DEV), torch.ones(V, H // 64, device=DEV)
    K.fused_grad_adamw_int8state(dyb.to(DEV), xb.to(DEV), wd, dmq, dvq, dms, dvs, qblock=64, **hp)
    assert_w_close(wn, wd, wf)
    np.testing.assert_allclose(np32(dms), ems, rtol=2e-5)
    np.testing.assert_allclose(np32(dvs), evs, rtol=4e-5)
    for e, a in ((emq, dmq), (evq, dvq)):
        d = (torch.from_numpy(e).int() - a.cpu().int()).abs()
        assert d.max().item() <= 1
        assert (d > 0).float().mean().item() < 0.01
    assert dmq.any()


@pytest.mark.parametrize("BT,V,H", [(64, 128, 256), (200, 392, 1040)])
@pytest.mark.parametrize("wdt", ["bf16", "f32"])
def test_fp8_tensor_exact(BT, V, H, wdt):
    dy, x, w, m, v = gen_inputs(9, BT, V, H, exact=True)
    ws, wf = as_dtype(w, _dt(wdt))
    s_m, s_v = np.float32(0.02), np.float32(6e-5)
    m8 = oracle.e4m3_encode(np32(m) / s_m)
    v8 = oracle.e5m2_encode(np32(v) / s_v)
    g = oracle.wgrad(np32(dy), np32(x))
    wn, em8, ev8 = np32(wf).copy(), m8.copy(), v8.copy()
    amax = np.array([0.5, 0.0], np.float32)   # a running max left by another launch must survive
    oracle.adamw_fp8tensor(wn, em8, ev8, s_m, s_v, amax, g, oracle.Hyper(**ADAMW), w_bf16=wdt == "bf16")

    class St:
        pass
    st = St()
    st.m_fp8 = torch.from_numpy(m8).to(DEV).view(torch.float8_e4m3fn)
    st.v_fp8 = torch.from_numpy(v8).to(DEV).view(torch.float8_e5m2)
    st.m_scale, st.v_scale = torch.tensor(float(s_m), device=DEV), torch.tensor(float(s_v), device=DEV)
    st.m_absmax_next, st.v_absmax_next = torch.tensor(0.5, device=DEV), torch.tensor(0.0, device=DEV)
    wd = ws.to(DEV)
    K.fused_grad_adamw_fp8state(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), wd, st, **ADAMW)
    assert_w_close(wn, wd, wf)
    assert_bits_equal(em8, st.m_fp8.view(torch.uint8), "m codes")
    assert_bits_equal(ev8, st.v_fp8.view(torch.uint8), "v codes")
    assert st.m_absmax_next.item() == amax[0] and st.v_absmax_next.item() == amax[1]


def test_fp8_prestep_matches_oracle(golden_dir):
    import json
    import os
    rows = json.load(open(os.path.join(golden_dir, "fp8_prestep.json")))
    ms, vs = torch.ones((), device=DEV), torch.ones((), device=DEV)
    am, av = torch.zeros((), device=DEV), torch.zeros((), device=DEV)
    for r in rows:
        am.fill_(r["amax_m"])
        av.fill_(r["amax_v"])
        K.fp8_prestep(ms, vs, am, av)
        assert ms.item() == np.float32(r["m_scale"]) and vs.item() == np.float32(r["v_scale"])
        assert am.item() == 0.0 and av.item() == 0.0


# ------------------------------------------------------------------ optimizer-only kernels
@pytest.mark.parametrize("gdt", ["f32", "bf16"])
@pytest.mark.parametrize("wdt,sdt", [("bf16", "bf16"), ("f32", "f32"), ("bf16", "f32")])
def test_optimizer_only_adamw_bit_exact(gdt, wdt, sdt):
    V, H = 264, 528
    gen = torch.Generator().manual_seed(10)
    g = torch.randn(V, H, generator=gen) * 3
    _, _, w, m, v = gen_inputs(10, 8, V, H)
    gs, gf = as_dtype(g, _dt(gdt))
    ws, wf = as_dtype(w, _dt(wdt))
    ms, mf = as_dtype(m, _dt(sdt))
    vs, vf = as_dtype(v, _dt(sdt))
    wn, mn, vn = np32(wf).copy(), np32(mf).copy(), np32(vf).copy()
    oracle.adamw(wn, mn, vn, np32(gf), oracle.Hyper(**ADAMW), w_bf16=wdt == "bf16", s_bf16=sdt == "bf16")
    wd, md, vd = ws.to(DEV), ms.to(DEV), vs.to(DEV)
    K.optimizer_only_adamw(gs.to(DEV), wd, md, vd, **ADAMW)
    assert_w_close(wn, wd, wf)
    assert_bits_equal(mn, md, "m")
    assert_bits_equal(vn, vd, "v")


@pytest.mark.parametrize("kind", ["int8", "e4m3"])
def test_optimizer_only_blockq_bit_exact(kind):
    V, H = 200, 576
    gen = torch.Generator().manual_seed(11)
    g = torch.randn(V, H, generator=gen) * 0.05
    _, _, w, m, v = gen_inputs(11, 8, V, H)
    ws, wf = as_dtype(w, torch.bfloat16)
    mq, vq, ms, vs = _blockq_start(m, v, kind)
    wn = np32(wf).copy()
    emq, evq, ems, evs = mq.copy(), vq.copy(), ms.copy(), vs.copy()
    oracle.adamw_blockq(wn, emq, evq, ems, evs, np32(g), oracle.Hyper(**ADAMW), w_bf16=True, kind=kind)
    wd = ws.to(DEV)
    code_dt = torch.int8 if kind == "int8" else torch.uint8
    dmq, dvq = torch.from_numpy(mq).to(code_dt).to(DEV), torch.from_numpy(vq).to(code_dt).to(DEV)
    dms, dvs = torch.from_numpy(ms).to(DEV), torch.from_numpy(vs).to(DEV)
    fn = K.optimizer_only_adamw_int8state if kind == "int8" else K.optimizer_only_adamw_fp8block
    fn(g.to(DEV), wd, dmq, dvq, dms, dvs, qblock=64, **ADAMW)
    assert_w_close(wn, wd, wf)
    assert_bits_equal(ems, dms, "m_scale")
    assert_bits_equal(evs, dvs, "v_scale")
    assert_bits_equal(emq.view(np.uint8), dmq, "m codes")
    assert_bits_equal(evq.view(np.uint8), dvq, "v codes")


def test_fused_equals_unfused_twin_bitwise():
    """Determinism: the fused kernel run twice gives identical bits, and equals the optimizer-only
    kernel fed the gradient the SGD variant of the same mainloop reveals (lr=1, no decay: W' = W - g
    with W = 0 gives -g exactly)."""
    BT, V, H = 512, 1024, 1024
    dy, x, w, m, v = gen_inputs(12, BT, V, H)
    dyd, xd = dy.bfloat16().to(DEV), x.bfloat16().to(DEV)
    outs = []
    for _ in range(2):
        wd, md, vd = w.bfloat16().to(DEV), m.bfloat16().to(DEV), v.bfloat16().to(DEV)
        K.fused_grad_adamw(dyd, xd, wd, md, vd, **ADAMW)
        outs.append((wd, md, vd))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    gneg = torch.zeros(V, H, device=DEV)
    K.fused_grad_sgd(dyd, xd, gneg, lr=1.0, weight_decay=0.0)   # fp32 W: stores -g unrounded
    wd, md, vd = w.bfloat16().to(DEV), m.bfloat16().to(DEV), v.bfloat16().to(DEV)
    K.optimizer_only_adamw((-gneg).contiguous(), wd, md, vd, **ADAMW)
    for a, b in zip(outs[0], (wd, md, vd)):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


# the last shape has a single row tile: single-CTA units (no pairs), several rounds of them and a half-tile tail
@pytest.mark.parametrize("V,H", [(14336, 4096), (4096, 14336), (4096, 4096), (1024, 4096), (128, 81920)])
@pytest.mark.parametrize("mode", ["bf16", "int8"])
def test_full_size_fused_equals_unfused_twin(V, H, mode):
    """The Llama-3.1-8B projection shapes at BT = 512 (many rounds of work units per SM pair, the
    half-tile tail, every tile of the weight): the fused update equals, bit for bit, the
    optimizer-only kernel fed the gradient that the SGD variant of the same mainloop reveals."""
    BT = 512
    gen = torch.Generator(device=DEV).manual_seed(5)
    dyd = (torch.randn(BT, V, device=DEV, generator=gen) * 1e-2).bfloat16()
    xd = torch.randn(BT, H, device=DEV, generator=gen).bfloat16()
    w0 = (torch.randn(V, H, device=DEV, generator=gen) * 0.02).bfloat16()
    gneg = torch.zeros(V, H, device=DEV)
    K.fused_grad_sgd(dyd, xd, gneg, lr=1.0, weight_decay=0.0)   # fp32 W = 0: stores -g unrounded
    grad = (-gneg).contiguous()
    del gneg
    if mode == "bf16":
        m0 = (torch.randn(V, H, device=DEV, generator=gen) * 1e-3).bfloat16()
        v0 = (torch.randn(V, H, device=DEV, generator=gen).abs() * 1e-5).bfloat16()
        fused = (w0.clone(), m0.clone(), v0.clone())
        twin = (w0.clone(), m0.clone(), v0.clone())
        K.fused_grad_adamw(dyd, xd, *fused, **ADAMW)
        K.optimizer_only_adamw(grad, *twin, **ADAMW)
    else:
        mq = torch.randint(-127, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
        vq = torch.randint(0, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
        ms = torch.rand(V, H // 64, device=DEV, generator=gen) * 1e-5 + 1e-6
        vs = torch.rand(V, H // 64, device=DEV, generator=gen) * 1e-9 + 1e-10
        fused = (w0.clone(), mq.clone(), vq.clone(), ms.clone(), vs.clone())
        twin = (w0.clone(), mq.clone(), vq.clone(), ms.clone(), vs.clone())
        K.fused_grad_adamw_int8state(dyd, xd, *fused, **ADAMW)
        K.optimizer_only_adamw_int8state(grad, *twin, **ADAMW)
    torch.cuda.synchronize()
    assert not torch.equal(fused[0], w0)
    for name, a, b in zip(("W", "m", "v", "m_scale", "v_scale"), fused, twin):
        ai = a.view(torch.int16 if a.dtype == torch.bfloat16 else (torch.int32 if a.dtype == torch.float32 else torch.int8))
        bi = b.view(ai.dtype)
        assert torch.equal(ai, bi), f"{name}: {(ai != bi).sum().item()} of {ai.numel()} elements differ"


def test_concurrent_streams_equal_sequential_bitwise():
    """Several fused updates in flight at once on different streams (as in a multi-branch CUDA graph):
    every SM is taken by one update at a time and the launches take over each other's SMs at their
    ragged ends; each must produce the bits of a run on its own."""
    BT = 256
    shapes = [(1024, 4096), (4096, 1024), (2048, 2048), (136, 264), (4096, 4096), (1024, 1024)]
    gen = torch.Generator(device=DEV).manual_seed(9)
    jobs = []
    for V, H in shapes:
        dy = (torch.randn(BT, V, device=DEV, generator=gen) * 1e-2).bfloat16()
        x = torch.randn(BT, H, device=DEV, generator=gen).bfloat16()
        w = (torch.randn(V, H, device=DEV, generator=gen) * 0.02).bfloat16()
        m = (torch.randn(V, H, device=DEV, generator=gen) * 1e-3).bfloat16()
        v = (torch.randn(V, H, device=DEV, generator=gen).abs() * 1e-5).bfloat16()
        jobs.append((dy, x, w, m, v))
    ref = []
    for dy, x, w, m, v in jobs:
        st = (w.clone(), m.clone(), v.clone())
        for step in range(1, 4):
            K.fused_grad_adamw(dy, x, *st, **dict(ADAMW, step=step))
        ref.append(st)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(4)]
    got = [(w.clone(), m.clone(), v.clone()) for _, _, w, m, v in jobs]
    torch.cuda.synchronize()
    for step in range(1, 4):
        for i, (dy, x, *_rest) in enumerate(jobs):
            with torch.cuda.stream(streams[i % 4]):
                K.fused_grad_adamw(dy, x, *got[i], **dict(ADAMW, step=step))
    torch.cuda.synchronize()
    for a, b in zip(ref, got):
        for ta, tb in zip(a, b):
            assert torch.equal(ta.view(torch.int16), tb.view(torch.int16))


# ------------------------------------------------------------------ fp32 operands, edge cases, errors
@pytest.mark.parametrize("BT,V,H", [(128, 256, 128), (64, 512, 256), (256, 1024, 512), (50, 136, 264)])
def test_fp32_operands_close_to_fp32_oracle(BT, V, H):
    """fp32 dY/X go through the bf16 hi/lo split: agreement with the fp32 oracle well inside the
    reference's own tolerance for its TF32 dot (5e-3, tests/test_correctness.py:21-24)."""
    gen = torch.Generator().manual_seed(42)
    dy, x = torch.randn(BT, V, generator=gen), torch.randn(BT, H, generator=gen)
    w = torch.randn(V, H, generator=gen)
    m, v = torch.randn(V, H, generator=gen) * 0.01, torch.randn(V, H, generator=gen).abs() * 0.01
    wn, mn, vn, g = oracle_adamw(dy, x, w, m, v, ADAMW, False, False)
    wd, md, vd = w.to(DEV), m.to(DEV), v.to(DEV)
    K.fused_grad_adamw(dy.to(DEV), x.to(DEV), wd, md, vd, **ADAMW)
    np.testing.assert_allclose(np32(wd), wn, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(np32(md), mn, rtol=1e-3, atol=2e-4)
    np.testing.assert_allclose(np32(vd), vn, rtol=1e-3, atol=2e-4)
    # the split keeps 16 significand bits per operand: far inside the reference's TF32 (10 bits)
    assert np.abs(np32(md) - mn).max() < 1e-4 * np.abs(g).max() * 0.1 + 1e-6
    ws = w.clone().to(DEV)
    K.fused_grad_sgd(dy.to(DEV), x.to(DEV), ws, lr=0.01, weight_decay=0.1)
    wsn = np32(w).copy()
    oracle.sgd(wsn, g, oracle.Hyper(lr=0.01, weight_decay=0.1))
    np.testing.assert_allclose(np32(ws), wsn, rtol=1e-4, atol=2e-5)


def test_no_tokens_applies_decay_only():
    V, H = 128, 256
    _, _, w, m, v = gen_inputs(13, 8, V, H)
    wn, mn, vn = np32(w).copy(), np32(m).copy(), np32(v).copy()
    oracle.adamw(wn, mn, vn, np.zeros((V, H), np.float32), oracle.Hyper(**ADAMW))
    wd, md, vd = w.to(DEV), m.to(DEV), v.to(DEV)
    K.fused_grad_adamw(torch.zeros(0, V, dtype=torch.bfloat16, device=DEV),
                       torch.zeros(0, H, dtype=torch.bfloat16, device=DEV), wd, md, vd, **ADAMW)
    assert_w_close(wn, wd, w)
    assert_bits_equal(mn, md, "m")
    assert_bits_equal(vn, vd, "v")


def test_strided_weight_rows():
    """W, m, v as column slices of wider buffers (row pitch > H): neighbours must stay untouched."""
    BT, V, H, LD = 64, 128, 256, 384
    dy, x, w, m, v = gen_inputs(14, BT, V, H, exact=True)
    wn, mn, vn, _ = oracle_adamw(dy, x, w.bfloat16().float(), m.bfloat16().float(), v.bfloat16().float(),
                                 ADAMW, True, True)
    bufs = [torch.full((V, LD), 7.0, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    views = [b[:, 64:64 + H] for b in bufs]
    for vw, src in zip(views, (w, m, v)):
        vw.copy_(src.bfloat16())
    K.fused_grad_adamw(dy.bfloat16().to(DEV), x.bfloat16().to(DEV), *views, **ADAMW)
    assert_w_close(wn, views[0].contiguous(), w.bfloat16().float())
    assert_bits_equal(mn, views[1].contiguous(), "m")
    assert_bits_equal(vn, views[2].contiguous(), "v")
    for b in bufs:
        assert (b[:, :64] == 7.0).all() and (b[:, 64 + H:] == 7.0).all()


def test_error_conventions():
    dy = torch.zeros(64, 128, dtype=torch.bfloat16, device=DEV)
    x = torch.zeros(64, 96, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 96, dtype=torch.bfloat16, device=DEV)
    mq = torch.zeros(128, 96, dtype=torch.int8, device=DEV)
    sc = torch.ones(128, 1, device=DEV)
    with pytest.raises(AssertionError):          # H % qblock != 0: same assertion as the reference
        K.fused_grad_adamw_int8state(dy, x, w, mq, mq.clone(), sc, sc.clone(), qblock=64)
    with pytest.raises(AssertionError):          # non-contiguous operands
        K.fused_grad_sgd(dy.t().contiguous().t(), x, w)
    with pytest.raises(ValueError):              # shape mismatch
        K.fused_grad_sgd(dy, x[:32], w)
    with pytest.raises(ValueError):              # step 0 has no bias correction
        K.fused_grad_adamw(dy, x, w, w.clone(), w.clone(), step=0)
    from forge_b200 import _lib
    with pytest.raises(_lib.ForgeLibraryError):  # row pitch not a multiple of 16 bytes
        K.fused_grad_sgd(torch.zeros(64, 100, dtype=torch.bfloat16, device=DEV), x[:, :92].contiguous(),
                         torch.zeros(100, 92, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(_lib.ForgeLibraryError):  # CPU tensors: no fallback
        K.fused_grad_sgd(dy.cpu(), x.cpu(), w.cpu())


def test_device_hyper_and_graph_replay():
    """Hyper-parameters read from device memory: same bits as the direct path, and a captured CUDA
    graph replays correctly with a new lr / step after the device block is rewritten."""
    BT, V, H = 192, 384, 512
    dy, x, w, m, v = gen_inputs(31, BT, V, H)
    dyd, xd = dy.bfloat16().to(DEV), x.bfloat16().to(DEV)
    ref = [t.bfloat16().to(DEV) for t in (w, m, v)]
    got = [t.bfloat16().to(DEV) for t in (w, m, v)]
    hd = K.DeviceHyper(torch.device(DEV, torch.cuda.current_device()))
    # warm-up outside capture (first launch sets function attributes)
    scratch = [t.clone() for t in got]
    hd.update(lr=1e-3, step=1, weight_decay=0.01)
    K.fused_grad_adamw(dyd, xd, *scratch, hyper_device=hd)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        K.fused_grad_adamw(dyd, xd, *got, hyper_device=hd)
    for step, lr in ((1, 1e-3), (2, 5e-4), (3, 2e-3)):
        K.fused_grad_adamw(dyd, xd, *ref, lr=lr, weight_decay=0.01, step=step)
        hd.update(lr=lr, weight_decay=0.01, step=step)      # 64-byte copy ahead of the replay
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(ref, got):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16)), f"step {step}"
