"""The projection shapes of Llama-3.1-8B and Qwen3-32B at BT = 512, whole weights, every moment
storage: the fused kernel against the CPU oracle on sampled rows.

Rows of dW = dY^T X and of the update are independent of each other, so the oracle recomputes a few
row slices of each weight (all columns: every column tile, chunk and the half-tile tail) -- the rows
around the boundary between the two CTAs of the first pair tile, a slice of a middle tile, and the
last rows of the last (possibly ragged) tile.  Inputs are multiples of 1/8, for which every partial
sum of the gradient is exact in fp32 whatever the summation order, so moments, codes and scales
must equal the oracle's BIT FOR BIT and the AdamW weight must sit within one bf16 ULP."""

import numpy as np
import pytest
import torch

import oracle
from forge_b200 import kernel as K
from tests.util import ADAMW, assert_bits_equal, assert_w_close, np32

pytestmark = pytest.mark.gpu
DEV = "cuda"
BT = 512

LLAMA = [("llama q/o", 4096, 4096), ("llama k/v", 1024, 4096), ("llama gate/up", 14336, 4096),
         ("llama down", 4096, 14336), ("llama lm_head", 128256, 4096)]
QWEN = [("qwen q", 8192, 5120), ("qwen k/v", 1024, 5120), ("qwen o", 5120, 8192), ("qwen gate/up", 25600, 5120),
        ("qwen down", 5120, 25600), ("qwen lm_head", 151936, 5120)]


def _row_slices(V):
    tiles = (V + 255) // 256
    mid = (tiles // 2) * 256
    cand = [(0, 16), (96, 160), (mid + 32, mid + 96), (V - 64, V)]
    out = []
    for a, b in cand:
        a, b = max(0, a), min(V, b)
        if b > a and all(b <= c or a >= d for c, d in out):
            out.append((a, b))
    return out


def _exact(shape, gen):
    return (torch.randint(-16, 17, shape, device=DEV, generator=gen, dtype=torch.int32).float() / 8).bfloat16()


@pytest.mark.parametrize("mode", ["bf16", "int8", "fp8_block", "fp8"])
@pytest.mark.parametrize("name,V,H", LLAMA + QWEN, ids=[n for n, _, _ in LLAMA + QWEN])
def test_full_size_rows_against_oracle(name, V, H, mode):
    gen = torch.Generator(device=DEV).manual_seed(V * 31 + H)
    dy, x = _exact((BT, V), gen), _exact((BT, H), gen)
    w = (torch.randn(V, H, device=DEV, generator=gen) * 0.02).bfloat16()
    hp = oracle.Hyper(**ADAMW)
    if mode == "bf16":
        m = (torch.randn(V, H, device=DEV, generator=gen) * 0.05).bfloat16()
        v = (torch.randn(V, H, device=DEV, generator=gen).abs() * 0.05).bfloat16()
        state = (m, v)
    elif mode in ("int8", "fp8_block"):
        if mode == "int8":
            mq = torch.randint(-127, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
            vq = torch.randint(0, 128, (V, H), device=DEV, generator=gen, dtype=torch.int8)
        else:   # e4m3 codes: any finite code for m (0x7f / 0xff are NaN), non-negative for v
            mq = torch.randint(0, 127, (V, H), device=DEV, generator=gen, dtype=torch.uint8)
            mq = mq | (torch.randint(0, 2, (V, H), device=DEV, generator=gen, dtype=torch.uint8) << 7)
            vq = torch.randint(0, 127, (V, H), device=DEV, generator=gen, dtype=torch.uint8)
        ms = torch.rand(V, H // 64, device=DEV, generator=gen) * 0.05 + 1e-3
        vs = torch.rand(V, H // 64, device=DEV, generator=gen) * 0.5 + 1e-2
        state = (mq, vq, ms, vs)
    else:
        m8 = torch.randint(0, 127, (V, H), device=DEV, generator=gen, dtype=torch.uint8)
        m8 = m8 | (torch.randint(0, 2, (V, H), device=DEV, generator=gen, dtype=torch.uint8) << 7)
        v8 = torch.randint(0, 124, (V, H), device=DEV, generator=gen, dtype=torch.uint8)   # finite e5m2, non-negative
        s_m, s_v = np.float32(0.02), np.float32(6e-4)

        class St:
            pass
        st = St()
        st.m_fp8, st.v_fp8 = m8.view(torch.float8_e4m3fn), v8.view(torch.float8_e5m2)
        st.m_scale, st.v_scale = torch.tensor(float(s_m), device=DEV), torch.tensor(float(s_v), device=DEV)
        st.m_absmax_next, st.v_absmax_next = torch.zeros((), device=DEV), torch.zeros((), device=DEV)
        state = (m8, v8)

    slices = _row_slices(V)
    before = [(a, b, w[a:b].clone(), [t[a:b].clone() for t in state]) for a, b in slices]
    if mode == "bf16":
        K.fused_grad_adamw(dy, x, w, *state, **ADAMW)
    elif mode == "int8":
        K.fused_grad_adamw_int8state(dy, x, w, *state, qblock=64, **ADAMW)
    elif mode == "fp8_block":
        K.fused_grad_adamw_fp8block(dy, x, w, *state, qblock=64, **ADAMW)
    else:
        K.fused_grad_adamw_fp8state(dy, x, w, st, **ADAMW)
    torch.cuda.synchronize()

    xn = np32(x)
    amax_seen = np.zeros(2, np.float32)
    for a, b, w_old, st_old in before:
        tag = f"{name} rows {a}:{b}"
        g = oracle.wgrad(np32(dy[:, a:b]), xn)
        wf = w_old.float().cpu()
        wn = np32(wf).copy()
        if mode == "bf16":
            mn, vn = np32(st_old[0]).copy(), np32(st_old[1]).copy()
            oracle.adamw(wn, mn, vn, g, hp, w_bf16=True, s_bf16=True)
            assert_bits_equal(mn, state[0][a:b], f"{tag} m")
            assert_bits_equal(vn, state[1][a:b], f"{tag} v")
        elif mode in ("int8", "fp8_block"):
            emq = st_old[0].cpu().numpy().copy()
            evq = st_old[1].cpu().numpy().copy()
            if mode == "fp8_block":
                emq, evq = emq.view(np.uint8), evq.view(np.uint8)
            ems, evs = np32(st_old[2]).copy(), np32(st_old[3]).copy()
            oracle.adamw_blockq(wn, emq, evq, ems, evs, g, hp, w_bf16=True, kind="int8" if mode == "int8" else "e4m3")
            assert_bits_equal(ems, state[2][a:b], f"{tag} m_scale")
            assert_bits_equal(evs, state[3][a:b], f"{tag} v_scale")
            assert_bits_equal(emq.view(np.uint8), state[0][a:b], f"{tag} m codes")
            assert_bits_equal(evq.view(np.uint8), state[1][a:b], f"{tag} v codes")
        else:
            em8, ev8 = st_old[0].cpu().numpy().copy(), st_old[1].cpu().numpy().copy()
            amax = np.zeros(2, np.float32)
            oracle.adamw_fp8tensor(wn, em8, ev8, s_m, s_v, amax, g, hp, w_bf16=True)
            amax_seen = np.maximum(amax_seen, amax)
            assert_bits_equal(em8, state[0][a:b], f"{tag} m codes")
            assert_bits_equal(ev8, state[1][a:b], f"{tag} v codes")
        assert_w_close(wn, w[a:b], wf, what=f"{tag} W")
        assert not torch.equal(w[a:b], w_old), f"{tag}: weight did not change"
    if mode == "fp8":
        # the running maxima cover the whole tensor: at least what the sampled rows produced
        assert st.m_absmax_next.item() >= amax_seen[0] and st.v_absmax_next.item() >= amax_seen[1]
        assert np.isfinite(st.m_absmax_next.item()) and np.isfinite(st.v_absmax_next.item())
