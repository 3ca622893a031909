"""Helpers shared by the parity tests: seeded inputs, ULP distances, oracle drivers."""

from __future__ import annotations

import numpy as np
import torch

import oracle

ADAMW = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=5)


def gen_inputs(seed, BT, V, H, exact=False, dy_std=1e-2):
    """Seeded CPU tensors (fp32 values).  ``exact``: multiples of 1/8 in [-2, 2], for which every
    partial sum of dY^T X is exact in fp32, so the summation order of the device cannot matter."""
    g = torch.Generator().manual_seed(seed)
    if exact:
        dy = torch.randint(-16, 17, (BT, V), generator=g).float() / 8
        x = torch.randint(-16, 17, (BT, H), generator=g).float() / 8
    else:
        dy = torch.randn(BT, V, generator=g) * dy_std
        x = torch.randn(BT, H, generator=g)
    w = torch.randn(V, H, generator=g) * 0.02
    m = torch.randn(V, H, generator=g) * (0.05 if exact else 1e-3)
    v = torch.randn(V, H, generator=g).abs() * (0.05 if exact else 1e-5)
    return dy, x, w, m, v


def as_dtype(t: torch.Tensor, dtype):
    """Round a CPU fp32 tensor to `dtype`; returns (stored tensor, fp32 view of the stored values)."""
    s = t.to(dtype)
    return s, s.float()


def ordered_bf16(t: torch.Tensor) -> torch.Tensor:
    """bf16 tensor -> int32 keys that are monotonic in the represented value."""
    i = t.contiguous().view(torch.int16).int()
    return torch.where(i < 0, -(i & 0x7FFF), i)


def bf16_ulp_distance(expected_f32, actual: torch.Tensor) -> torch.Tensor:
    """Elementwise distance in bf16 ULPs between fp32 expected values (rounded to bf16) and a
    bf16 or fp32 tensor (fp32 is rounded to bf16 first)."""
    if isinstance(expected_f32, np.ndarray):
        expected_f32 = torch.from_numpy(expected_f32)
    e = ordered_bf16(expected_f32.float().bfloat16())
    a = ordered_bf16(actual.detach().cpu().float().bfloat16())
    return (e - a).abs()


def np32(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().float().numpy())


def oracle_adamw(dy, x, w, m, v, hp, w_bf16, s_bf16):
    """Oracle step on fp32-valued CPU tensors; returns numpy (w', m', v', g)."""
    g = oracle.wgrad(np32(dy), np32(x))
    wn, mn, vn = np32(w).copy(), np32(m).copy(), np32(v).copy()
    oracle.adamw(wn, mn, vn, g, oracle.Hyper(**hp), w_bf16=w_bf16, s_bf16=s_bf16)
    return wn, mn, vn, g


def assert_bits_equal(expected: np.ndarray, actual: torch.Tensor, what: str):
    a = actual.detach().cpu()
    if a.dtype == torch.bfloat16:
        e = torch.from_numpy(expected).bfloat16()
        assert torch.equal(e.view(torch.int16), a.view(torch.int16)), f"{what}: bf16 bits differ " \
            f"({(e.view(torch.int16) != a.view(torch.int16)).sum().item()} elements)"
    elif a.dtype == torch.float32:
        e = torch.from_numpy(expected)
        assert torch.equal(e.view(torch.int32), a.view(torch.int32)), f"{what}: fp32 bits differ " \
            f"({(e.view(torch.int32) != a.view(torch.int32)).sum().item()} elements, " \
            f"max abs {(e - a).abs().max().item():.3e})"
    else:
        e = torch.from_numpy(expected.view(np.uint8))
        av = a.view(torch.uint8)
        assert torch.equal(e, av), f"{what}: codes differ ({(e != av).sum().item()} elements)"


def bf16_ulp(x: torch.Tensor) -> torch.Tensor:
    """Size of one bf16 ULP at magnitude |x| (8 significand bits), with a floor at the smallest normal."""
    ax = x.abs().double().clamp_min(2.0 ** -126)
    return torch.pow(2.0, torch.floor(torch.log2(ax)) - 7)


def assert_one_ulp(expected, actual: torch.Tensor, scale, what: str, noise=4e-6):
    """|actual - expected| <= one bf16 ULP of the expected value + fp32 summation noise at the scale
    of the terms that were added (`scale`, tensor or float).  The ULP term covers a rounding that
    flips at a bf16 boundary; the noise term covers results that cancelled to far below their
    operands, where a distance counted in ULPs of the result is meaningless."""
    if isinstance(expected, np.ndarray):
        expected = torch.from_numpy(expected)
    e = expected.double()
    a = actual.detach().cpu().double()
    sc = scale.double().abs() if isinstance(scale, torch.Tensor) else torch.full_like(e, float(scale))
    # one ULP of whichever of the two values lies in the larger binade, plus the noise floor
    tol = torch.maximum(bf16_ulp(e), bf16_ulp(a)) + noise * sc
    bad = (a - e).abs() > tol
    assert not bad.any(), (f"{what}: {int(bad.sum())} elements beyond one bf16 ULP; worst "
                           f"{((a - e).abs() / tol).max().item():.2f}x the bound")


def assert_w_close(expected, actual: torch.Tensor, w_in: torch.Tensor, what="W"):
    """AdamW weight: within one bf16 ULP of the oracle (the device evaluates the bias-corrected
    quotient with approximate reciprocal / square root); fp32 weights additionally within fp32
    noise of the update."""
    if isinstance(expected, np.ndarray):
        expected = torch.from_numpy(expected)
    scale = w_in.detach().cpu().float().abs() + 1e-2
    assert_one_ulp(expected, actual, scale, what, noise=1e-6)
    if actual.dtype == torch.float32:
        d = (actual.detach().cpu().double() - expected.double()).abs()
        bound = 1e-7 + 1e-6 * w_in.detach().cpu().double().abs()
        assert (d <= bound).all(), f"{what}: fp32 weight off by {d.max().item():.3e}"
