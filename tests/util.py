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
