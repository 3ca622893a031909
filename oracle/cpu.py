"""numpy front end of ``liboracle.so`` (``forge_oracle.c``).  TEST INFRASTRUCTURE ONLY.

Arrays are numpy float32 (bf16 / fp8 values widened to fp32 where noted) and are updated in place,
mirroring the in-place contract of the operators under test.
"""

from __future__ import annotations

import ctypes
import os

import numpy as np

from oracle.build import build as _build

_LIB = None


class _CHyper(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float), ("bc1", ctypes.c_float),
                ("bc2", ctypes.c_float), ("momentum", ctypes.c_float), ("one_m_beta1", ctypes.c_float),
                ("one_m_beta2", ctypes.c_float), ("decay", ctypes.c_float), ("nesterov", ctypes.c_int)]


def _lib():
    global _LIB
    if _LIB is None:
        path = _build()
        lib = ctypes.CDLL(path)
        fp = ctypes.POINTER(ctypes.c_float)
        u8 = ctypes.POINTER(ctypes.c_uint8)
        hp = ctypes.POINTER(_CHyper)
        L = ctypes.c_long
        I = ctypes.c_int
        F = ctypes.c_float
        sigs = {
            "oracle_round_bf16": (F, [F]),
            "oracle_e4m3_to_float": (F, [ctypes.c_uint8]),
            "oracle_e5m2_to_float": (F, [ctypes.c_uint8]),
            "oracle_float_to_e4m3": (ctypes.c_uint8, [F]),
            "oracle_float_to_e5m2": (ctypes.c_uint8, [F]),
            "oracle_wgrad": (None, [fp, fp, L, L, L, fp]),
            "oracle_adamw": (None, [fp, fp, fp, fp, L, hp, I, I]),
            "oracle_sgd": (None, [fp, fp, L, hp, I]),
            "oracle_sgdm": (None, [fp, fp, fp, L, hp, I, I]),
            "oracle_lion": (None, [fp, fp, fp, L, hp, I, I]),
            "oracle_adamw_blockq": (None, [fp, u8, u8, fp, fp, fp, L, L, L, hp, I, I]),
            "oracle_adamw_fp8tensor": (None, [fp, u8, u8, F, F, fp, fp, fp, L, hp, I]),
            "oracle_fp8_prestep": (None, [fp, fp, fp, fp]),
            "oracle_int8_quantise": (None, [fp, L, L, L, u8, fp]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = lib
    return _LIB


class Hyper:
    """Hyper-parameters narrowed the way the reference's kernel arguments are: every scalar becomes
    fp32; ``bc = 1 - beta**step`` (``kernel.py:1367-1368``), ``1 - beta`` and ``1 - lr*wd`` are
    evaluated in Python double first and then narrowed."""

    def __init__(self, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1,
                 momentum=0.0, nesterov=False):
        self.c = _CHyper(lr, beta1, beta2, eps, weight_decay, 1.0 - beta1 ** step, 1.0 - beta2 ** step,
                         momentum, 1.0 - beta1, 1.0 - beta2, 1.0 - lr * weight_decay, int(bool(nesterov)))

    def ref(self):
        return ctypes.byref(self.c)


def _f32(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"], (a.dtype, a.flags)
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _u8(a: np.ndarray):
    assert a.dtype in (np.uint8, np.int8) and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8))


def round_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32, vectorised with integer arithmetic."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32).reshape(a.shape)


def wgrad(dy: np.ndarray, x: np.ndarray) -> np.ndarray:
    """g[v,h] = sum_bt dy[bt,v] x[bt,h] with fp32 accumulation in ascending bt."""
    BT, V = dy.shape
    H = x.shape[1]
    g = np.empty((V, H), dtype=np.float32)
    _lib().oracle_wgrad(_f32(dy), _f32(x), BT, V, H, _f32(g))
    return g


def adamw(w, m, v, g, hyper: Hyper, w_bf16=False, s_bf16=False):
    _lib().oracle_adamw(_f32(w), _f32(m), _f32(v), _f32(g), w.size, hyper.ref(), int(w_bf16), int(s_bf16))


def sgd(w, g, hyper: Hyper, w_bf16=False):
    _lib().oracle_sgd(_f32(w), _f32(g), w.size, hyper.ref(), int(w_bf16))


def sgdm(w, buf, g, hyper: Hyper, w_bf16=False, s_bf16=False):
    _lib().oracle_sgdm(_f32(w), _f32(buf), _f32(g), w.size, hyper.ref(), int(w_bf16), int(s_bf16))


def lion(w, m, g, hyper: Hyper, w_bf16=False, s_bf16=False):
    _lib().oracle_lion(_f32(w), _f32(m), _f32(g), w.size, hyper.ref(), int(w_bf16), int(s_bf16))


def adamw_blockq(w, mq, vq, ms, vs, g, hyper: Hyper, qblock=64, w_bf16=False, kind="int8"):
    """AdamW with block-quantised moments; ``mq``/``vq`` are int8 (kind="int8") or uint8 e4m3 codes
    (kind="e4m3"), ``ms``/``vs`` the (V, H // qblock) fp32 scales.  All updated in place."""
    V, H = w.shape
    assert qblock <= 256
    _lib().oracle_adamw_blockq(_f32(w), _u8(mq), _u8(vq), _f32(ms), _f32(vs), _f32(g), V, H, qblock,
                               hyper.ref(), int(w_bf16), 0 if kind == "int8" else 1)


def adamw_fp8tensor(w, m8, v8, s_m, s_v, amax, g, hyper: Hyper, w_bf16=False):
    """AdamW with e4m3 m / e5m2 v codes (uint8) and per-tensor scales; ``amax`` is a float32[2]
    array holding the running max |m'|, |v'| and is updated in place."""
    _lib().oracle_adamw_fp8tensor(_f32(w), _u8(m8), _u8(v8), float(s_m), float(s_v),
                                  _f32(amax[0:1]), _f32(amax[1:2]), _f32(g), w.size, hyper.ref(), int(w_bf16))


def fp8_prestep(scales: np.ndarray, amax: np.ndarray):
    """In place on float32[2] arrays (m, v): promote absmax to scale with the 2x ramp cap."""
    _lib().oracle_fp8_prestep(_f32(scales[0:1]), _f32(scales[1:2]), _f32(amax[0:1]), _f32(amax[1:2]))


def int8_quantise(x: np.ndarray, qblock=64):
    V, H = x.shape
    q = np.empty((V, H), dtype=np.int8)
    s = np.empty((V, H // qblock), dtype=np.float32)
    _lib().oracle_int8_quantise(_f32(x), V, H, qblock, _u8(q), _f32(s))
    return q, s


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    lib = _lib()
    lut = np.array([lib.oracle_e4m3_to_float(i) for i in range(256)], dtype=np.float32)
    return lut[codes.astype(np.uint8)]


def e5m2_decode(codes: np.ndarray) -> np.ndarray:
    lib = _lib()
    lut = np.array([lib.oracle_e5m2_to_float(i) for i in range(256)], dtype=np.float32)
    return lut[codes.astype(np.uint8)]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    lib = _lib()
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    return np.array([lib.oracle_float_to_e4m3(float(t)) for t in flat], dtype=np.uint8).reshape(x.shape)


def e5m2_encode(x: np.ndarray) -> np.ndarray:
    lib = _lib()
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    return np.array([lib.oracle_float_to_e5m2(float(t)) for t in flat], dtype=np.uint8).reshape(x.shape)
