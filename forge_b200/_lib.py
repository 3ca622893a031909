"""ctypes binding of ``libforge_b200.so`` -- the C ABI declared in ``include/forge_b200.h``.

The library is the only compute path of this package: if it is missing or fails to load, every
operator raises ``ForgeLibraryError``; there is no PyTorch or CPU fallback.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libforge_b200.so")

# error codes (include/forge_b200.h)
FORGE_OK = 0
FORGE_ERR_INVALID_ARG = -1
FORGE_ERR_ALIGNMENT = -2
FORGE_ERR_SHAPE = -3
FORGE_ERR_UNSUPPORTED = -4
FORGE_ERR_CUDA = -5
FORGE_ERR_DEVICE = -6
FORGE_ERR_TIMEOUT = -7
FORGE_ERR_SCRATCH = -8

DT_BF16, DT_F32 = 0, 1
OPT_ADAMW, OPT_SGD, OPT_SGDM, OPT_LION = 0, 1, 2, 3
ST_NONE, ST_F32, ST_BF16, ST_INT8, ST_FP8_BLOCK, ST_FP8_TENSOR = 0, 1, 2, 3, 4, 5

OPTIMIZER_IDS = {"adamw": OPT_ADAMW, "sgd": OPT_SGD, "sgdm": OPT_SGDM, "lion": OPT_LION}


class ForgeLibraryError(RuntimeError):
    """The native library is missing, could not be loaded, or reported a runtime failure."""


class ForgeHyper(ctypes.Structure):
    _fields_ = [
        ("lr", ctypes.c_double),
        ("beta1", ctypes.c_double),
        ("beta2", ctypes.c_double),
        ("eps", ctypes.c_double),
        ("weight_decay", ctypes.c_double),
        ("momentum", ctypes.c_double),
        ("nesterov", ctypes.c_int32),
        ("step", ctypes.c_int32),
    ]


class ForgeState(ctypes.Structure):
    _fields_ = [
        ("mode", ctypes.c_int32),
        ("qblock", ctypes.c_int32),
        ("m", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("ld_state", ctypes.c_int64),
        ("m_scale", ctypes.c_void_p),
        ("v_scale", ctypes.c_void_p),
        ("ld_scale", ctypes.c_int64),
        ("m_absmax_next", ctypes.c_void_p),
        ("v_absmax_next", ctypes.c_void_p),
    ]


class ForgeWgradArgs(ctypes.Structure):
    _fields_ = [
        ("dY", ctypes.c_void_p),
        ("X", ctypes.c_void_p),
        ("W", ctypes.c_void_p),
        ("BT", ctypes.c_int64),
        ("V", ctypes.c_int64),
        ("H", ctypes.c_int64),
        ("ld_dy", ctypes.c_int64),
        ("ld_x", ctypes.c_int64),
        ("ld_w", ctypes.c_int64),
        ("operand_dtype", ctypes.c_int32),
        ("w_dtype", ctypes.c_int32),
        ("optimizer", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("state", ForgeState),
        ("hyper", ForgeHyper),
        ("scratch", ctypes.c_void_p),
        ("scratch_bytes", ctypes.c_size_t),
        ("status", ctypes.c_void_p),
        ("hyper_device", ctypes.c_void_p),
    ]


class ForgeDgradSegment(ctypes.Structure):
    _fields_ = [("dY", ctypes.c_void_p), ("W", ctypes.c_void_p), ("V", ctypes.c_int64), ("ld_dy", ctypes.c_int64),
                ("ld_w", ctypes.c_int64)]


class ForgeDgradScatterArgs(ctypes.Structure):
    _fields_ = [("segments", ctypes.POINTER(ForgeDgradSegment)), ("count", ctypes.c_int32), ("BT", ctypes.c_int64),
                ("H", ctypes.c_int64), ("slots", ctypes.POINTER(ctypes.c_void_p)),
                ("arrivals", ctypes.POINTER(ctypes.c_void_p)), ("counter", ctypes.c_void_p), ("epoch", ctypes.c_void_p),
                ("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("status", ctypes.c_void_p),
                ("all_ranks", ctypes.c_int32)]


class ForgeLinearGatheredArgs(ctypes.Structure):
    _fields_ = [("X", ctypes.c_void_p), ("W", ctypes.c_void_p), ("BT", ctypes.c_int64), ("H", ctypes.c_int64),
                ("V_r", ctypes.c_int64), ("ld_x", ctypes.c_int64), ("ld_w", ctypes.c_int64),
                ("x_arrivals", ctypes.c_void_p), ("epoch", ctypes.c_void_p), ("rank", ctypes.c_int32),
                ("world", ctypes.c_int32), ("y", ctypes.c_void_p), ("ld_y", ctypes.c_int64),
                ("y_dst", ctypes.POINTER(ctypes.c_void_p)), ("y_col", ctypes.c_int64), ("y_pitch", ctypes.c_int64),
                ("y_arrivals", ctypes.POINTER(ctypes.c_void_p)), ("y_counter", ctypes.c_void_p),
                ("status", ctypes.c_void_p)]


class ForgeOptimArgs(ctypes.Structure):
    _fields_ = [
        ("grad", ctypes.c_void_p),
        ("W", ctypes.c_void_p),
        ("V", ctypes.c_int64),
        ("H", ctypes.c_int64),
        ("ld_grad", ctypes.c_int64),
        ("ld_w", ctypes.c_int64),
        ("grad_dtype", ctypes.c_int32),
        ("w_dtype", ctypes.c_int32),
        ("optimizer", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("state", ForgeState),
        ("hyper", ForgeHyper),
    ]


# every symbol include/forge_b200.h declares, with its ctypes signature
_SIGNATURES = {
    "forge_wgrad_update": (ctypes.c_int, [ctypes.POINTER(ForgeWgradArgs), ctypes.c_void_p]),
    "forge_wgrad_update_group": (ctypes.c_int, [ctypes.POINTER(ForgeWgradArgs), ctypes.c_int32, ctypes.c_void_p]),
    "forge_wgrad_update_static_scratch": (ctypes.c_int, [ctypes.POINTER(ForgeWgradArgs), ctypes.c_void_p]),
    "forge_hyper_pack": (ctypes.c_int, [ctypes.POINTER(ForgeHyper), ctypes.c_void_p]),
    "forge_wgrad_scratch_bytes": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32]),
    "forge_optimizer_update": (ctypes.c_int, [ctypes.POINTER(ForgeOptimArgs), ctypes.c_void_p]),
    "forge_fp8_prestep": (ctypes.c_int, [ctypes.c_void_p] * 5),
    "forge_dgrad": (ctypes.c_int, [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 6 + [ctypes.c_void_p] * 2),
    "forge_dgrad_sum": (ctypes.c_int, [ctypes.POINTER(ForgeDgradSegment), ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]),
    "forge_dgrad_scatter": (ctypes.c_int, [ctypes.POINTER(ForgeDgradScatterArgs), ctypes.c_void_p]),
    "forge_reduce_slots": (ctypes.c_int, [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 3 + [ctypes.c_int32, ctypes.c_void_p,
                                                                                        ctypes.c_void_p]),
    "forge_set_arrival_wait_ns": (ctypes.c_int, [ctypes.c_uint64]),
    "forge_push_block": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_int64,
                                        ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]),
    "forge_linear_gathered": (ctypes.c_int, [ctypes.POINTER(ForgeLinearGatheredArgs), ctypes.c_void_p]),
    "forge_collect": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p,
                                     ctypes.c_void_p]),
    "forge_rmsnorm_forward": (ctypes.c_int, [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 4 + [ctypes.c_double, ctypes.c_void_p]),
    "forge_rmsnorm_backward": (ctypes.c_int, [ctypes.c_void_p] * 5 + [ctypes.c_int32] * 2 + [ctypes.c_int64] * 5
                               + [ctypes.c_double, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "forge_rmsnorm_backward_scratch_bytes": (ctypes.c_size_t, [ctypes.c_int64, ctypes.c_int64]),
    "forge_state_bytes": (
        ctypes.c_int,
        [ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
         ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_int32)],
    ),
    "forge_read_status": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.c_void_p]),
    "forge_selftest_wait_timeout": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]),
    "forge_last_error_string": (ctypes.c_char_p, []),
    "forge_abi_version": (ctypes.c_int, []),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None
_lib_lock = threading.Lock()


def load():
    """Load the shared library once and attach signatures. Raises ForgeLibraryError if absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ForgeLibraryError(
                f"{LIB_PATH} not found: build it with `python -m forge_b200.build` "
                "(nvcc, sm_100a). forge_b200 has no fallback path."
            )
        try:
            lib = ctypes.CDLL(LIB_PATH)
        except OSError as e:  # pragma: no cover - depends on the host
            raise ForgeLibraryError(f"could not load {LIB_PATH}: {e}") from e
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().forge_last_error_string().decode("utf-8", "replace")


def check(rc: int, what: str):
    """Map a FORGE_ERR_* return code to the exception type the reference raises in that case."""
    if rc == FORGE_OK:
        return
    msg = f"{what}: {last_error()} (code {rc})"
    if rc in (FORGE_ERR_INVALID_ARG, FORGE_ERR_SHAPE, FORGE_ERR_UNSUPPORTED):
        raise ValueError(msg)
    raise ForgeLibraryError(msg)


def dtype_id(t: torch.dtype) -> int:
    if t == torch.bfloat16:
        return DT_BF16
    if t == torch.float32:
        return DT_F32
    raise ValueError(f"unsupported dtype {t}: forge_b200 handles bfloat16 and float32")


def state_mode_id(t: torch.dtype) -> int:
    if t == torch.bfloat16:
        return ST_BF16
    if t == torch.float32:
        return ST_F32
    raise ValueError(f"unsupported moment dtype {t}: use bfloat16 or float32 (or int8 / fp8 state modes)")


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# one status word per device, checked on demand (forge_read_status synchronises the stream)
_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def read_status(device: torch.device) -> int:
    """Synchronise the current stream and raise if a kernel abandoned a bounded wait."""
    lib = load()
    code = ctypes.c_int32(0)
    w = status_word(device)
    with torch.cuda.device(w.device):
        rc = lib.forge_read_status(w.data_ptr(), ctypes.byref(code), current_stream_ptr(w.device))
    check(rc, "forge_read_status")
    return code.value
