"""The optional C++ autograd node (``forge_b200/_forge_autograd.so``, built by
``python -m forge_b200.build`` from ``csrc_torch/forge_autograd.cpp``).

It replaces the Python ``FusedLinearFunction`` on the plain fused branch -- bf16 activations on CUDA,
an optimizer config set, no gradient accumulation pending -- so that a backward pass of ~225 fused
linears enters Python zero times; every other branch of the reference's table keeps the Python
function.  Counterpart of the reference's opt-in ``FUSED_LINEAR_CPP=1`` node
(``src/fused_grad_optimizer/module.py:127-133``, ``csrc/fused_linear_cpp/fused_linear.cpp``), which
still calls back into Python for the kernel; this one calls the C ABI directly.  Both nodes issue the
same library calls, so results are bit-identical.  ``FORGE_NATIVE_AUTOGRAD=0`` keeps the Python
function everywhere; a missing extension does the same (the CUDA library itself is never optional).
"""

from __future__ import annotations

import ctypes
import os

_mod = None
_tried = False


def module():
    """The extension module, or None when it is not built or switched off."""
    global _mod, _tried
    if not _tried:
        _tried = True
        if os.environ.get("FORGE_NATIVE_AUTOGRAD", "1") != "0":
            try:
                from forge_b200 import _forge_autograd as m
                from forge_b200._lib import ForgeWgradArgs
                if m.args_size() != ctypes.sizeof(ForgeWgradArgs):
                    raise ImportError("argument block layout mismatch between the extension and the ctypes binding")
                _mod = m
            except ImportError:
                _mod = None
    return _mod


def reset():
    """Forget the cached lookup (tests flip FORGE_NATIVE_AUTOGRAD)."""
    global _mod, _tried
    _mod, _tried = None, False
