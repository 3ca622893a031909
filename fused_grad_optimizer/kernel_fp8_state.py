"""Alias of the fp8-moment operators under the reference module name
(``src/fused_grad_optimizer/kernel_fp8_state.py``)."""

from forge_b200.kernel import (FP8_E4M3_MAX, FP8_E5M2_MAX, fused_grad_adamw_fp8state,  # noqa: F401
                               optimizer_only_adamw_fp8state)
