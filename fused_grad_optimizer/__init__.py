"""Import-name alias: code written against the reference package (``import fused_grad_optimizer``)
resolves to ``forge_b200`` without edits.  The submodules re-export the matching forge_b200 modules."""

from forge_b200 import (FusedLinear, FusedOptimizerManager, FusedOptimizerState, OptimizerConfig,
                        __version__)

__all__ = ["FusedLinear", "FusedOptimizerManager", "OptimizerConfig", "FusedOptimizerState"]
