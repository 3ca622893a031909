"""forge_b200 -- B200 (sm_100a) implementation of the fused weight-gradient + optimizer path.

Public surface, same names as the reference package (``src/fused_grad_optimizer/__init__.py:14-18``):
``FusedLinear``, ``FusedOptimizerManager``, ``OptimizerConfig``, ``FusedOptimizerState``.  The
compute path is ``libforge_b200.so`` (hand-written CUDA behind a C ABI, see ``include/forge_b200.h``);
importing the package does not load it, the first operator call does and fails loudly if it is
missing.
"""

from forge_b200.module import FusedLinear, FusedOptimizerManager
from forge_b200.state import FusedOptimizerState, OptimizerConfig

__version__ = "0.1.0"
__all__ = ["FusedLinear", "FusedOptimizerManager", "OptimizerConfig", "FusedOptimizerState"]
# also here: forge_b200.rmsnorm_linear (FusedRMSNormLinear, fuse_rmsnorm_linear_pairs), forge_b200.tensor_parallel,
# forge_b200.kernel (operator wrappers, UpdateGroup)
