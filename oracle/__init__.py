"""CPU oracle of the fused weight-gradient + optimizer path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this package; the product (``forge_b200``) never does.  Two layers:

* ``forge_oracle.c`` (built by ``oracle/build.py``): scalar C restatement of the reference kernels'
  arithmetic, one IEEE rounding per operation -- the bit-level checker for the update, the int8
  quantiser and the fp8 codecs.
* ``torch_steps``: the reference's own PyTorch restatement of a step
  (``tests/test_correctness.py:27-55`` and ``:170-180``), run on CPU tensors -- the tolerance-level
  checker for whole steps and the timed CPU baseline.

Both are pinned by ``tests/golden`` against outputs of the reference's code run in the build
container (``tests/golden/make_golden.py``).
"""

from oracle.cpu import (Hyper, adamw, adamw_blockq, adamw_fp8tensor, e4m3_decode, e4m3_encode,  # noqa: F401
                        e5m2_decode, e5m2_encode, fp8_prestep, int8_quantise, lion, round_bf16, sgd,
                        sgdm, wgrad)
from oracle import torch_steps  # noqa: F401
