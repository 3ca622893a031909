"""Build the reference's own Blackwell kernel (CUTLASS Sm100 EVT fused wgrad+AdamW,
``src/fused_grad_optimizer/csrc/cutlass_b200_evt/fused_adamw_evt_sm100.cu``) as a side-by-side
baseline.  Everything lands under ``baseline/_ref/`` (git-ignored): a copy of the source trimmed to
the three tile variants the reference's picker uses by default and that contain no cluster-broadcast
TMA load (``128x128_1sm``, ``256x128_2sm_etile128x64``, ``256x256_2sm_etile128x64``,
``cutlass_evt_b200.py:194-196``), compiled with the reference's own flags
(``cutlass_evt_b200.py:90-101``) against the CUTLASS headers shipped in the image.  Needs the
reference checkout (``REFERENCE_ROOT``); never loaded by the product, only by
``baseline/compare_kernels.py`` in single-GPU runs.
"""

import os
import re
import sys

REF = os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("set REFERENCE_ROOT to the reference checkout")
HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "evt")
KEEP = ("128x128_1sm", "256x128_2sm_etile128x64", "256x256_2sm_etile128x64")


def main():
    import torch
    from torch.utils.cpp_extension import load
    src = open(os.path.join(REF, "src", "fused_grad_optimizer", "csrc", "cutlass_b200_evt", "fused_adamw_evt_sm100.cu")).read()
    # drop the launchers and bindings of every other variant (unused `using` aliases cost nothing)
    src = "\n".join(l for l in src.split("\n")
                    if not (l.startswith("EVT_ADAMW_LAUNCHER(") and l.split("(")[1].split(",")[0].strip() not in KEEP))
    head, tail = src.split("PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {")
    defs = "".join(f'  mod.def("blackwell_evt_adamw_{k}", &blackwell_evt_adamw_{k}, "reference Sm100 EVT {k}");\n' for k in KEEP)
    src = head + "PYBIND11_MODULE(TORCH_EXTENSION_NAME, mod) {\n" + defs + "}\n"
    os.makedirs(os.path.join(OUT, "build"), exist_ok=True)
    cu = os.path.join(OUT, "fused_adamw_evt_sm100_trimmed.cu")
    open(cu, "w").write(src)
    site = os.path.dirname(os.path.dirname(torch.__file__))
    cutlass = os.environ.get("CUTLASS_PATH", os.path.join(site, "flashinfer", "data", "cutlass"))
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    load(name="ref_evt_sm100", sources=[cu], build_directory=os.path.join(OUT, "build"),
         extra_include_paths=[os.path.join(cutlass, "include"), os.path.join(cutlass, "tools", "util", "include")],
         extra_cuda_cflags=["-gencode=arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "--use_fast_math",
                            "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                            "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
                            "--expt-relaxed-constexpr", "--expt-extended-lambda",
                            "-DCUTLASS_ARCH_MMA_SM100_SUPPORTED=1", "--ftemplate-depth=2048"],
         verbose=True)
    print("built", os.path.join(OUT, "build"))


if __name__ == "__main__":
    sys.exit(main())
