"""Build ``libforge_b200.so`` in-tree with nvcc for sm_100a.

    python -m forge_b200.build [--force] [--verbose]

Every ``csrc/*.cu`` is compiled to an object under ``build/`` (in parallel) with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into ``forge_b200/libforge_b200.so``.
No GPU is needed to build.  Objects are rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "forge_b200")
LIB = os.path.join(PKG, "libforge_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest_header_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(ROOT, "include", "forge_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_m = _newest_header_mtime()
    jobs = []
    objs = []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_m):
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    if jobs:
        with ThreadPoolExecutor(max_workers=min(4, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        run([_nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


TORCH_SRC = os.path.join(PKG, "csrc_torch", "forge_autograd.cpp")
TORCH_EXT = os.path.join(PKG, "_forge_autograd.so")


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    """Compile the C++ autograd node (``csrc_torch/forge_autograd.cpp``) against the installed PyTorch
    into ``forge_b200/_forge_autograd.so`` (g++, no GPU needed).  It links against ``libforge_b200.so``
    next to it, so ``build()`` must have run."""
    import torch
    from torch.utils import cpp_extension as C
    hdr = os.path.join(ROOT, "include", "forge_b200.h")
    if (not force and os.path.exists(TORCH_EXT)
            and os.path.getmtime(TORCH_EXT) >= max(os.path.getmtime(TORCH_SRC), os.path.getmtime(hdr), os.path.getmtime(LIB))):
        return TORCH_EXT
    import sysconfig
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [*C.include_paths(), sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=_forge_autograd",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in inc], TORCH_SRC, "-o", TORCH_EXT,
           *[f"-L{d}" for d in C.library_paths()], f"-L{PKG}", f"-L{os.path.join(cuda_home, 'lib64')}",
           "-l:libforge_b200.so", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python", "-lcudart",
           "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in C.library_paths()]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("g++ failed: " + " ".join(cmd))
    return TORCH_EXT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_torch_ext(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
