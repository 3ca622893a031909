"""Compile the CPU oracle (``forge_oracle.c``) into ``oracle/liboracle.so`` with gcc.

One IEEE rounding per operation is part of the oracle's definition, hence ``-ffp-contract=off`` and
no fast-math.  Test infrastructure: only tests/, ``__graft_entry__`` and bench.py's CPU baseline use it.
"""

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "forge_oracle.c")
OUT = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-shared", "-fPIC",
           "-o", OUT, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
