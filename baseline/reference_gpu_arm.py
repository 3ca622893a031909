"""Times the reference's own default GPU kernel (``fused_grad_optimizer.kernel.fused_grad_adamw``, Triton) on
this GPU over one Llama-3.1-8B decoder layer's seven projections at BT = 512 (bf16 W, bf16 moments), as a
record beside ``bench.py --impl reference``'s CPU figure.  Runs in a process of its own because the reference
package and this repository's alias package share the import name; the reference comes from ``baseline/_ref``
(``pip install --target baseline/_ref <reference>``).  Prints one JSON object; on any failure the object says why.

    python baseline/reference_gpu_arm.py [--steps K] [--warmup W]
"""

import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "_ref"))

BT = 512
LAYER = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096), ("gate", 14336, 4096),
         ("up", 14336, 4096), ("down", 4096, 14336)]
HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    t_start = time.time()
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        import fused_grad_optimizer.kernel as RK
        if "_ref" not in RK.__file__:
            raise RuntimeError(f"imported {RK.__file__}, not the reference under baseline/_ref")
        dev = "cuda"
        g = torch.Generator(device=dev).manual_seed(0)
        layer = []
        for _, V, H in LAYER:
            w = (torch.randn(V, H, device=dev, generator=g) * 0.02).bfloat16()
            layer.append(((torch.randn(BT, V, device=dev, generator=g) * 1e-2).bfloat16(),
                          torch.randn(BT, H, device=dev, generator=g).bfloat16(), w, torch.zeros_like(w), torch.zeros_like(w)))

        def step(s):
            for dy, x, w, m, v in layer:
                RK.fused_grad_adamw(dy, x, w, m, v, step=s, **HYPER)

        for s in range(1, max(args.warmup, 3) + 1):       # the first call per shape autotunes
            step(s)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(args.steps):
            step(10 + s)
        e1.record()
        torch.cuda.synchronize()
        layer_ms = e0.elapsed_time(e1) / args.steps
        print(json.dumps({"layer_ms": layer_ms, "steps": args.steps, "params": sum(V * H for _, V, H in LAYER),
                          "kernel": "fused_grad_optimizer.kernel.fused_grad_adamw (reference, Triton)",
                          "wall_s": round(time.time() - t_start, 1)}))
    except Exception as e:  # pragma: no cover - depends on the box
        print(json.dumps({"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}))


if __name__ == "__main__":
    main()
