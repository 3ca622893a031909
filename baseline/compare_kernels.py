"""Side-by-side timing of the fused wgrad+AdamW kernel against the reference's own GPU kernels on the
same B200, per Llama-3.1-8B projection shape at BT = 512 (bf16 W, bf16 moments).

    python baseline/compare_kernels.py            # single GPU only

Arms (each skipped with a note if it cannot be loaded):
  forge        forge_b200.kernel.fused_grad_adamw (this repository)
  ref-triton   the reference's default kernel, ``fused_grad_optimizer.kernel.fused_grad_adamw``
               (persistent Triton kernel for >= 256 tiles, autotuned one below)
  ref-b200     the reference's B200 Triton kernel, ``kernel_b200_ws.fused_grad_adamw_b200_ws``
  ref-evt      the reference's CUTLASS Sm100 EVT kernel with its picker's default tile per shape
               (needs ``baseline/build_reference_evt.py`` to have been run)
  unfused      dW = dY^T X by cuBLAS, then ``torch._fused_adamw_`` (torch.optim.AdamW(fused=True))

The reference is imported from ``baseline/_ref`` (``pip install --target baseline/_ref <reference>``),
which must come first on ``sys.path`` because this repository ships an alias package of the same
import name.  Timing: CUDA events, median of 30, a 256 MB buffer written between iterations to flush L2;
every row carries the SM clocks sampled while it was timed (``time x median MHz`` compares runs taken
at different clocks).  One JSON object per shape on stdout, then ``--steps N`` (default 50) free-running
steps with int8 moments against the reference's own int8 kernel from the same fresh state.
"""

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(HERE, "_ref"))          # the reference's fused_grad_optimizer
sys.path.append(ROOT)                                   # forge_b200 (and, later in the path, the alias)

import torch  # noqa: E402

BT = 512
SHAPES = [("q/o", 4096, 4096), ("k/v", 1024, 4096), ("gate/up", 14336, 4096), ("down", 4096, 14336)]
HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)
HBM = 6460.2e9


def timeit(fn, flush, iters=30):
    for s in range(1, 4):
        fn(s)
    torch.cuda.synchronize()
    ts = []
    for it in range(iters):
        flush.fill_(it & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(4 + it)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def load_arms():
    arms, notes = {}, {}
    from forge_b200 import kernel as FK
    arms["forge"] = FK.fused_grad_adamw
    try:
        import fused_grad_optimizer.kernel as RK
        assert "_ref" in RK.__file__, RK.__file__
        arms["ref-triton"] = RK.fused_grad_adamw
    except Exception as e:  # pragma: no cover
        notes["ref-triton"] = f"{type(e).__name__}: {e}"
    try:
        from fused_grad_optimizer.kernel_b200_ws import fused_grad_adamw_b200_ws
        arms["ref-b200"] = fused_grad_adamw_b200_ws
    except Exception as e:  # pragma: no cover
        notes["ref-b200"] = f"{type(e).__name__}: {e}"
    try:
        sys.path.insert(0, os.path.join(HERE, "_ref", "evt", "build"))
        import ref_evt_sm100 as EVT
        from fused_grad_optimizer.cutlass_evt_b200 import _BT_HINT, _pick_tile

        def evt(go, inp, w, m, v, lr, beta1, beta2, eps, weight_decay, step):
            _BT_HINT["BT"] = go.shape[0]
            tile = _pick_tile(go.shape[1], inp.shape[1])
            fn = getattr(EVT, "blackwell_evt_adamw_" + tile)
            fn(go, inp, w, m, v, lr, beta1, beta2, eps, weight_decay, 1.0 - beta1 ** step, 1.0 - beta2 ** step)
        arms["ref-evt"] = evt
    except Exception as e:  # pragma: no cover
        notes["ref-evt"] = f"{type(e).__name__}: {e}"

    def unfused(go, inp, w, m, v, lr, beta1, beta2, eps, weight_decay, step):
        g = go.t() @ inp
        torch._fused_adamw_([w], [g], [m], [v], [], [unfused.step_t], amsgrad=False, lr=lr, beta1=beta1, beta2=beta2,
                            weight_decay=weight_decay, eps=eps, maximize=False)
    unfused.step_t = torch.tensor(3.0, device="cuda")
    arms["unfused"] = unfused
    return arms, notes


def int8_trajectory(steps):
    """``steps`` training steps with int8 moments, fresh Gaussian dY / X per step, from the reference's
    initial state (codes 0, scales 1): this library and the reference's Triton int8 kernel
    (``kernel.py:1487-1539``) side by side, no resynchronisation; agreement of W, codes and scales at
    the end (the Llama-3.1-8B int8 configuration asks for it over 50 steps)."""
    dev = "cuda"
    from forge_b200 import kernel as FK
    try:
        import fused_grad_optimizer.kernel as RK
        assert "_ref" in RK.__file__, RK.__file__
    except Exception as e:  # pragma: no cover
        print(json.dumps({"int8_trajectory": "unavailable", "why": f"{type(e).__name__}: {e}"}), flush=True)
        return
    for name, V, H in (("k/v", 1024, 4096), ("q/o", 4096, 4096)):
        g0 = torch.Generator(device=dev).manual_seed(3)
        w0 = (torch.randn(V, H, device=dev, generator=g0) * 0.02).bfloat16()

        def fresh():
            return (w0.clone(), torch.zeros(V, H, dtype=torch.int8, device=dev), torch.zeros(V, H, dtype=torch.int8, device=dev),
                    torch.ones(V, H // 64, device=dev), torch.ones(V, H // 64, device=dev))
        a, b = fresh(), fresh()
        for step in range(1, steps + 1):
            g = torch.Generator(device=dev).manual_seed(1000 + step)
            x = torch.randn(BT, H, device=dev, generator=g).bfloat16()
            dy = (torch.randn(BT, V, device=dev, generator=g) * 1e-2).bfloat16()
            FK.fused_grad_adamw_int8state(dy, x, *a, step=step, **HYPER)
            RK.fused_grad_adamw_int8state(dy, x, *b, step=step, **HYPER)
        torch.cuda.synchronize()
        row = {"int8_trajectory": name, "V": V, "H": H, "BT": BT, "steps": steps}
        dw = (a[0].float() - b[0].float()).abs()
        ulp = torch.pow(2.0, torch.floor(torch.log2(torch.maximum(a[0].float().abs(), b[0].float().abs()).clamp_min(2.0 ** -126))) - 7)
        row["W_max_abs_diff"] = float(dw.max())
        row["W_frac_beyond_one_bf16_ulp"] = float((dw > ulp).float().mean())
        for nm, i in (("m", 1), ("v", 2)):
            d = (a[i].int() - b[i].int()).abs()
            row[nm + "_codes_equal_frac"] = float((d == 0).float().mean())
            row[nm + "_codes_max_diff"] = int(d.max())
        row["m_scale_max_rel"] = float(((a[3] - b[3]).abs() / b[3].abs()).max())
        row["v_scale_max_rel"] = float(((a[4] - b[4]).abs() / b[4].abs()).max())
        row["note"] = ("the reference's kernel evaluates the update with Triton's approximate division / square root and "
                       "fused multiply-adds; this library rounds every moment operation separately (as the reference's "
                       "torch checker does) -- the codes differ where a quotient lands within that noise of .5")
        print(json.dumps(row), flush=True)


def main():
    import argparse
    from bench import ClockSampler
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50, help="free-running int8 steps against the reference's int8 kernel (0: skip)")
    ap.add_argument("--no-timing", action="store_true", help="only the int8 trajectory")
    args = ap.parse_args()
    dev = "cuda"
    if args.no_timing:
        int8_trajectory(args.steps)
        return
    arms, notes = load_arms()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for name, V, H in SHAPES:
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        g = torch.Generator(device=dev).manual_seed(0)
        dy = (torch.randn(BT, V, device=dev, generator=g) * 1e-2).bfloat16()
        x = torch.randn(BT, H, device=dev, generator=g).bfloat16()
        row = {"shape": name, "V": V, "H": H, "BT": BT}
        bytes_ = 12 * V * H + 2 * BT * (V + H)
        row["roofline_us"] = bytes_ / HBM * 1e6
        ref_w = None
        for arm, fn in arms.items():
            w = (torch.randn(V, H, device=dev, generator=torch.Generator(device=dev).manual_seed(1)) * 0.02).bfloat16()
            m, v = torch.zeros_like(w), torch.zeros_like(w)
            try:
                us = timeit(lambda s: fn(dy, x, w, m, v, step=s, **HYPER), flush)
                row[arm + "_us"] = round(us, 1)
                row[arm + "_frac"] = round(row["roofline_us"] / us, 3)
            except Exception as e:  # pragma: no cover
                row[arm + "_error"] = f"{type(e).__name__}: {str(e)[:160]}"
                torch.cuda.synchronize()
                continue
            # agreement after one step from identical state
            w1 = (torch.randn(V, H, device=dev, generator=torch.Generator(device=dev).manual_seed(1)) * 0.02).bfloat16()
            m1, v1 = torch.zeros_like(w1), torch.zeros_like(w1)
            fn(dy, x, w1, m1, v1, step=1, **HYPER)
            torch.cuda.synchronize()
            if arm == "forge":
                ref_w = (w1.float(), m1.float(), v1.float())
            elif ref_w is not None and arm != "unfused":
                row[arm + "_max_abs_dW_vs_forge"] = float((w1.float() - ref_w[0]).abs().max())
                row[arm + "_max_rel_dm_vs_forge"] = float(((m1.float() - ref_w[1]).abs() / (ref_w[1].abs() + 1e-6)).max())
        for k, vnote in notes.items():
            row[k + "_unavailable"] = vnote
        row["clocks"] = sampler.stop()
        print(json.dumps(row), flush=True)
        int8_row(name, V, H, dy, x, flush)
    if args.steps > 0:
        int8_trajectory(args.steps)


def int8_row(name, V, H, dy, x, flush):
    """int8 moments (codes + one fp32 scale per row and 64 columns): this library against the reference's
    own Triton kernel (``kernel.py:1487-1539``) from identical state -- time, and agreement of W, codes
    and scales after one step (the two sum the token axis in different orders, so a code may differ by
    one where x / scale sits within fp32 noise of a rounding boundary)."""
    dev = "cuda"
    from forge_b200 import kernel as FK
    row = {"shape": name, "V": V, "H": H, "BT": BT, "moments": "int8"}
    bytes_ = (2 * 4 + 2 * 2 * 4 / 64) * V * H + 2 * BT * (V + H)
    row["roofline_us"] = bytes_ / HBM * 1e6
    try:
        import fused_grad_optimizer.kernel as RK
        assert "_ref" in RK.__file__, RK.__file__
        arms = {"forge": FK.fused_grad_adamw_int8state, "ref-triton": RK.fused_grad_adamw_int8state}
    except Exception as e:  # pragma: no cover
        arms = {"forge": FK.fused_grad_adamw_int8state}
        row["ref-triton_unavailable"] = f"{type(e).__name__}: {e}"

    def fresh():
        g = torch.Generator(device=dev).manual_seed(2)
        w = (torch.randn(V, H, device=dev, generator=g) * 0.02).bfloat16()
        mq = torch.randint(-127, 128, (V, H), device=dev, generator=g, dtype=torch.int8)
        vq = torch.randint(0, 128, (V, H), device=dev, generator=g, dtype=torch.int8)
        ms = torch.rand(V, H // 64, device=dev, generator=g) * 1e-5 + 1e-6
        vs = torch.rand(V, H // 64, device=dev, generator=g) * 1e-9 + 1e-10
        return w, mq, vq, ms, vs

    outs = {}
    for arm, fn in arms.items():
        st = fresh()
        try:
            us = timeit(lambda s: fn(dy, x, *st, step=s, **HYPER), flush)
            row[arm + "_us"] = round(us, 1)
            row[arm + "_frac"] = round(row["roofline_us"] / us, 3)
            st = fresh()
            fn(dy, x, *st, step=5, **HYPER)
            torch.cuda.synchronize()
            outs[arm] = st
        except Exception as e:  # pragma: no cover
            row[arm + "_error"] = f"{type(e).__name__}: {str(e)[:160]}"
            torch.cuda.synchronize()
    if len(outs) == 2:
        a, b = outs["forge"], outs["ref-triton"]
        row["max_abs_dW"] = float((a[0].float() - b[0].float()).abs().max())
        for nm, i in (("m", 1), ("v", 2)):
            d = (a[i].int() - b[i].int()).abs()
            row[nm + "_codes_equal_frac"] = float((d == 0).float().mean())
            row[nm + "_codes_max_diff"] = int(d.max())
        row["m_scale_max_rel"] = float(((a[3] - b[3]).abs() / b[3].abs()).max())
        row["v_scale_max_rel"] = float(((a[4] - b[4]).abs() / b[4].abs()).max())
    print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
