"""Benchmark of the fused weight-gradient + AdamW path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl forge|reference] [--workload NAME]

Workload (default ``llama3.1-8b-linears``): every linear of the Llama-3.1-8B architecture that the
reference fuses -- 32 decoder layers x (q 4096x4096, k 1024x4096, v 1024x4096, o 4096x4096,
gate 14336x4096, up 14336x4096, down 4096x14336) plus lm_head 128256x4096 -- at BT = 512 tokens,
bf16 weights and bf16 AdamW moments, random-initialised, synthetic activations X ~ N(0,1) and
gradients dY ~ N(0, 1e-2) in bf16.  A *step* is one fused wgrad+AdamW update of each of the 225
weights.  ``--group layer`` (default) issues the projections of two decoder layers (14 weights) as ONE
kernel launch (``forge_wgrad_update_group``: 17 launches per step; ``--layers-per-launch 1``: 33), ``--group x`` one launch per set of
linears that share their input (q/k/v, gate/up), ``--group none`` one launch per weight as the
reference does.  Every weight and its moments are distinct buffers (45 GB in total), so each launch
streams cold state; only the small X / dY panels may sit in L2, as they do in training where the
preceding kernel has just produced them.

``value``  ms per step with X / dY already resident in device memory (CUDA events around the K
           timed steps on the launching stream, max over ranks).
``e2e``    the same step through the public operator API with HOST inputs: every launch first copies
           its X and dY from pinned host memory, and each step ends with a device-to-host read of a
           status word and one updated weight.  At N > 1 a rank's host inputs are its feature shard of
           X and its rows' slice of dY (what the row-sharded mode hands a rank between linears); the
           full X is formed by the NCCL all-gather inside the timed step.
N > 1      row-sharded tensor parallelism: rank r owns rows [r V/N, (r+1) V/N) of every weight and
           moment and updates them from its dY slice and the full X.  The path itself has no exchange
           step: the forward pass has already all-gathered X (it needs it for Y = X W^T) and autograd
           saved the gathered tensor, so the backward's fused update is purely local; strong scaling.
           ``--gather-x`` re-gathers X by NCCL inside the timed step (once per group of linears that
           share it) for a design that saves the activation shards instead.  ``tp_step`` in the output
           line times what the mode runs around the path (dX GEMM, reduce-scatter, updates), with
           NCCL collectives and with the reduce-scatter fused into this library's dX GEMM.
``--impl reference``  the reference's own CPU-runnable path for this update -- torch autograd +
           ``torch.optim.AdamW`` on the host cores -- on a bounded sample (one decoder layer's seven
           projections), scaled to the full workload by parameter count.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BT = 512
HIDDEN, KV, FFN, VOCAB, LAYERS = 4096, 1024, 14336, 128256, 32
# name, V (out), H (in), group that shares one gathered X
LAYER_LINEARS = [("q", HIDDEN, HIDDEN, "attn_in"), ("k", KV, HIDDEN, "attn_in"), ("v", KV, HIDDEN, "attn_in"),
                 ("o", HIDDEN, HIDDEN, "attn_out"), ("gate", FFN, HIDDEN, "mlp_in"), ("up", FFN, HIDDEN, "mlp_in"),
                 ("down", HIDDEN, FFN, "mlp_out")]
HYPER = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01)


def workload_linears(name):
    if name == "llama3.1-8b-linears":
        lin = [(f"l{i}.{n}", V, H, f"l{i}.{g}") for i in range(LAYERS) for n, V, H, g in LAYER_LINEARS]
        lin.append(("lm_head", VOCAB, HIDDEN, "lm_head"))
        return lin
    if name == "llama3.1-8b-layer":   # one decoder layer: the seven projection shapes of Llama-3.1-8B
        return [(n, V, H, g) for n, V, H, g in LAYER_LINEARS]
    if name == "qwen3-32b-linears":   # Qwen3-32B: 64 layers, hidden 5120, 64/8 heads of 128, FFN 25600
        hid, qd, kv, ffn, vocab = 5120, 8192, 1024, 25600, 151936
        layer = [("q", qd, hid, "attn_in"), ("k", kv, hid, "attn_in"), ("v", kv, hid, "attn_in"), ("o", hid, qd, "attn_out"),
                 ("gate", ffn, hid, "mlp_in"), ("up", ffn, hid, "mlp_in"), ("down", hid, ffn, "mlp_out")]
        lin = [(f"l{i}.{n}", V, H, f"l{i}.{g}") for i in range(64) for n, V, H, g in layer]
        lin.append(("lm_head", vocab, hid, "lm_head"))
        return lin
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(V, H, bt=BT, state_bytes=6):
    """read W,m,v + write W,m,v + read X once + read dY once (bf16 W, bf16 moments)."""
    return 2 * state_bytes * V * H + 2 * bt * (V + H)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [t.strip() for t in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            busy = [s for s in sm if s >= 0.5 * max(sm)] or sm
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------------------
def run_reference(args):
    """torch autograd + torch.optim.AdamW on the host cores, one decoder layer per step."""
    import torch
    from oracle import torch_steps as T
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = workload_linears("llama3.1-8b-layer")
    full = workload_linears(args.workload)
    g = torch.Generator().manual_seed(0)
    layers = []
    for _, V, H, _ in sample:
        w = torch.randn(V, H, generator=g) * 0.02
        layers.append((T.TorchAdamWLinear(w, HYPER["lr"], (HYPER["beta1"], HYPER["beta2"]), HYPER["eps"], HYPER["weight_decay"]),
                       torch.randn(BT, H, generator=g).bfloat16(), (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()))
    steps = max(1, min(args.steps, 20))
    warmup = max(1, min(args.warmup, 3))

    def one_step():
        for lin, x, dy in layers:
            lin.step(x, dy)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    sample_ms = (time.perf_counter() - t0) * 1e3 / steps
    scale = sum(V * H for _, V, H, _ in full) / sum(V * H for _, V, H, _ in sample)
    value = sample_ms * scale
    desc = (f"one decoder layer (7 projections, {sum(V * H for _, V, H, _ in sample) / 1e6:.0f}M parameters), {steps} timed steps "
            f"at {sample_ms:.0f} ms each, scaled x{scale:.1f} by parameter count to the full workload")
    line = {
        "impl": "reference", "metric": "fused_wgrad_adamw_ms_per_step", "value": value, "unit": "ms/step",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": value, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "bt": BT, "state": "fp32 W/m/v on the host (torch.optim.AdamW)",
                   "reference_path": "torch autograd + torch.optim.AdamW on CPU"},
        "cpu_baseline": {"value": value, "unit": "ms/step", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "ms/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    gpu = reference_gpu_kernel(scale)
    if gpu is not None:
        line["reference_gpu_kernel"] = gpu
    print(json.dumps(line))


def reference_gpu_kernel(scale):
    """Beside the CPU figure: the reference's own default GPU kernel (Triton ``fused_grad_adamw``) timed on
    this box's GPU over one decoder layer and scaled like the CPU sample -- the kernel this library is
    written to beat.  Only where the installed reference (``baseline/_ref``) and a GPU are present; runs in
    a process of its own (the reference shares its import name with this repository's alias package)."""
    script = os.path.join(ROOT, "baseline", "reference_gpu_arm.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref")) or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return None
    try:
        out = subprocess.run([sys.executable, script, "--steps", "10", "--warmup", "3"], capture_output=True, text=True,
                             timeout=240)
        rec = json.loads(out.stdout.strip().splitlines()[-1])
    except Exception as e:  # noqa: BLE001 - the record is optional
        return {"unavailable": f"{type(e).__name__}: {str(e)[:120]}"}
    if "layer_ms" in rec:
        rec["value"] = rec["layer_ms"] * scale
        rec["unit"] = "ms/step"
        rec["sample"] = "one decoder layer's seven projections on the GPU, scaled by parameter count like the CPU sample"
    return rec


# ------------------------------------------------------------------------------------------------
def run_forge(args):
    import torch
    import torch.distributed as dist
    from forge_b200 import _lib
    from forge_b200 import kernel as K
    from forge_b200.tensor_parallel import all_gather_features, feature_range, row_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: forge_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    linears = workload_linears(args.workload)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    shard_world = args.shard_of if (world == 1 and args.shard_of > 1) else world   # see --shard-of

    # state: this rank's rows of every weight and moment
    params = []
    for name, V, H, grp in linears:
        r0, r1 = row_range(V, rank, shard_world)
        w = torch.empty(r1 - r0, H, dtype=torch.bfloat16, device=dev).normal_(0.0, 0.02, generator=gen)
        if args.moments in ("int8", "fp8_block"):   # codes 0, scales 1: the reference's initial state (state.py:108-117)
            code = torch.int8 if args.moments == "int8" else torch.float8_e4m3fn
            m = (torch.zeros(r1 - r0, H, dtype=code, device=dev), torch.ones(r1 - r0, H // 64, device=dev))
            v = (torch.zeros(r1 - r0, H, dtype=code, device=dev), torch.ones(r1 - r0, H // 64, device=dev))
        else:
            m = torch.zeros_like(w)
            v = torch.zeros_like(w)
        params.append((name, V, H, grp, r0, r1, w, m, v))

    # launches: lists of indices into `params` whose updates are issued together
    # decoder layers per launch: two (14 weights; the fixed cost of a launch is paid half as often, which is
    # worth 2 % on one GPU and 4 % at the shard sizes of eight ranks)
    lpl = min(2, args.layers_per_launch) if args.layers_per_launch > 0 else 2
    if args.group == "none":
        launches_idx = [[i] for i in range(len(params))]
    else:
        keyed: dict[str, list[int]] = {}
        for i, (name, V, H, grp, *_r) in enumerate(params):
            # "l17.q" -> decoder layer 17; the one-layer workload's bare names form one layer; lm_head stands alone
            if args.group == "x":
                key = grp
            elif "." in name:
                key = "l%d" % (int(name.split(".")[0][1:]) // lpl)
            else:
                key = "layer" if name != "lm_head" else name
            keyed.setdefault(key, []).append(i)
        # largest weights first inside a launch: the small ones fill the ragged end
        launches_idx = [sorted(ix, key=lambda i: -(params[i][5] - params[i][4]) * params[i][2]) for ix in keyed.values()]

    def update(dy, x, w, m, v):
        if args.moments == "int8":
            K.fused_grad_adamw_int8state(dy, x, w, m[0], v[0], m[1], v[1], hyper_device=hyper_dev)
        elif args.moments == "fp8_block":
            K.fused_grad_adamw_fp8block(dy, x, w, m[0], v[0], m[1], v[1], hyper_device=hyper_dev)
        else:
            K.fused_grad_adamw(dy, x, w, m, v, hyper_device=hyper_dev)

    # activations: one X per distinct in-features (feature shard when N > 1), one dY per distinct V_r
    x_full, x_shard, dys = {}, {}, {}
    for name, V, H, grp, r0, r1, *_ in params:
        if H not in x_full:
            full = torch.randn(BT, H, device=dev, generator=gen).bfloat16()
            x_full[H] = full
            if world > 1:
                c0, c1 = feature_range(H, rank, world)
                x_shard[H] = full[:, c0:c1].contiguous()
        if (r1 - r0) not in dys:
            dys[r1 - r0] = (torch.randn(BT, r1 - r0, device=dev, generator=gen) * 1e-2).bfloat16()

    # host copies for the end-to-end arm
    pin = {}

    def pinned(t):
        key = (tuple(t.shape), t.data_ptr())
        if key not in pin:
            pin[key] = t.cpu().pin_memory()
        return pin[key]

    hyper_dev = K.DeviceHyper(dev)

    def set_step(step_no):
        """New bias corrections for this step: 64 bytes packed on the host and copied to the device
        block the kernels read (enqueued on the stream ahead of the step, captured or not)."""
        hyper_dev.update(step=step_no, **HYPER)

    # The 225 updates of a step are independent of each other (each touches its own W, m, v), so they
    # are spread round-robin over a few streams: a kernel that does not fill the GPU (the last wave of
    # a large projection, the small k / v projections, every shard in the row-sharded mode) overlaps
    # with its neighbours.  Under graph capture the streams become parallel branches of the graph.
    n_streams = max(1, args.streams)
    side_streams = [torch.cuda.Stream() for _ in range(n_streams - 1)]
    do_gather = world > 1 and args.gather_x
    # End-to-end arm at N > 1: a rank's host inputs are what the row-sharded mode hands it between linears --
    # its feature shard of X and its slice of dY; the full X is formed by the NCCL all-gather inside the
    # timed step (uploading the full X on every rank would measure the host's memory system N times over).
    e2e_gather = world > 1
    comm_stream = torch.cuda.Stream() if do_gather else None

    def step_device(step_no=None):
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        lanes = [main] + side_streams
        for st in side_streams:
            st.wait_event(start)
        # row-sharded mode: the gathers run on their own stream, ahead of the updates that use them
        gathered = {}
        if do_gather:
            comm_stream.wait_event(start)
            last_grp = None
            for name, V, H, grp, *_ in params:
                if grp != last_grp:
                    with torch.cuda.stream(comm_stream):
                        xg = all_gather_features(x_shard[H])     # NCCL, lands in local memory
                        ev = torch.cuda.Event()
                        ev.record(comm_stream)
                    gathered[grp] = (xg, ev)
                    last_grp = grp
        for li, members in enumerate(launches_idx):
            st = lanes[li % n_streams]
            with torch.cuda.stream(st), K.UpdateGroup():
                for i in members:
                    name, V, H, grp, r0, r1, w, m, v = params[i]
                    if do_gather:
                        x, ev = gathered[grp]
                        st.wait_event(ev)
                    else:
                        x = x_full[H]
                    update(dys[r1 - r0], x, w, m, v)
        for st in side_streams + ([comm_stream] if do_gather else []):
            done = torch.cuda.Event()
            done.record(st)
            main.wait_event(done)

    stage = {}

    def staged(t, tag):
        key = (tag, tuple(t.shape), t.dtype)
        if key not in stage:
            stage[key] = torch.empty_like(t)
        return stage[key]

    host_result = torch.zeros(2, dtype=torch.float32).pin_memory()

    copy_stream = torch.cuda.Stream()
    last_use = {}     # staging buffer -> event after the kernel that last read it

    def step_host(step_no=None, sync=True):
        """Same step, inputs start in pinned host memory; returns H2D / D2H bytes moved.  The copies of
        launch i+1 run on a second stream while launch i computes (two staging sets per shape)."""
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        copy_stream.wait_event(start)     # orders this step's copies after the previous step's kernels
        last_use.clear()
        h2d = 0

        def upload(src_dev, tag, slot):
            nonlocal h2d
            src_h = pinned(src_dev)
            dst = staged(src_dev, (tag, slot))
            with torch.cuda.stream(copy_stream):
                ev = last_use.get(dst.data_ptr())
                if ev is not None:
                    copy_stream.wait_event(ev)
                dst.copy_(src_h, non_blocking=True)
            h2d += src_h.numel() * 2
            return dst

        # Linears of one group (q/k/v; gate/up) consume the same activation: X is uploaded once per
        # group, into staging sets that alternate per group; every linear uploads its own dY.
        # two staging sets, alternating per launch; inside a launch every member has buffers of its own
        for li, members in enumerate(launches_idx):
            slot = li & 1
            staged_in, x_by_grp = [], {}
            for k, i in enumerate(members):
                name, V, H, grp, r0, r1, w, m, v = params[i]
                dy_d = upload(dys[r1 - r0], ("dy", k), slot)
                if grp not in x_by_grp:
                    x_by_grp[grp] = upload(x_shard[H] if e2e_gather else x_full[H], ("x", len(x_by_grp)), slot)
                staged_in.append((dy_d, x_by_grp[grp]))
            ready = torch.cuda.Event()
            ready.record(copy_stream)
            main.wait_event(ready)
            gathered_x = {g: all_gather_features(t) for g, t in x_by_grp.items()} if e2e_gather else x_by_grp
            with K.UpdateGroup():
                for (dy_d, _xd), i in zip(staged_in, members):
                    name, V, H, grp, r0, r1, w, m, v = params[i]
                    update(dy_d, gathered_x[grp], w, m, v)
            done = torch.cuda.Event()
            done.record(main)
            for dy_d, xd in staged_in:
                last_use[dy_d.data_ptr()] = done
                last_use[xd.data_ptr()] = done
        # the step's result: the device status word and one updated weight, read back to the host
        host_result[0:1].copy_(_lib.status_word(dev)[0:1].float(), non_blocking=True)
        host_result[1:2].copy_(params[-1][6][0, 0:1].float(), non_blocking=True)
        join = torch.cuda.Event()
        join.record(copy_stream)
        main.wait_event(join)
        if sync:
            main.synchronize()
        return h2d, 8

    # ---------------------------------------------------------------- the sharded mode's whole linear backward
    # What a row-sharded layer really runs in its backward, per set of linears that share an input
    # (q/k/v, o, gate/up, down, lm_head): the partial dX = sum_members dY_r W_r (library GEMM or
    # forge_dgrad) and its reduce-scatter over the ranks by NCCL on a communication stream; the fused
    # updates are recorded as the sets go by and issued once per launch group (two decoder layers), as
    # FusedOptimizerManager.group_updates does in training.  `regather` adds the all-gather of X for a
    # design that keeps only activation shards between forward and backward.  At N = 1 the collectives
    # vanish.
    from forge_b200.autograd import _grad_input
    from forge_b200.tensor_parallel import reduce_scatter_features
    x_groups = []
    for i, (name, V, H, grp, *_r) in enumerate(params):
        if x_groups and x_groups[-1][0] == grp:
            x_groups[-1][1].append(i)
        else:
            x_groups.append((grp, [i]))
    tp_comm = torch.cuda.Stream()
    dx_bufs = {}       # (H, slot) -> partial dX buffer; two per width so the next GEMM does not wait for the last scatter
    dx_free = {}       # buffer -> event after the collective that last read it

    # the same with the reduce-scatter fused into this library's dX GEMM (peer stores from the epilogue,
    # forge_b200/peer.py): built on first use, where every feature block is a multiple of 128 columns
    fused_rs = {}

    def get_fused_rs():
        if "rs" not in fused_rs:
            from forge_b200.peer import DgradReduceScatter
            fused_rs["rs"] = DgradReduceScatter([(BT, params[m[0]][2]) for _, m in x_groups], device=dev)
            fused_rs["tick"] = torch.zeros(1, device=dev)
        return fused_rs["rs"]

    def step_tp_fused(step_no=None):
        rs = get_fused_rs()
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        tp_comm.wait_event(start)
        rs.begin_step()
        if world > 1:
            # stands in for the collectives of the next forward pass: no rank overwrites a receive buffer
            # that another rank is still reading from the step before
            dist.all_reduce(fused_rs["tick"])
        pending = K.UpdateGroup()
        launch_of = {i: li for li, ix in enumerate(launches_idx) for i in ix}
        last_launch = None
        for gi, (grp, members) in enumerate(x_groups):
            if last_launch is not None and launch_of[members[0]] != last_launch:
                pending.flush()
            last_launch = launch_of[members[0]]
            H = params[members[0]][2]
            # the owner's wait-and-sum runs beside the next set's GEMM, like the NCCL reduce-scatter above
            rs.run(gi, [(dys[params[i][5] - params[i][4]], params[i][6]) for i in members], reduce_stream=tp_comm)
            with pending.record():
                for i in members:
                    name, V, _H, _g, r0, r1, w, m, v = params[i]
                    update(dys[r1 - r0], x_full[H], w, m, v)
        pending.flush()
        end = torch.cuda.Event()
        end.record(tp_comm)
        main.wait_event(end)

    def step_tp(step_no=None, parts=("dx", "rs", "update"), regather=False):
        main = torch.cuda.current_stream()
        start = torch.cuda.Event()
        start.record(main)
        tp_comm.wait_event(start)
        dx_free.clear()
        pending = K.UpdateGroup()
        waits = []            # gathers the recorded updates still have to wait for
        launch_of = {i: li for li, ix in enumerate(launches_idx) for i in ix}
        last_launch = None
        for gi, (grp, members) in enumerate(x_groups):
            if "update" in parts and last_launch is not None and launch_of[members[0]] != last_launch:
                for ev in waits:
                    main.wait_event(ev)
                waits.clear()
                pending.flush()
            last_launch = launch_of[members[0]]
            H = params[members[0]][2]
            x = x_full[H]
            if regather and world > 1:
                with torch.cuda.stream(tp_comm):
                    x = all_gather_features(x_shard[H])
                    ev_x = torch.cuda.Event()
                    ev_x.record(tp_comm)
            key = (H, gi & 1)
            if "dx" in parts or "rs" in parts:
                if key not in dx_bufs:
                    dx_bufs[key] = torch.empty(BT, H, dtype=torch.bfloat16, device=dev)
                dx = dx_bufs[key]
            if "dx" in parts:
                ev = dx_free.get(key)
                if ev is not None:
                    main.wait_event(ev)
                for k, i in enumerate(members):
                    name, V, _H, _g, r0, r1, w, m, v = params[i]
                    part = _grad_input(dys[r1 - r0], w)
                    if k == 0:
                        dx.copy_(part)
                    else:
                        dx.add_(part)
            if "rs" in parts and world > 1:
                ready = torch.cuda.Event()
                ready.record(main)
                tp_comm.wait_event(ready)
                with torch.cuda.stream(tp_comm):
                    reduce_scatter_features(dx)
                    done = torch.cuda.Event()
                    done.record(tp_comm)
                dx_free[key] = done
            if "update" in parts:
                if regather and world > 1:
                    waits.append(ev_x)
                with pending.record():
                    for i in members:
                        name, V, _H, _g, r0, r1, w, m, v = params[i]
                        update(dys[r1 - r0], x, w, m, v)
        if "update" in parts:
            for ev in waits:
                main.wait_event(ev)
            pending.flush()
        end = torch.cuda.Event()
        end.record(tp_comm)
        main.wait_event(end)

    def tp_parity_check():
        """One row-sharded linear trained for two steps with the real NCCL all-gather and reduce-scatter,
        per moment storage; the gathered weight must equal an unsharded FusedLinear's, bit for bit."""
        from forge_b200 import FusedLinear
        from forge_b200.tensor_parallel import RowShardedFusedLinear
        out = {}
        for mode in ("bf16", "int8", "fp8_block"):
            g = torch.Generator().manual_seed(77)
            bt, H, V = 128, 1024, 1288          # 161 groups of 8 rows: unequal shards at every world size
            w0 = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
            tp = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode=mode).train()
            full = FusedLinear(H, V, optimizer_type="adamw", state_mode=mode)
            full.weight.data = w0.clone()
            full = full.to(dev).to(torch.bfloat16).train()
            c0, c1 = feature_range(H, rank, world)
            for _ in range(2):
                x = torch.randn(bt, H, generator=g).bfloat16()
                gy = (torch.randn(bt, V, generator=g) * 1e-2).bfloat16()
                tp.local.update_optimizer_config(lr=1e-2, weight_decay=0.01)
                tp(x[:, c0:c1].to(dev).requires_grad_(True)).backward(gy[:, tp.row_start:tp.row_end].to(dev))
                full.update_optimizer_config(lr=1e-2, weight_decay=0.01)
                full(x.to(dev).requires_grad_(True)).backward(gy.to(dev))
            gathered = tp.gather_full_weight()
            nd = (gathered.view(torch.int16) != full.weight.detach().view(torch.int16)).sum().reshape(1)
            dist.all_reduce(nd, op=dist.ReduceOp.MAX)
            out[mode] = int(nd.item())
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(fn):
        """The step as a CUDA graph: 225 launches (+ gathers / copies) replayed with one call, the
        per-step hyper-parameters arriving through the device block.  Falls back to eager launches if
        capture is refused."""
        if args.eager:
            return None
        try:
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()                       # warm-up on the capture stream
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                fn()
            return g
        except Exception as e:  # pragma: no cover - depends on the driver / NCCL
            sys.stderr.write(f"[bench] graph capture failed ({type(e).__name__}: {e}); eager launches\n")
            torch.cuda.synchronize()
            return None

    def timed(fn, steps, first_step, graph=None, after=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        extra = None
        for s in range(steps):
            set_step(first_step + s)
            if graph is not None:
                graph.replay()
            else:
                extra = fn(first_step + s)
            if after is not None:
                after()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms, extra

    W = max(args.warmup, 3)
    step_no = 1
    set_step(step_no)
    step_device()                        # first launches set function attributes; never captured
    step_no += 1
    torch.cuda.synchronize()
    g_dev = capture(step_device)
    for _ in range(W):
        set_step(step_no)
        g_dev.replay() if g_dev is not None else step_device()
        step_no += 1
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    torch.cuda.nvtx.range_push("timed")          # lets a profiler select exactly the timed steps
    ms_dev, _ = timed(step_device, args.steps, step_no, graph=g_dev)
    torch.cuda.nvtx.range_pop()
    step_no += args.steps

    # end-to-end arm: host inputs copied in every step, result read back and waited for every step
    set_step(step_no)
    moved = step_host()
    step_no += 1
    g_e2e = capture(lambda: step_host(sync=False))
    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e, _ = timed(step_host, e2e_steps, step_no, graph=g_e2e,
                      after=(lambda: torch.cuda.current_stream().synchronize()) if g_e2e is not None else None)
    step_no += e2e_steps
    clocks = sampler.stop() if sampler else None

    # the sharded mode's full linear backward (see step_tp), and what each part costs alone
    tp_steps = max(1, min(args.steps, 5))
    tp_ms, tp_errors = {}, {}
    if not args.no_tp_step:
        variants = [("step", dict()), ("dx_gemm", dict(parts=("dx",))), ("update", dict(parts=("update",)))]
        if world > 1:
            variants += [("step_regather_x", dict(regather=True)), ("reduce_scatter", dict(parts=("rs",))),
                         ("all_gather_x", dict(parts=(), regather=True))]
        fused_ok = all(params[m[0]][2] % world == 0 and (params[m[0]][2] // world) % 128 == 0 and len(m) <= 4 for _, m in x_groups)
        if fused_ok:
            variants.append(("step_fused", None))
        for label, kw in variants:
            fn = step_tp_fused if kw is None else (lambda kw: (lambda step_no=None: step_tp(step_no, **kw)))(kw)
            # these records explain the mode around the path; none of them may cost the headline its line
            try:
                set_step(step_no)
                fn()
                g_tp = capture(fn)
                set_step(step_no)
                g_tp.replay() if g_tp is not None else fn()
                tp_ms[label], _ = timed(fn, tp_steps, step_no, graph=g_tp)
                del g_tp
            except Exception as e:  # noqa: BLE001
                tp_ms[label] = None
                tp_errors[label] = f"{type(e).__name__}: {e}"[:300]
        step_no += 1
    parity = None
    if world > 1:
        try:
            parity = tp_parity_check()
        except Exception as e:  # noqa: BLE001
            tp_errors["tp_parity"] = f"{type(e).__name__}: {e}"[:300]
    status = _lib.read_status(dev)

    peak_gb = torch.cuda.max_memory_allocated(dev) / 1e9
    if world > 1:
        t = torch.tensor([peak_gb], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        peak_gb = t.item()

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        launches = len(launches_idx)
        # algorithmic bytes this rank moves per step (row shard of the state, full X, dY slice)
        state_bytes = 6 if args.moments == "bf16" else 4 + 2 * 4 / 64   # per element: W + m + v (+ scales)
        alg = sum(algorithmic_bytes(r1 - r0, H, state_bytes=state_bytes) for _, V, H, _, r0, r1, *_ in params)
        achieved = alg / (ms_dev * 1e-3) / 1e9
        flops = sum(2 * BT * (r1 - r0) * H for _, V, H, _, r0, r1, *_ in params)
        line = {
            "metric": "fused_wgrad_adamw_ms_per_step", "value": ms_dev, "unit": "ms/step", "n_gpus": world,
            "steps": args.steps, "warmup": W, "ms_per_step": ms_dev, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "bt": BT, "linears": len(params), "launches_per_step": launches,
                       "grouping": args.group + (f" x{lpl}" if args.group == "layer" and lpl > 1 else ""), "weights": "bf16", "moments": args.moments,
                       "optimizer": "adamw", "launch": "cuda_graph" if g_dev is not None else "eager", "streams": n_streams,
                       "parallelism": (f"tp{world}-rows" + ("+gather-x" if do_gather else "")) if world > 1 else "single",
                       "l2": f"each weight and its moments are distinct buffers ({peak_gb:.0f} GB in total), so every launch "
                             "streams state that is not in L2; no flush needed",
                       "parameters": sum(V * H for _, V, H, *_ in params)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
                         "kernel": f"forge_wgrad_kernel<bf16 W, {args.moments} moments, AdamW>",
                         "algorithmic_bytes_per_launch": alg / launches, "avg_launch_us": ms_dev * 1e3 / launches,
                         "tflops": flops / (ms_dev * 1e-3) / 1e12,
                         # dram read+write per launch from the ncu capture in profiles/, scaled by bytes
                         "traffic": TRAFFIC_RATIO * alg / launches if (TRAFFIC_RATIO and args.moments == "bf16") else None,
                         "traffic_source": "ncu capture of one grouped decoder-layer launch (profiles/), scaled by algorithmic bytes"},
            "e2e": {"value": ms_e2e, "unit": "ms/step", "h2d_bytes_per_step": moved[0], "d2h_bytes_per_step": moved[1],
                    "steps": e2e_steps,
                    "inputs": ("per rank: its feature shard of X and its rows' slice of dY from pinned host memory; "
                               "X all-gathered by NCCL inside the step") if e2e_gather else
                              "X and dY of every linear from pinned host memory"},
            "gpu_launches": launches * args.steps,
            "peak_hbm_gb": peak_gb, "device_status": status, "clocks": clocks,
        }
        if tp_ms:
            n_rs = len(x_groups)
            act_full = sum(BT * params[m[0]][2] * 2 for _, m in x_groups)
            line["tp_step"] = {
                "what": "per set of linears sharing an input: partial dX GEMM and NCCL reduce-scatter of dX on a communication "
                        "stream; fused updates issued once per launch group; *_alone are the same parts timed by themselves",
                "ms": tp_ms.get("step"), "dx_gemm_alone_ms": tp_ms.get("dx_gemm"), "update_alone_ms": tp_ms.get("update"),
                "reduce_scatter_alone_ms": tp_ms.get("reduce_scatter"), "reduce_scatters_per_step": n_rs if world > 1 else 0,
                "ms_regather_x": tp_ms.get("step_regather_x"), "all_gather_x_alone_ms": tp_ms.get("all_gather_x"),
                "ms_fused_dx_reduce_scatter": tp_ms.get("step_fused"),
                "fused": "forge_dgrad_scatter + forge_reduce_slots: this library's dX GEMM stores its tiles into the owner "
                         "ranks' receive buffers over peer memory, no NCCL reduce-scatter",
                "dx_gemm": "forge_dgrad" if __import__("forge_b200.autograd", fromlist=["x"]).use_forge_dgrad else "cuBLAS",
                "saved_activation_bytes_per_rank": {"gathered_x": act_full, "x_shards": act_full // world},
                "steps": tp_steps, "launch": "cuda_graph" if not args.eager else "eager"}
        if tp_errors:
            line["tp_errors"] = tp_errors
        if parity is not None:
            line["tp_parity"] = "bit-equal" if not any(parity.values()) else f"{sum(parity.values())} differ"
            line["tp_parity_modes"] = parity
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line))
    if world > 1:
        # replayed graphs hold NCCL work: drop them and drain the device before tearing NCCL down, and do
        # not let a stuck finaliser keep the job alive after the result line is out
        sys.stdout.flush()
        del g_dev, g_e2e
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)


# dram bytes (read + write) inside the launches per algorithmic byte, from the ncu capture of one grouped
# decoder-layer launch summarised in profiles/wgrad_adamw_layer_group_llama8b_ncu.md (reads are slightly
# below the algorithmic reads because linears of a group share X in L2; the writes still dirty in L2
# when a launch ends make the in-launch total smaller than the algorithmic one)
TRAFFIC_RATIO = 0.97


def cpu_baseline(workload):
    """The oracle's torch restatement (torch autograd + torch.optim.AdamW, fp32) on the host cores:
    one decoder layer, a few steps, scaled by parameter count."""
    import torch
    from oracle import torch_steps as T
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample = workload_linears("llama3.1-8b-layer")
    full = workload_linears(workload)
    g = torch.Generator().manual_seed(0)
    layers = []
    for _, V, H, _ in sample:
        layers.append((T.TorchAdamWLinear(torch.randn(V, H, generator=g) * 0.02, HYPER["lr"],
                                          (HYPER["beta1"], HYPER["beta2"]), HYPER["eps"], HYPER["weight_decay"]),
                       torch.randn(BT, H, generator=g).bfloat16(), (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()))
    for lin, x, dy in layers:
        lin.step(x, dy)
    steps = 5
    t0 = time.perf_counter()
    for _ in range(steps):
        for lin, x, dy in layers:
            lin.step(x, dy)
    sample_ms = (time.perf_counter() - t0) * 1e3 / steps
    scale = sum(V * H for _, V, H, _ in full) / sum(V * H for _, V, H, _ in sample)
    return {"value": sample_ms * scale, "unit": "ms/step", "cores": cores, "kind": "port",
            "sample": f"torch autograd + torch.optim.AdamW (fp32) on one decoder layer's 7 projections, {steps} steps at "
                      f"{sample_ms:.0f} ms, scaled x{scale:.1f} by parameter count"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="forge", choices=["forge", "reference"])
    ap.add_argument("--workload", default="llama3.1-8b-linears")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--moments", default="bf16", choices=["bf16", "int8", "fp8_block"],
                    help="storage of the AdamW moments (int8 / fp8_block: codes + one fp32 absmax scale per row and 64 columns)")
    ap.add_argument("--group", default="layer", choices=["layer", "x", "none"],
                    help="weights per kernel launch: the projections of a decoder layer, the linears that share an input, or one")
    ap.add_argument("--layers-per-launch", type=int, default=0,
                    help="with --group layer: decoder layers per kernel launch (1 or 2; default 2)")
    ap.add_argument("--streams", type=int, default=4, help="streams the independent updates of a step are spread over")
    ap.add_argument("--gather-x", action="store_true",
                    help="N > 1: all-gather the feature-sharded X by NCCL inside the timed step")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="single-GPU diagnostic: give this GPU the row shard rank 0 would own in a job of this "
                         "many ranks (no communication), to time the kernels at shard sizes")
    ap.add_argument("--no-tp-step", action="store_true", help="skip the tp_step record (dX GEMM + collectives + update)")
    ap.add_argument("--eager", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_forge(args)


if __name__ == "__main__":
    main()
