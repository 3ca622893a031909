"""Whole-model training step with every ``nn.Linear`` fused (Llama-3.1-8B with bf16 or int8 moments,
Qwen3-32B with fp8 moments; batch 1 x 512 tokens).

Builds a Llama-3.1-8B (or Qwen3-32B) architecture from its config with random weights -- no
checkpoint, no dataset: tokens are uniform over the vocabulary -- swaps every ``nn.Linear`` for
``FusedLinear.from_linear`` (same recipe as the reference's README), leaves embeddings and norms to a
regular ``torch.optim.AdamW``, and reports the median step time and the peak device memory.

    python examples/llama_step.py --model llama3.1-8b --state bf16 --steps 20
    python examples/llama_step.py --model llama3.1-8b --baseline      # vanilla fused torch AdamW
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/llama_step.py \
        --model qwen3-32b --state fp8_block --tp 8                    # row-sharded over 8 GPUs (examples/tp_model.py)

One JSON line on stdout (rank 0), with the SM clocks sampled while the timed steps ran.
"""

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def build_config(name, layers=None):
    if name == "llama3.1-8b":
        from transformers import LlamaConfig
        cfg = LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                          num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5,
                          rope_theta=500000.0, max_position_embeddings=8192, tie_word_embeddings=False,
                          attention_bias=False, mlp_bias=False)
    elif name == "qwen3-32b":
        from transformers import Qwen3Config
        cfg = Qwen3Config(vocab_size=151936, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64,
                          num_attention_heads=64, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                          rope_theta=1000000.0, max_position_embeddings=40960, tie_word_embeddings=False,
                          attention_bias=False)
    else:
        raise SystemExit(f"unknown model {name}")
    if layers:
        cfg.num_hidden_layers = layers
    return cfg


def swap_linears(module, state_mode, use_dgrad):
    from forge_b200 import FusedLinear
    n = 0
    for name, child in list(module.named_children()):
        if isinstance(child, torch.nn.Linear):
            setattr(module, name, FusedLinear.from_linear(child, optimizer_type="adamw", state_mode=state_mode))
            n += 1
        else:
            n += swap_linears(child, state_mode, use_dgrad)
    return n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--state", default="bf16", choices=["bf16", "int8", "fp8", "fp8_block"])
    ap.add_argument("--baseline", action="store_true", help="plain nn.Linear + torch.optim.AdamW(fused=True)")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (debugging)")
    ap.add_argument("--forge-dgrad", action="store_true", help="dX through the library's GEMM instead of cuBLAS")
    ap.add_argument("--graph", action="store_true",
                    help="capture forward + backward (with the fused updates) + the small optimizer into one CUDA "
                         "graph and replay it; hyper-parameters reach the fused kernels through device memory")
    ap.add_argument("--fuse-norm", action="store_true",
                    help="single GPU: fold input_layernorm into q/k/v and post_attention_layernorm into gate/up "
                         "(FusedRMSNormLinear: the normalised activation is recomputed in backward, not saved)")
    ap.add_argument("--tp", type=int, default=0,
                    help="row-sharded tensor parallelism over this many ranks (launch with torch.distributed.run); "
                         "uses the decoder of examples/tp_model.py instead of the transformers model")
    ap.add_argument("--fused-scatter", action="store_true",
                    help="--tp: the input gradients of o and down through this library's dX GEMM with the reduce-scatter "
                         "fused into its epilogue (peer stores) instead of a library GEMM + NCCL reduce-scatter")
    ap.add_argument("--fused-gather", action="store_true",
                    help="--tp: the outputs of o and down through this library's forward GEMM with the all-gathers of "
                         "its input and of its output fused in (peer stores) instead of NCCL all-gathers around a library GEMM")
    ap.add_argument("--fused-scatter-sets", choices=("all", "gathered"), default="all",
                    help="--fused-scatter: 'gathered' keeps q/k/v and gate/up (replicated input) on library GEMMs + NCCL "
                         "all-reduce; 'all' also forms their input gradient with one GEMM launch per set whose tiles go to every rank")
    ap.add_argument("--torch-norm", action="store_true", help="--tp: RMSNorm as torch ops instead of the library's kernels")
    ap.add_argument("--no-group", action="store_true", help="one launch per linear instead of one per decoder layer")
    args = ap.parse_args()
    if args.tp:
        return run_tp(args)

    from bench import ClockSampler
    from transformers import AutoModelForCausalLM
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = build_config(args.model, args.layers)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(0)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16)
    model.train()
    model.config.use_cache = False
    n_params = sum(p.numel() for p in model.parameters())
    mem = {"parameters_gb": torch.cuda.memory_allocated(dev) / 1e9}

    if args.baseline:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True, capturable=args.graph)
        manager, fused = None, 0
    else:
        from forge_b200 import FusedOptimizerManager, autograd
        autograd.use_forge_dgrad = args.forge_dgrad
        fused = swap_linears(model, args.state, args.forge_dgrad)
        if args.fuse_norm:
            from forge_b200.rmsnorm_linear import fuse_rmsnorm_linear_pairs
            fuse_rmsnorm_linear_pairs(model, state_mode=args.state, weight_decay=0.01)
        manager = FusedOptimizerManager(model)
        if not args.no_group:
            manager.group_updates("layer")
        if args.graph:
            manager.enable_device_hyper(dev)
        opt = torch.optim.AdamW(manager.get_non_fused_params(), lr=1e-4, weight_decay=0.01, fused=True,
                                capturable=args.graph)

    torch.cuda.reset_peak_memory_stats(dev)
    times, losses = [], []
    static_ids = torch.zeros(1, args.seq, dtype=torch.long, device=dev)
    static_loss = torch.zeros((), device=dev)

    def one_step(ids):
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    graph = None
    # whole-network capture: the eager warm-up must not run on the legacy default stream, or autograd
    # later ties the captured backward to it
    side = torch.cuda.Stream() if args.graph else None
    if side is not None:
        side.wait_stream(torch.cuda.current_stream())
        torch.cuda.set_stream(side)
    sampler = ClockSampler(0)
    for step in range(args.warmup + args.steps):
        if step == args.warmup:
            sampler.start()
        g = torch.Generator(device=dev).manual_seed(1000 + step)
        ids = torch.randint(0, cfg.vocab_size, (1, args.seq), device=dev, generator=g)
        if args.graph and graph is None and step == 2:
            # two eager steps have allocated every state buffer; capture the third
            static_ids.copy_(ids)
            if manager is not None:
                manager.pre_step(lr=1e-4, weight_decay=0.01)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_loss.copy_(one_step(static_ids).detach())
            graph.replay()
            torch.cuda.synchronize()
            losses.append(static_loss.item())
            continue
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if manager is not None:
            manager.pre_step(lr=1e-4, weight_decay=0.01)
        if graph is not None:
            static_ids.copy_(ids)
            graph.replay()
            loss = static_loss
        else:
            loss = one_step(ids)
        torch.cuda.synchronize()
        if step >= args.warmup:
            times.append((time.perf_counter() - t0) * 1e3)
        losses.append(loss.item())
        if step == 0:      # parameters + every optimizer state, nothing of the step itself
            del loss
            mem["parameters_and_state_gb"] = torch.cuda.memory_allocated(dev) / 1e9
    clocks = sampler.stop()
    status = 0
    if manager is not None:
        from forge_b200 import _lib
        status = _lib.read_status(dev)
    print(json.dumps({
        "clocks": clocks, "grouped_launches": manager is not None and not args.no_group,
        "model": args.model, "layers": cfg.num_hidden_layers, "parameters": n_params, "seq": args.seq, "batch": 1,
        "impl": "torch AdamW(fused=True) baseline" if args.baseline else f"forge_b200 fused linears ({args.state} moments)",
        "fused_linears": fused, "median_ms_per_step": statistics.median(times), "min_ms": min(times), "max_ms": max(times),
        "steps": args.steps, "peak_hbm_gb": torch.cuda.max_memory_allocated(dev) / 1e9, "memory": mem,
        "first_loss": losses[0], "last_loss": losses[-1], "device_status": status,
        "forge_dgrad": bool(args.forge_dgrad), "fuse_norm": bool(args.fuse_norm and not args.baseline),
        "cuda_graph": bool(args.graph), "data": "synthetic uniform tokens, random init",
    }))


def run_tp(args):
    """Whole-model step with every linear row-sharded over ``--tp`` ranks (one process per GPU)."""
    import torch.distributed as dist
    from bench import ClockSampler
    from examples.tp_model import CONFIGS, TPDecoder
    from forge_b200 import FusedOptimizerManager, _lib, autograd

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.tp:
        raise SystemExit(f"--tp {args.tp} needs {args.tp} ranks (torch.distributed.run --nproc-per-node {args.tp}); got {world}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    autograd.use_forge_dgrad = args.forge_dgrad
    cfg = dict(CONFIGS[args.model])
    if args.layers:
        cfg["layers"] = args.layers
    if args.torch_norm:
        from examples import tp_model
        tp_model.RMSNorm.library_kernels = False
    model = TPDecoder(cfg, state_mode=args.state, device=dev).train()
    if args.fused_scatter and world > 1:
        model.use_fused_scatter(args.seq, replicated_sets=args.fused_scatter_sets == "all")
    if args.fused_gather and world > 1:
        model.use_fused_gather(args.seq)
    manager = FusedOptimizerManager(model)
    if not args.no_group:
        manager.group_updates("layer")
    if args.graph:
        manager.enable_device_hyper(dev)
    opt = torch.optim.AdamW(manager.get_non_fused_params(), lr=1e-4, weight_decay=0.01, fused=True, capturable=args.graph)
    head_norms = model.head_sharded_norm_params()
    n_local = sum(p.numel() for p in model.parameters())
    n_sharded = sum(m.weight.numel() for m in manager._fused_modules)
    n_total = (n_local - n_sharded) + sum(m.in_features * m.out_features for m in model.modules()
                                          if m.__class__.__name__ == "RowShardedFusedLinear")

    def one_step(ids):
        loss = model(ids)
        loss.backward()
        for p in head_norms:                      # per-head norm weights: sums over heads that live on other ranks
            dist.all_reduce(p.grad)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    static_ids = torch.zeros(1, args.seq, dtype=torch.long, device=dev)
    static_loss = torch.zeros((), device=dev)
    graph = None
    side = torch.cuda.Stream() if args.graph else None
    if side is not None:
        side.wait_stream(torch.cuda.current_stream())
        torch.cuda.set_stream(side)
    torch.cuda.reset_peak_memory_stats(dev)
    times, losses = [], []
    sampler = ClockSampler(local) if rank == 0 else None
    for step in range(args.warmup + args.steps):
        if step == args.warmup and sampler:
            sampler.start()
        g = torch.Generator(device=dev).manual_seed(1000 + step)        # the same tokens on every rank
        ids = torch.randint(0, cfg["vocab"], (1, args.seq), device=dev, generator=g)
        if args.graph and graph is None and step == 2:
            static_ids.copy_(ids)
            manager.pre_step(lr=1e-4, weight_decay=0.01)
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    static_loss.copy_(one_step(static_ids).detach())
                    left = sum(g.pending() for g in manager._update_groups)
                    if left:     # an update outside the graph would never be replayed
                        raise RuntimeError(f"{left} fused updates were still waiting for their group at the end of the backward pass")
                graph.replay()
                torch.cuda.synchronize()
                losses.append(static_loss.item())
                continue
            except Exception as e:  # pragma: no cover - depends on the NCCL build
                sys.stderr.write(f"[tp] graph capture failed ({type(e).__name__}: {e}); eager steps\n")
                graph, args.graph = None, False
                torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        manager.pre_step(lr=1e-4, weight_decay=0.01)
        if graph is not None:
            static_ids.copy_(ids)
            graph.replay()
            loss = static_loss
        else:
            loss = one_step(ids)
        e1.record()
        torch.cuda.synchronize()
        if step >= args.warmup:
            times.append(e0.elapsed_time(e1))
        losses.append(loss.item())
    clocks = sampler.stop() if sampler else None
    status = _lib.read_status(dev)
    stats = torch.tensor([statistics.median(times), torch.cuda.max_memory_allocated(dev) / 1e9, float(status)], device=dev)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)            # slowest rank, largest footprint
    if rank == 0:
        ms = stats[0].item()
        print(json.dumps({
            "model": args.model, "layers": cfg["layers"], "parameters": n_total, "parameters_per_rank": n_local,
            "seq": args.seq, "batch": 1, "tp": world,
            "impl": f"forge_b200 row-sharded fused linears ({args.state} moments), " + (
                "NCCL all-gather / reduce-scatter" if not (args.fused_gather or args.fused_scatter) or world == 1 else
                "collectives of o / down" + (" and of q/k/v, gate/up" if args.fused_scatter and args.fused_scatter_sets == "all" else "")
                + " fused into this library's GEMMs (" + " + ".join(
                    n for n, on in (("forward gathers", args.fused_gather), ("backward scatters", args.fused_scatter)) if on)
                + "), NCCL for the rest"),
            "median_ms_per_step": ms, "tokens_per_s": args.seq / (ms * 1e-3), "steps": args.steps,
            "peak_hbm_gb_per_rank": stats[1].item(), "first_loss": losses[0], "last_loss": losses[-1],
            "device_status": int(stats[2].item()), "cuda_graph": bool(graph is not None),
            "grouped_launches": not args.no_group, "forge_dgrad": bool(args.forge_dgrad),
            "fused_scatter": (args.fused_scatter_sets if args.fused_scatter and world > 1 else False),
            "fused_gather": bool(args.fused_gather and world > 1), "library_rmsnorm": not args.torch_norm, "clocks": clocks,
            "timing": "CUDA events per step, median over steps, max over ranks",
            "data": "synthetic uniform tokens (same on every rank), random init"}))
    sys.stdout.flush()
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
