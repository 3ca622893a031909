"""The row-sharded decoder of ``examples/tp_model.py`` on two gloo ranks (CPU) against the same
network unsharded: loss, the gradients of the replicated parameters (embedding, norms, per-head q / k
norms after their all-reduce) and every shard's weight gradient against the matching rows of the full
gradient.  Without an optimizer config the fused linears behave like plain linears, so no CUDA kernel
is involved; what is tested is the data flow -- which collective sits where, forward and backward --
and the vocabulary-parallel cross entropy."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

CFG = dict(vocab=96, hidden=32, ffn=64, layers=2, q_heads=4, kv_heads=2, head_dim=8, eps=1e-5, rope_theta=10000.0, qk_norm=True)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from examples.tp_model import TPDecoder
        from forge_b200.tensor_parallel import RowShardedFusedLinear
        solo = dist.new_group([rank])          # every rank builds the unsharded network in a group of its own
        for r in range(world):                 # (new_group is collective: all ranks create all groups)
            if r != rank:
                dist.new_group([r])
        torch.manual_seed(7)
        full = TPDecoder(CFG, group=solo, state_mode="bf16", dtype=torch.float32, device=torch.device("cpu"))
        torch.manual_seed(7)
        # same seed: make the full weights identical on both ranks
        for p in full.parameters():
            p.data = torch.randn(p.shape, generator=torch.Generator().manual_seed(p.numel() % 9973 + p.shape[0])) * 0.1
        tp = TPDecoder(CFG, group=None, state_mode="bf16", dtype=torch.float32, device=torch.device("cpu"))
        fm = dict(full.named_modules())
        for name, m in tp.named_modules():
            if isinstance(m, RowShardedFusedLinear):
                m.local.weight.data = fm[name].local.weight.data[m.row_start:m.row_end].clone()
        fp = dict(full.named_parameters())
        for name, p in tp.named_parameters():
            if ".local." not in name:
                p.data = fp[name].data.clone()
        full.train()
        tp.train()
        ids = torch.randint(0, CFG["vocab"], (2, 12), generator=torch.Generator().manual_seed(3))
        loss_f = full(ids)
        loss_f.backward()
        loss_t = tp(ids)
        loss_t.backward()
        for p in tp.head_sharded_norm_params():
            dist.all_reduce(p.grad)
        assert torch.allclose(loss_f, loss_t, rtol=1e-5, atol=1e-6), (loss_f.item(), loss_t.item())
        gp = dict(full.named_parameters())
        checked = 0
        for name, p in tp.named_parameters():
            ref = gp[name].grad
            if ".local." in name:
                m = dict(tp.named_modules())[name.rsplit(".local.", 1)[0]]
                ref = ref[m.row_start:m.row_end]
            assert p.grad is not None, name
            assert torch.allclose(p.grad, ref, rtol=2e-4, atol=2e-6), f"{name}: max diff {(p.grad - ref).abs().max().item():.3e}"
            checked += 1
        assert checked == len(gp)
        result.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        import traceback
        result.put((rank, f"{type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}"))
    finally:
        dist.destroy_process_group()


def test_two_rank_decoder_matches_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert out == [(0, "ok"), (1, "ok")], out
