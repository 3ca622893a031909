"""Host-side logic of the row-sharded tensor-parallel mode on two gloo ranks (CPU): shard
arithmetic, the feature all-gather / reduce-scatter pair and its autograd, and a sharded linear
against the unsharded one (without an optimizer config the module behaves like a plain linear, so no
CUDA kernel is involved)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from forge_b200.tensor_parallel import feature_range, row_range


def test_row_and_feature_ranges():
    for V, world in [(4096, 8), (1024, 8), (128256, 8), (151936, 8), (1024, 3), (8, 2), (24, 5)]:
        spans = [row_range(V, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == V
        for (s0, e0), (s1, e1) in zip(spans, spans[1:]):
            assert e0 == s1
        assert all(s % 8 == 0 and e % 8 == 0 for s, e in spans)
        sizes = [e - s for s, e in spans]
        assert max(sizes) - min(sizes) <= 8
    assert row_range(128256, 0, 8) == (0, 16032)
    with pytest.raises(ValueError):
        row_range(100, 0, 2)
    assert feature_range(4096, 3, 8) == (1536, 2048)
    with pytest.raises(ValueError):
        feature_range(100, 0, 8)


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
        from forge_b200.tensor_parallel import (RowShardedFusedLinear, all_gather_features, gather_rows,
                                                reduce_scatter_features)
        torch.manual_seed(0)                      # same tensors on every rank
        BT, H, V = 6, 16, 40                      # 40 rows -> shards of 24 and 16 rows
        x = torch.randn(2, 3, H)
        w = torch.randn(V, H)
        gy = torch.randn(2, 3, V)
        c0, c1 = feature_range(H, rank, world)
        # gather / scatter
        xg = all_gather_features(x[..., c0:c1].contiguous())
        assert torch.equal(xg, x)
        rs = reduce_scatter_features(x * (rank + 1))
        assert torch.allclose(rs, x[..., c0:c1] * sum(range(1, world + 1)))
        # sharded linear == full linear (forward slice, dX shard, dW rows)
        xs = x[..., c0:c1].clone().requires_grad_(True)
        lin = RowShardedFusedLinear.from_full_weight(w)
        lin.train()
        y = lin(xs)
        r0, r1 = lin.row_start, lin.row_end
        full_y = x @ w.t()
        assert torch.allclose(y, full_y[..., r0:r1], atol=1e-5)
        y.backward(gy[..., r0:r1])
        full_dx = gy @ w
        assert torch.allclose(xs.grad, full_dx[..., c0:c1], atol=1e-4)
        full_dw = gy.reshape(-1, V).t() @ x.reshape(-1, H)
        assert torch.allclose(lin.weight.grad, full_dw[r0:r1], atol=1e-4)
        assert torch.equal(lin.gather_full_weight(), w)
        assert torch.equal(gather_rows(w[r0:r1], V, rank, world), w)
        # a set of linears on one replicated input: on the host (no fused collective attached, CPU tensors)
        # it runs its members one by one and says that the input gradient still has to be summed
        from forge_b200.tensor_parallel import RowShardedLinearSet
        members = [RowShardedFusedLinear.from_full_weight(w, gather_input=False),
                   RowShardedFusedLinear.from_full_weight(w[:16], gather_input=False)]
        group = RowShardedLinearSet(members)
        assert not list(group.parameters()), "the set does not own its members"
        xr = x.clone().requires_grad_(True)
        assert not group.fused(xr)
        outs, complete = group(xr)
        assert not complete and len(outs) == 2
        assert torch.allclose(outs[0], full_y[..., members[0].row_start:members[0].row_end], atol=1e-5)
        with pytest.raises(ValueError):
            RowShardedLinearSet([lin])                       # gathers its own input: not a member of a set
        with pytest.raises(ValueError):
            RowShardedLinearSet([members[0], RowShardedFusedLinear(8, 16, gather_input=False)])   # another input
        assert not lin.returns_full_output(xs)
        result.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        result.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(out) == [(0, "ok"), (1, "ok")], out
