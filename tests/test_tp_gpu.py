"""Row-sharded tensor parallelism on real GPUs (needs two; skipped otherwise): two NCCL ranks train a
sharded linear for three steps and must reproduce, row for row and bit for bit, the weight a single
GPU produces; the reduce-scattered input gradient must match the unsharded one."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        from forge_b200 import FusedLinear
        from forge_b200.tensor_parallel import RowShardedFusedLinear, feature_range
        g = torch.Generator().manual_seed(5)
        BT, H, V = 96, 512, 776            # 776 rows -> shards of 392 and 384 rows
        w0 = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
        xs = [torch.randn(BT, H, generator=g).bfloat16() for _ in range(3)]
        gys = [(torch.randn(BT, V, generator=g) * 1e-2).bfloat16() for _ in range(3)]
        tp = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode=mode)
        tp.train()
        c0, c1 = feature_range(H, rank, world)
        full = None
        if rank == 0:
            full = FusedLinear(H, V, optimizer_type="adamw", state_mode=mode)
            full.weight.data = w0.clone()
            full = full.to(dev).to(torch.bfloat16).train()
        for x, gy in zip(xs, gys):
            tp.local.update_optimizer_config(lr=1e-2, weight_decay=0.01)
            xin = x[:, c0:c1].to(dev).requires_grad_(True)
            y = tp(xin)
            y.backward(gy[:, tp.row_start:tp.row_end].to(dev))
            if rank == 0:
                w_before = full.weight.detach().clone()
                full.update_optimizer_config(lr=1e-2, weight_decay=0.01)
                xf = x.to(dev).requires_grad_(True)
                full(xf).backward(gy.to(dev))
                ref_dx = (gy.to(dev).double() @ w_before.double())[:, c0:c1]
                err = (xin.grad.double() - ref_dx).abs().max().item()
                # each rank's partial dX is rounded to bf16 before NCCL sums it in bf16
                assert err < 1.5e-2 * ref_dx.abs().max().item() + 1e-6, f"dX shard off by {err}"
        gathered = tp.gather_full_weight()
        if rank == 0:
            assert torch.equal(gathered.view(torch.int16), full.weight.detach().view(torch.int16)), \
                f"{(gathered != full.weight.detach()).sum().item()} weights differ from the single-GPU run"
        torch.cuda.synchronize()
        dist.barrier()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        q.put((rank, f"{type(e).__name__}: {e}"))
        q.close()
        q.join_thread()  # the message is on its way before the process goes
        os._exit(1)      # do not wait for a peer that is blocked in a collective


@pytest.mark.parametrize("mode", ["bf16", "int8", "fp8_block"])
def test_two_rank_nccl_matches_single_gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in procs:
            out.append(q.get(timeout=150))
            if out[-1][1] != "ok":
                break
    except Exception:
        out.append(("parent", "timed out waiting for the ranks"))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert sorted(out) == [(0, "ok"), (1, "ok")], out


def _scatter_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from forge_b200 import _lib
        from forge_b200.peer import DgradReduceScatter
        from forge_b200.tensor_parallel import reduce_scatter_features, row_range
        BT, H = 384, 1024
        Vs = (776, 264)                               # two linears sharing an input; unequal row shards
        rs = DgradReduceScatter([(BT, H), (BT, H)], device=dev)
        g = torch.Generator().manual_seed(11)         # the same full tensors on every rank
        outs = []
        for step in range(3):
            rs.begin_step()
            members, partial = [], torch.zeros(BT, H, dtype=torch.float64)
            full_ref = torch.zeros(BT, H, dtype=torch.float64)
            for V in Vs:
                dy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
                w = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
                full_ref += dy.double() @ w.double()
                r0, r1 = row_range(V, rank, world)
                members.append((dy[:, r0:r1].contiguous().to(dev), w[r0:r1].contiguous().to(dev)))
            out = rs.run(step % 2, members)
            # the NCCL path on the same partial products
            part = sum((a.float() @ b.float() for a, b in members)).bfloat16()
            ref_nccl = reduce_scatter_features(part)
            s = H // world
            ref = full_ref[:, rank * s:(rank + 1) * s]
            err = (out.double().cpu() - ref).abs().max().item()
            err_nccl = (ref_nccl.double().cpu() - ref).abs().max().item()
            assert err <= 2.0 * err_nccl + 1e-4 * ref.abs().max().item(), (err, err_nccl)
            outs.append(out.clone())
            dist.barrier()                            # buffers alternate; a collective separates their reuse
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 0
        dist.barrier()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e} {traceback.format_exc()[-800:]}"))
        q.close()
        q.join_thread()
        os._exit(1)


def test_two_rank_fused_dgrad_reduce_scatter():
    """GEMM with the reduce-scatter fused into its epilogue (peer stores + arrival words) on two ranks:
    as close to the exact sum as the library GEMM + NCCL reduce-scatter, three steps in a row."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_scatter_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in procs:
            out.append(q.get(timeout=150))
            if out[-1][1] != "ok":
                break
    except Exception:
        out.append(("parent", "timed out waiting for the ranks"))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert sorted(out) == [(0, "ok"), (1, "ok")], out


def _module_scatter_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from forge_b200 import _lib
        from forge_b200.peer import DgradReduceScatter
        from forge_b200.tensor_parallel import RowShardedFusedLinear, feature_range
        BT, H, V = 128, 512, 776
        g = torch.Generator().manual_seed(7)
        w0 = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
        plain = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode="int8").train()
        fused = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode="int8").train()
        rs = DgradReduceScatter([(BT, H)], device=dev)
        fused.attach_fused_scatter(rs, 0)
        c0, c1 = feature_range(H, rank, world)
        for step in range(3):
            x = torch.randn(BT, H, generator=g).bfloat16()
            gy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
            grads = []
            for layer in (plain, fused):
                layer.local.update_optimizer_config(lr=1e-2, weight_decay=0.01)
                if layer is fused:
                    rs.begin_step()
                xin = x[:, c0:c1].to(dev).requires_grad_(True)
                y = layer(xin)
                if layer is fused:
                    assert "ShardedLinearFusedScatter" in y.grad_fn.name()
                y.backward(gy[:, layer.row_start:layer.row_end].to(dev))
                grads.append(xin.grad)
            ref = (gy.double() @ w0.double())[:, c0:c1] if step == 0 else None
            scale = grads[0].float().abs().max().item()
            assert (grads[0].float() - grads[1].float()).abs().max().item() <= 2e-2 * scale + 1e-6
            dist.barrier()
        # the update sees the same dY and the same gathered X on both paths: identical weights and states
        assert torch.equal(plain.local.weight.data.view(torch.int16), fused.local.weight.data.view(torch.int16))
        sa, sb = plain.local.get_optimizer_state_dict(), fused.local.get_optimizer_state_dict()
        for k, v in sa.items():
            if torch.is_tensor(v):
                assert torch.equal(v.view(torch.uint8), sb[k].view(torch.uint8)), k
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 0
        dist.barrier()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e} {traceback.format_exc()[-800:]}"))
        q.close()
        q.join_thread()
        os._exit(1)


def test_two_rank_sharded_linear_with_fused_scatter():
    """``RowShardedFusedLinear`` with the fused GEMM + reduce-scatter attached against the same layer on
    the library GEMM + NCCL path: the same weights and optimizer state bit for bit, input gradients
    equal up to the rounding of the partial products."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_module_scatter_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in procs:
            out.append(q.get(timeout=150))
            if out[-1][1] != "ok":
                break
    except Exception:
        out.append(("parent", "timed out waiting for the ranks"))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert sorted(out) == [(0, "ok"), (1, "ok")], out


def _set_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from forge_b200 import _lib
        from forge_b200.peer import DgradReduceScatter
        from forge_b200.tensor_parallel import RowShardedFusedLinear, RowShardedLinearSet
        BT, H = 200, 528                              # ragged in both directions; H does not split into 128s
        Vs = (776, 264, 264)
        g = torch.Generator().manual_seed(3)
        w0 = [(torch.randn(V, H, generator=g) * 0.05).bfloat16() for V in Vs]

        def make():
            return [RowShardedFusedLinear.from_full_weight(w.to(dev), gather_input=False, optimizer_type="adamw",
                                                           state_mode="bf16").train() for w in w0]
        plain, members = make(), make()
        fused = RowShardedLinearSet(members)
        rs = DgradReduceScatter([(BT, H, "allreduce")], device=dev)
        fused.attach_fused_scatter(rs, 0)
        for step in range(3):
            x = torch.randn(BT, H, generator=g).bfloat16()
            gys = [(torch.randn(BT, V, generator=g) * 1e-2).bfloat16() for V in Vs]
            for layer in plain + members:
                layer.local.update_optimizer_config(lr=1e-2, weight_decay=0.01)
            # library GEMMs, autograd's additions and an NCCL all-reduce
            xin = x.to(dev).requires_grad_(True)
            outs = [m(xin) for m in plain]
            torch.autograd.backward(outs, [gy[:, m.row_start:m.row_end].to(dev) for gy, m in zip(gys, plain)])
            ref = xin.grad.clone()
            dist.all_reduce(ref)
            # one GEMM launch whose tiles go to both ranks
            rs.begin_step()
            xin2 = x.to(dev).requires_grad_(True)
            outs2, complete = fused(xin2)
            assert complete and "ShardedSetFusedAllReduce" in outs2[0].grad_fn.name()
            for a, b in zip(outs, outs2):
                assert torch.equal(a, b)
            torch.autograd.backward(outs2, [gy[:, m.row_start:m.row_end].to(dev) for gy, m in zip(gys, members)])
            exact = sum(gy.double() @ w.double() for gy, w in zip(gys, w0)) if step == 0 else None
            scale = ref.float().abs().max().item()
            assert (ref.float() - xin2.grad.float()).abs().max().item() <= 2e-2 * scale + 1e-6
            if exact is not None:
                err = (xin2.grad.double().cpu() - exact).abs().max().item()
                err_ref = (ref.double().cpu() - exact).abs().max().item()
                assert err <= 2.0 * err_ref + 1e-4 * exact.abs().max().item(), (err, err_ref)
            # both ranks hold the same sum, bit for bit (fixed order of addition)
            mine = xin2.grad.clone()
            other = mine.clone()
            dist.broadcast(other, src=0)
            assert torch.equal(mine.view(torch.int16), other.view(torch.int16))
            dist.barrier()
        for a, b in zip(plain, members):
            assert torch.equal(a.local.weight.data.view(torch.int16), b.local.weight.data.view(torch.int16))
            sa, sb = a.local.get_optimizer_state_dict(), b.local.get_optimizer_state_dict()
            for k, v in sa.items():
                if torch.is_tensor(v):
                    assert torch.equal(v.view(torch.uint8), sb[k].view(torch.uint8)), k
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 0
        dist.barrier()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e} {traceback.format_exc()[-800:]}"))
        q.close()
        q.join_thread()
        os._exit(1)


def test_two_rank_linear_set_with_fused_all_reduce():
    """Three sharded linears on one replicated input: one GEMM launch that accumulates over the members
    and stores its tiles into both ranks' buffers, against three library GEMMs + NCCL all-reduce.  Same
    outputs, weights and optimizer state bit for bit; the input gradient as close to the exact sum, and
    identical on the two ranks."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_set_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in procs:
            out.append(q.get(timeout=150))
            if out[-1][1] != "ok":
                break
    except Exception:
        out.append(("parent", "timed out waiting for the ranks"))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert sorted(out) == [(0, "ok"), (1, "ok")], out


def _gather_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        from forge_b200 import _lib
        from forge_b200.peer import DgradReduceScatter, GatheredLinear
        from forge_b200.tensor_parallel import RowShardedFusedLinear, feature_range
        BT, H, V = 200, 1280, 528                      # ragged rows; 640-column input blocks, 264-row shards
        g = torch.Generator().manual_seed(9)
        w0 = (torch.randn(V, H, generator=g) * 0.05).bfloat16()
        plain = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode="int8").train()
        fused = RowShardedFusedLinear.from_full_weight(w0.to(dev), optimizer_type="adamw", state_mode="int8").train()
        rs = DgradReduceScatter([(BT, H)], device=dev)
        gl = GatheredLinear([(BT, H, V)], device=dev)
        fused.attach_fused_scatter(rs, 0)
        fused.attach_fused_gather(gl, 0)
        c0, c1 = feature_range(H, rank, world)
        for step in range(3):
            x = torch.randn(BT, H, generator=g).bfloat16()
            gy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
            for layer in (plain, fused):
                layer.local.update_optimizer_config(lr=1e-2, weight_decay=0.01)
            xin = x[:, c0:c1].to(dev).requires_grad_(True)
            y = plain(xin)                                       # this rank's columns
            y.backward(gy[:, plain.row_start:plain.row_end].to(dev))
            rs.begin_step()
            gl.begin_step()
            xin2 = x[:, c0:c1].to(dev).requires_grad_(True)
            assert fused.returns_full_output(xin2)
            y2 = fused(xin2)                                     # all columns, the same on both ranks
            assert "ShardedLinearFusedGather" in y2.grad_fn.name() and y2.shape == (BT, V)
            ref = x.double() @ w0.double().t() if step == 0 else None
            if ref is not None:
                err = (y2.double().cpu() - ref).abs().max().item()
                err_lib = (y.double().cpu() - ref[:, plain.row_start:plain.row_end]).abs().max().item()
                assert err <= 2.0 * err_lib + 1e-3 * ref.abs().max().item(), (err, err_lib)
            other = y2.detach().clone()
            dist.broadcast(other, src=0)
            assert torch.equal(other.view(torch.int16), y2.detach().view(torch.int16))
            y2.backward(gy.to(dev))
            scale = xin.grad.float().abs().max().item()
            assert (xin.grad.float() - xin2.grad.float()).abs().max().item() <= 2e-2 * scale + 1e-6
            dist.barrier()
        # the update saw the same dY and the same gathered X on both paths
        assert torch.equal(plain.local.weight.data.view(torch.int16), fused.local.weight.data.view(torch.int16))
        sa, sb = plain.local.get_optimizer_state_dict(), fused.local.get_optimizer_state_dict()
        for k, v in sa.items():
            if torch.is_tensor(v):
                assert torch.equal(v.view(torch.uint8), sb[k].view(torch.uint8)), k
        torch.cuda.synchronize()
        assert _lib.read_status(dev) == 0
        dist.barrier()
        q.put((rank, "ok"))
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, f"{type(e).__name__}: {e} {traceback.format_exc()[-800:]}"))
        q.close()
        q.join_thread()
        os._exit(1)


def test_two_rank_sharded_linear_with_fused_gathers():
    """``RowShardedFusedLinear`` whose forward pushes its input block to the peer, multiplies the blocks as
    they arrive and stores its output tiles into both ranks' gathered output, against all-gather + library
    GEMM: the output as close to the exact product and identical on both ranks, the same weights and
    optimizer state bit for bit after three steps."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in procs:
            out.append(q.get(timeout=150))
            if out[-1][1] != "ok":
                break
    except Exception:
        out.append(("parent", "timed out waiting for the ranks"))
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
    assert sorted(out) == [(0, "ok"), (1, "ok")], out
