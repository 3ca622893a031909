"""GPU parity of the dX GEMM (``forge_dgrad``): dX = dY W with bf16 operands, fp32 accumulation and
bf16 output, against an fp32 CPU matmul of the same bf16 values (the reference computes
``grad_output @ weight``, ``autograd.py:55``)."""

import pytest
import torch

from forge_b200 import kernel as K
from tests.util import assert_one_ulp

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = [(128, 128, 128), (512, 1024, 1024), (200, 392, 1032), (8, 8, 64), (64, 4096, 256), (520, 136, 264)]


@pytest.mark.parametrize("BT,V,H", SHAPES)
def test_dgrad_exact_sums(BT, V, H):
    """Multiples of 1/8: every partial sum is exact in fp32, so the bf16 result is unique."""
    g = torch.Generator().manual_seed(21)
    dy = (torch.randint(-8, 9, (BT, V), generator=g).float() / 8).bfloat16()
    w = (torch.randint(-8, 9, (V, H), generator=g).float() / 8).bfloat16()
    expect = (dy.float() @ w.float()).bfloat16()
    out = K.dgrad(dy.to(DEV), w.to(DEV))
    assert out.shape == (BT, H) and out.dtype == torch.bfloat16
    assert torch.equal(out.cpu().view(torch.int16), expect.view(torch.int16))


@pytest.mark.parametrize("BT,V,H", SHAPES)
def test_dgrad_gaussian(BT, V, H):
    g = torch.Generator().manual_seed(22)
    dy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16()
    w = (torch.randn(V, H, generator=g) * 0.02).bfloat16()
    expect = dy.double() @ w.double()
    scale = dy.double().abs() @ w.double().abs()
    out = K.dgrad(dy.to(DEV), w.to(DEV))
    assert_one_ulp(expect.float(), out, scale.float(), "dX", noise=4e-6)


def test_dgrad_strided_and_module_path():
    """Row-pitched operands, and the autograd path with the library GEMM switched on."""
    from forge_b200 import FusedLinear, autograd
    BT, V, H = 96, 256, 320
    g = torch.Generator().manual_seed(23)
    dyw = (torch.randn(BT, V + 64, generator=g) * 1e-2).bfloat16().to(DEV)
    ww = (torch.randn(V, H + 64, generator=g) * 0.02).bfloat16().to(DEV)
    dy, w = dyw[:, :V], ww[:, 32:32 + H]
    out = K.dgrad(dy, w)
    assert_one_ulp((dy.double().cpu() @ w.double().cpu()).float(), out,
                   (dy.double().abs().cpu() @ w.double().abs().cpu()).float(), "dX")
    layer = FusedLinear(H, V, optimizer_type="sgd").to(DEV).to(torch.bfloat16).train()
    layer.update_optimizer_config(lr=1e-2, weight_decay=0.0)
    x = torch.randn(4, 24, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w0 = layer.weight.detach().clone()
    old = autograd.use_forge_dgrad
    autograd.use_forge_dgrad = True
    try:
        y = layer(x)
        gy = torch.randn_like(y) * 1e-2
        y.backward(gy)
    finally:
        autograd.use_forge_dgrad = old
    expect = (gy.double().reshape(-1, V) @ w0.double()).reshape(4, 24, H)   # the PRE-update weight
    assert x.grad.shape == x.shape
    assert_one_ulp(expect.float().cpu(), x.grad, (gy.double().abs().reshape(-1, V) @ w0.double().abs()).reshape(4, 24, H).float().cpu(), "x.grad")
    assert not torch.equal(layer.weight.detach(), w0)


@pytest.mark.parametrize("BT,H,Vs", [(512, 1024, (1024, 256, 256)), (200, 520, (136, 264)), (64, 256, (72, 8, 640, 128))])
def test_dgrad_sum_of_several_pairs(BT, H, Vs):
    """dX = sum_i dY_i W_i in one launch (q / k / v share their input gradient): exact-sum inputs, so the
    bf16 result is unique whatever the accumulation order across and inside the segments."""
    g = torch.Generator().manual_seed(24)
    members, expect = [], torch.zeros(BT, H)
    for V in Vs:
        dy = (torch.randint(-8, 9, (BT, V), generator=g).float() / 8).bfloat16()
        w = (torch.randint(-8, 9, (V, H), generator=g).float() / 8).bfloat16()
        expect += dy.float() @ w.float()
        members.append((dy.to(DEV), w.to(DEV)))
    out = K.dgrad_sum(members)
    assert torch.equal(out.cpu().view(torch.int16), expect.bfloat16().view(torch.int16))
    with pytest.raises(ValueError):
        K.dgrad_sum(members + members + members)


def test_scatter_and_reduce_on_one_rank_equal_the_plain_gemm():
    """The fused GEMM + reduce-scatter with a world of one: the epilogue's direct stores into the (only)
    receive slot, the arrival word and the reduce kernel, against ``dgrad_sum`` bit for bit; and a reduce
    whose arrival never comes gives up, reports code 211 and leaves its output untouched."""
    import torch.distributed as dist
    from forge_b200 import _lib
    from forge_b200.peer import DgradReduceScatter
    own_group = not dist.is_initialized()
    if own_group:
        import socket
        sock = socket.socket()
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
        sock.close()
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    g = torch.Generator().manual_seed(25)
    BT, H = 520, 1152
    sets = [(BT, H), (BT, 256), (BT, 1000, "allreduce")]
    rs = DgradReduceScatter(sets, device=torch.device(DEV, torch.cuda.current_device()))
    for step in range(2):                       # the same buffers two steps in a row
        rs.begin_step()
        members = [((torch.randn(BT, V, generator=g) * 1e-2).bfloat16().to(DEV), (torch.randn(V, H, generator=g) * 0.02).bfloat16().to(DEV))
                   for V in (392, 136)]
        out = rs.run(0, members)
        assert torch.equal(out.view(torch.int16), K.dgrad_sum(members).view(torch.int16))
        small = [((torch.randn(BT, 64, generator=g)).bfloat16().to(DEV), (torch.randn(64, 256, generator=g)).bfloat16().to(DEV))]
        assert torch.equal(rs.run(1, small).view(torch.int16), K.dgrad_sum(small).view(torch.int16))
        # every-rank mode: slots are full width and H need not split into 128-column blocks
        ragged = [((torch.randn(BT, V, generator=g) * 1e-2).bfloat16().to(DEV), (torch.randn(V, 1000, generator=g) * 0.02).bfloat16().to(DEV))
                  for V in (136, 72, 264)]
        out = rs.run(2, ragged)
        assert out.shape == (BT, 1000)
        assert torch.equal(out.view(torch.int16), K.dgrad_sum(ragged).view(torch.int16))
    with pytest.raises(RuntimeError, match="already run"):
        rs.run(1, small)                          # twice in one step: the receive buffers are still in use
    torch.cuda.synchronize()
    dev = torch.device(DEV, torch.cuda.current_device())
    assert _lib.read_status(dev) == 0
    # an arrival that never comes: the epoch moves on but nobody stores
    lib = _lib.load()
    rs.begin_step()
    out = torch.full((BT, 256), 7.0, dtype=torch.bfloat16, device=DEV)
    import ctypes
    fn = lib.forge_reduce_slots
    assert fn(rs.slots.data_ptr(), rs.arrivals.data_ptr(), rs.epoch.data_ptr(), None, BT, 256, 256, 1, None, None) == _lib.FORGE_ERR_INVALID_ARG
    assert lib.forge_set_arrival_wait_ns(20_000_000) == 0          # 20 ms instead of the production two seconds
    rc = fn(rs.slots.data_ptr() + rs._slot_off[1], rs.arrivals.data_ptr() + 4, rs.epoch.data_ptr(), out.data_ptr(), BT, 256, 256, 1,
            _lib.status_word(dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert (out == 7.0).all()
    assert lib.forge_set_arrival_wait_ns(2_000_000_000) == 0
    with pytest.raises(_lib.ForgeLibraryError, match="211"):
        _lib.read_status(dev)
    if own_group:
        dist.destroy_process_group()


def test_gathered_linear_on_one_rank_equals_the_plain_product():
    """The forward GEMM of the row-sharded mode with a world of one: push of the (only) input block, the
    K-major product, both output forms (local TMA store; peer-store epilogue + collect), ragged sizes."""
    from forge_b200 import _lib
    from forge_b200.peer import GatheredLinear
    g = torch.Generator().manual_seed(31)
    dev = torch.device(DEV, torch.cuda.current_device())
    sets = [(200, 1000, 264), (512, 4096, 1024), (64, 64, 8)]
    gl = GatheredLinear(sets, device=dev)
    for step in range(2):
        gl.begin_step()
        for i, (bt, h, v) in enumerate(sets):
            x = torch.randn(bt, h, generator=g).bfloat16().to(DEV)
            w = (torch.randn(v, h, generator=g) * 0.05).bfloat16().to(DEV)
            gl.push(i, x)
            assert torch.equal(gl.gathered_input(i), x)
            ref = x.double() @ w.double().t()
            lib = torch.nn.functional.linear(x, w)
            scale = ref.abs().max().item()
            err_lib = (lib.double() - ref).abs().max().item()
            for full in (False, True):
                y = gl.linear(i, w, full_output=full)
                assert y.shape == (bt, v)
                err = (y.double() - ref).abs().max().item()
                assert err <= 2.0 * err_lib + 1e-3 * scale, (i, full, err, err_lib)
    with pytest.raises(RuntimeError, match="already been pushed"):
        gl.push(0, torch.zeros(200, 1000, dtype=torch.bfloat16, device=DEV))      # a second forward in one step
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0


def _ptr_array(ptrs):
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def test_two_ranks_emulated_on_one_gpu_through_the_c_abi():
    """Both ranks of the row-sharded forward and backward products, run one after the other on ONE GPU
    with every "peer" buffer in local memory (each launch only waits for arrivals that earlier launches
    have already raised): pushes -> gathered products with pushed outputs -> collect, and the backward's
    GEMM + reduce-scatter, against the unsharded products.  Then a product whose second input block never
    arrives: the producer's wait runs out, the status word reads 211 and the context stays usable."""
    import ctypes
    from forge_b200 import _lib
    lib = _lib.load()
    dev = torch.device(DEV, torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    status = _lib.status_word(dev).data_ptr()
    g = torch.Generator().manual_seed(41)
    R, BT, H, V = 2, 200, 1280, 528
    blk, vr = H // R, V // R
    x = torch.randn(BT, H, generator=g).bfloat16().to(DEV)
    w = (torch.randn(V, H, generator=g) * 0.05).bfloat16().to(DEV)
    dy = (torch.randn(BT, V, generator=g) * 1e-2).bfloat16().to(DEV)
    xg = [torch.zeros(BT, H, dtype=torch.bfloat16, device=DEV) for _ in range(R)]      # each rank's gathered input
    yg = [torch.zeros(BT, V, dtype=torch.bfloat16, device=DEV) for _ in range(R)]      # each rank's gathered output
    arr = [torch.zeros(2 * R, dtype=torch.int32, device=DEV) for _ in range(R)]         # [0:R] input, [R:2R] output arrivals
    counters = torch.zeros(2 * R, dtype=torch.int32, device=DEV)
    epoch = torch.full((1,), 5, dtype=torch.int32, device=DEV)
    x_dst, y_dst = _ptr_array([t.data_ptr() for t in xg]), _ptr_array([t.data_ptr() for t in yg])
    x_arr = _ptr_array([t.data_ptr() for t in arr])
    y_arr = _ptr_array([t.data_ptr() + 4 * R for t in arr])
    for r in range(R):
        xb = x[:, r * blk:(r + 1) * blk]
        _lib.check(lib.forge_push_block(xb.data_ptr(), BT, blk, xb.stride(0), x_dst, r * blk, H, x_arr,
                                        counters.data_ptr() + 4 * r, epoch.data_ptr(), r, R, status, stream), "push")
    for r in range(R):
        assert torch.equal(xg[r], x)
    for r in range(R):
        wr = w[r * vr:(r + 1) * vr]
        a = _lib.ForgeLinearGatheredArgs()
        a.X, a.W, a.BT, a.H, a.V_r, a.ld_x, a.ld_w = xg[r].data_ptr(), wr.data_ptr(), BT, H, vr, H, wr.stride(0)
        a.x_arrivals, a.epoch, a.rank, a.world = arr[r].data_ptr(), epoch.data_ptr(), r, R
        a.y, a.y_dst, a.y_col, a.y_pitch, a.y_arrivals = None, y_dst, r * vr, V, y_arr
        a.y_counter, a.status = counters.data_ptr() + 4 * (R + r), status
        _lib.check(lib.forge_linear_gathered(ctypes.byref(a), stream), "forge_linear_gathered")
    ref = x.double() @ w.double().t()
    lib_y = torch.nn.functional.linear(x, w)
    err_lib = (lib_y.double() - ref).abs().max().item()
    outs = []
    for r in range(R):
        out = torch.empty(BT, V, dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.forge_collect(yg[r].data_ptr(), V, arr[r].data_ptr() + 4 * R, epoch.data_ptr(), out.data_ptr(), BT, V, V,
                                     R, status, stream), "forge_collect")
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert (outs[0].double() - ref).abs().max().item() <= 2.0 * err_lib + 1e-3 * ref.abs().max().item()
    # backward: every rank's partial dX tiles into the owners' slots, then each owner's sum
    slots = [torch.zeros(R, BT, blk, dtype=torch.bfloat16, device=DEV) for _ in range(R)]
    sarr = [torch.zeros(R, dtype=torch.int32, device=DEV) for _ in range(R)]
    sc = torch.zeros(R, dtype=torch.int32, device=DEV)
    s_ptrs, a_ptrs = _ptr_array([t.data_ptr() for t in slots]), _ptr_array([t.data_ptr() for t in sarr])
    for r in range(R):
        dyr, wr = dy[:, r * vr:(r + 1) * vr].contiguous(), w[r * vr:(r + 1) * vr]
        seg = (_lib.ForgeDgradSegment * 1)()
        seg[0].dY, seg[0].W, seg[0].V, seg[0].ld_dy, seg[0].ld_w = dyr.data_ptr(), wr.data_ptr(), vr, dyr.stride(0), wr.stride(0)
        a = _lib.ForgeDgradScatterArgs()
        a.segments, a.count, a.BT, a.H, a.slots, a.arrivals = seg, 1, BT, H, s_ptrs, a_ptrs
        a.counter, a.epoch, a.rank, a.world, a.status, a.all_ranks = sc.data_ptr() + 4 * r, epoch.data_ptr(), r, R, status, 0
        _lib.check(lib.forge_dgrad_scatter(ctypes.byref(a), stream), "forge_dgrad_scatter")
        torch.cuda.synchronize()          # dyr stays alive until its launch has run
    ref_dx = dy.double() @ w.double()
    lib_dx = dy @ w
    err_lib = (lib_dx.double() - ref_dx).abs().max().item()
    for r in range(R):
        out = torch.empty(BT, blk, dtype=torch.bfloat16, device=DEV)
        _lib.check(lib.forge_reduce_slots(slots[r].data_ptr(), sarr[r].data_ptr(), epoch.data_ptr(), out.data_ptr(), BT, blk, blk,
                                          R, status, stream), "forge_reduce_slots")
        err = (out.double() - ref_dx[:, r * blk:(r + 1) * blk]).abs().max().item()
        assert err <= 3.0 * err_lib + 1e-3 * ref_dx.abs().max().item(), (r, err, err_lib)
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
    # a block that never arrives
    epoch.add_(1)
    out = torch.full((BT, vr), 3.0, dtype=torch.bfloat16, device=DEV)
    wr = w[:vr]
    a = _lib.ForgeLinearGatheredArgs()
    a.X, a.W, a.BT, a.H, a.V_r, a.ld_x, a.ld_w = xg[0].data_ptr(), wr.data_ptr(), BT, H, vr, H, wr.stride(0)
    a.x_arrivals, a.epoch, a.rank, a.world = arr[0].data_ptr(), epoch.data_ptr(), 0, R
    a.y, a.ld_y, a.status = out.data_ptr(), vr, status
    assert lib.forge_set_arrival_wait_ns(20_000_000) == 0
    _lib.check(lib.forge_linear_gathered(ctypes.byref(a), stream), "forge_linear_gathered")
    torch.cuda.synchronize()
    assert lib.forge_set_arrival_wait_ns(2_000_000_000) == 0
    with pytest.raises(_lib.ForgeLibraryError, match="211"):
        _lib.read_status(dev)
    # the context is still usable
    assert torch.equal(K.dgrad(dy, w).view(torch.int16), K.dgrad(dy, w).view(torch.int16))
    torch.cuda.synchronize()
    assert _lib.read_status(dev) == 0
