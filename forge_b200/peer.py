"""Fused dX GEMM + reduce-scatter for the row-sharded tensor-parallel mode, over peer memory.

The reference has no distributed code.  In this mode every rank holds rows of each weight, so the input
gradient of a linear is a sum over ranks of partial products ``dY_r W_r``; ``tensor_parallel.py`` forms
it with a library GEMM followed by an NCCL reduce-scatter.  Here the two are one step: the GEMM
(``forge_dgrad_scatter``) stores every output tile directly into the receive buffer of the rank that
owns its feature block, with plain peer stores over NVLink while the other tiles are still being
computed, and raises an arrival word on the owner when its last tile is out; the owner
(``forge_reduce_slots``) waits for all arrival words -- a bounded wait: after two seconds it gives up
and reports through the status word -- and adds the ``world`` slots in rank order in fp32, so the result
is bit-reproducible.  No collective library call, no bulk-tensor copy and no multicast touches peer
memory.

Receive buffers are symmetric allocations shared over CUDA IPC (one process per GPU on one node).  A
buffer is written by every rank and may be reused only when all ranks have finished reading it: each
linear set of a step gets a buffer of its own here, and between two steps the ranks meet in a
collective anyway (the forward pass of the next step gathers activations).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from forge_b200 import _lib


def _world_and_rank(group=None):
    """(1, 0) in a process without a process group: the single-GPU forms of the kernels."""
    if not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _share(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    """Views of every rank's tensor `t` (same shape everywhere) mapped into this process."""
    from torch.multiprocessing.reductions import reduce_tensor
    world, rank = _world_and_rank(group)
    if world == 1:
        return [t]
    fn, args = reduce_tensor(t)
    gathered = [None] * world
    dist.all_gather_object(gathered, (fn, args), group=group)
    out = []
    for r, (f, a) in enumerate(gathered):
        if r == rank:
            out.append(t)
        else:
            a = list(a)
            a[6] = t.device.index          # open the peer's allocation on this rank's device
            out.append(f(*a))
    return out


class DgradReduceScatter:
    """The input gradients of a step's linear sets, each ``dX[:, my block] = sum_r sum_i dY_r,i W_r,i``.

    ``sets``: one ``(BT, H)`` or ``(BT, H, "allreduce")`` per set of linears that share an input.  The
    plain form scatters: each rank ends up with its feature block ``(BT, H / world)`` of the summed
    gradient (layers whose input was gathered from feature shards).  ``"allreduce"`` sends every tile to
    every rank instead, and each rank sums the full ``(BT, H)`` itself -- one step instead of a
    reduce-scatter followed by an all-gather -- for sets whose input is replicated (q / k / v, gate / up).
    Every rank must construct this with the same list (collective).  ``begin_step()`` advances the epoch that
    tells this step's arrivals from the last one's (a one-element device add: it can sit inside a
    captured graph).  ``run(i, [(dY, W), ...])`` launches the GEMM + peer stores and the reduce on the
    current stream and returns this rank's ``(BT, H / world)`` block.
    """

    def __init__(self, sets, group=None, device=None):
        self.group = group
        self.world, self.rank = _world_and_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.sets, self.all_ranks = [], []
        for entry in sets:
            bt, h = int(entry[0]), int(entry[1])
            everywhere = len(entry) > 2 and entry[2] == "allreduce"
            if everywhere:
                if h % 8:
                    raise ValueError(f"H ({h}) must be a multiple of 8")
            elif h % self.world or (h // self.world) % 128:
                raise ValueError(f"H ({h}) must split into {self.world} feature blocks that are multiples of 128 columns")
            self.sets.append((bt, h))
            self.all_ranks.append(everywhere)
        offs, total = [], 0
        for (bt, h), everywhere in zip(self.sets, self.all_ranks):
            offs.append(total)
            total += (bt * h * 2 * (self.world if everywhere else 1) + 255) // 256 * 256
        self._slot_off = offs
        self._used: set[int] = set()
        n = len(self.sets)
        self.slots = torch.zeros(max(total, 256), dtype=torch.uint8, device=self.device)
        self.arrivals = torch.zeros(max(n * self.world, 1), dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(max(n, 1), dtype=torch.int32, device=self.device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self._peer_slots = _share(self.slots, group)
        self._peer_arrivals = _share(self.arrivals, group)
        self._slot_ptrs, self._arr_ptrs = [], []
        for i in range(n):
            self._slot_ptrs.append((ctypes.c_void_p * self.world)(*[p.data_ptr() + offs[i] for p in self._peer_slots]))
            self._arr_ptrs.append((ctypes.c_void_p * self.world)(*[p.data_ptr() + 4 * i * self.world
                                                                   for p in self._peer_arrivals]))
        if self.world > 1:
            dist.barrier(group=group)

    def begin_step(self):
        self.epoch.add_(1)
        self._used.clear()

    def run(self, index: int, members, out: torch.Tensor | None = None, reduce_stream=None) -> torch.Tensor:
        """``reduce_stream``: run the owner's wait-and-sum there (after the GEMM, by an event) so that the
        current stream can go on while the peers' tiles are still arriving; the caller orders its use of
        the result after that stream."""
        if index in self._used:
            # a second launch would store into receive buffers that a peer may still be summing
            raise RuntimeError(f"set {index} has already run in this step; call begin_step() between steps")
        self._used.add(index)
        bt, h = self.sets[index]
        everywhere = self.all_ranks[index]
        s = h if everywhere else h // self.world
        if not 1 <= len(members) <= 4:
            raise ValueError("one to four (dY, W) pairs per set")
        segs = (_lib.ForgeDgradSegment * len(members))()
        for k, (dy, w) in enumerate(members):
            if dy.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or dy.shape[0] != bt or w.shape[1] != h \
                    or dy.shape[1] != w.shape[0] or dy.stride(1) != 1 or w.stride(1) != 1:
                raise ValueError(f"member {k}: expected bf16 dY ({bt}, V) and W (V, {h}) with contiguous rows")
            segs[k].dY, segs[k].W, segs[k].V = dy.data_ptr(), w.data_ptr(), dy.shape[1]
            segs[k].ld_dy, segs[k].ld_w = dy.stride(0), w.stride(0)
        a = _lib.ForgeDgradScatterArgs()
        a.segments, a.count, a.BT, a.H = segs, len(members), bt, h
        a.slots = self._slot_ptrs[index]
        a.arrivals = self._arr_ptrs[index]
        a.counter = self.counters.data_ptr() + 4 * index
        a.epoch = self.epoch.data_ptr()
        a.rank, a.world = self.rank, self.world
        a.all_ranks = 1 if everywhere else 0
        status = _lib.status_word(self.device).data_ptr()
        a.status = status
        lib = _lib.load()
        if out is None:
            out = torch.empty(bt, s, dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            stream = _lib.current_stream_ptr(self.device)
            _lib.check(lib.forge_dgrad_scatter(ctypes.byref(a), stream), "forge_dgrad_scatter")
            if reduce_stream is not None:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream(self.device))
                reduce_stream.wait_event(ev)
                stream = reduce_stream.cuda_stream
            _lib.check(lib.forge_reduce_slots(self.slots.data_ptr() + self._slot_off[index],
                                              self.arrivals.data_ptr() + 4 * index * self.world, self.epoch.data_ptr(),
                                              out.data_ptr(), bt, s, out.stride(0), self.world, status, stream),
                       "forge_reduce_slots")
        return out


class GatheredLinear:
    """The forward products of a step's feature-sharded-input linears (o, down), ``Y = gather(X) W_r^T``,
    with both all-gathers of the row-sharded mode fused in (``forge_push_block`` / ``forge_linear_gathered``
    / ``forge_collect``): every rank pushes its block of X into every rank's gathered input with plain
    peer stores; the GEMM starts on the own block and waits for another block only when it reaches it;
    its epilogue stores the output tiles into every rank's gathered output, which a small kernel copies
    out once all ranks have arrived.  No reference counterpart (``F.linear``, ``autograd.py:34``).

    ``sets``: one ``(BT, H, V)`` per linear (full sizes).  ``begin_step()`` advances the epoch and runs one
    tiny collective: a buffer of the step before may be rewritten only when every rank has finished
    with it, and a collective on the stream after that step's work is what shows it.  The gathered input
    of a set stays valid until the next ``begin_step`` (the backward pass reads it).  Collective
    constructor; at most 8 ranks.
    """

    def __init__(self, sets, group=None, device=None):
        self.group = group
        self.world, self.rank = _world_and_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.sets = [(int(bt), int(h), int(v)) for bt, h, v in sets]
        for bt, h, v in self.sets:
            if h % (8 * self.world) or v % (8 * self.world):
                raise ValueError(f"H ({h}) and V ({v}) must split into {self.world} blocks that are multiples of 8")
        xo, yo, total_x, total_y = [], [], 0, 0
        for bt, h, v in self.sets:
            xo.append(total_x)
            yo.append(total_y)
            total_x += (bt * h * 2 + 255) // 256 * 256
            total_y += (bt * v * 2 + 255) // 256 * 256
        self._x_off, self._y_off = xo, yo
        self._pushed: set[int] = set()
        n = len(self.sets)
        self.x_buf = torch.zeros(max(total_x, 256), dtype=torch.uint8, device=self.device)
        self.y_buf = torch.zeros(max(total_y, 256), dtype=torch.uint8, device=self.device)
        # per set: `world` arrival words for the input blocks, `world` for the output blocks
        self.arrivals = torch.zeros(max(2 * n * self.world, 1), dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(max(2 * n, 1), dtype=torch.int32, device=self.device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.tick = torch.zeros(1, dtype=torch.float32, device=self.device)
        torch.cuda.synchronize(self.device)
        px, py, pa = _share(self.x_buf, group), _share(self.y_buf, group), _share(self.arrivals, group)
        self._keep = (px, py, pa)
        w = self.world
        arr = ctypes.c_void_p * w
        self._x_dst = [arr(*[t.data_ptr() + xo[i] for t in px]) for i in range(n)]
        self._y_dst = [arr(*[t.data_ptr() + yo[i] for t in py]) for i in range(n)]
        self._x_arr = [arr(*[t.data_ptr() + 4 * (2 * i) * w for t in pa]) for i in range(n)]
        self._y_arr = [arr(*[t.data_ptr() + 4 * (2 * i + 1) * w for t in pa]) for i in range(n)]
        if self.world > 1:
            dist.barrier(group=group)

    def begin_step(self):
        self.epoch.add_(1)
        self._pushed.clear()
        if self.world > 1:
            dist.all_reduce(self.tick, group=self.group)

    def gathered_input(self, index: int) -> torch.Tensor:
        bt, h, _ = self.sets[index]
        return self.x_buf[self._x_off[index]: self._x_off[index] + bt * h * 2].view(torch.bfloat16).view(bt, h)

    def push(self, index: int, x_block: torch.Tensor):
        """This rank's ``(BT, H / world)`` block of the input into every rank's gathered input."""
        bt, h, _ = self.sets[index]
        blk = h // self.world
        if x_block.dtype != torch.bfloat16 or tuple(x_block.shape) != (bt, blk) or x_block.stride(1) != 1:
            raise ValueError(f"expected a bf16 ({bt}, {blk}) block with contiguous rows")
        if index in self._pushed:
            # the gathered input of the first pass is still wanted by its backward pass (and by peers' products)
            raise RuntimeError(f"set {index} has already been pushed in this step; call begin_step() between steps")
        self._pushed.add(index)
        lib = _lib.load()
        with torch.cuda.device(self.device):
            _lib.check(lib.forge_push_block(x_block.data_ptr(), bt, blk, x_block.stride(0), self._x_dst[index],
                                            self.rank * blk, h, self._x_arr[index],
                                            self.counters.data_ptr() + 4 * (2 * index), self.epoch.data_ptr(),
                                            self.rank, self.world, _lib.status_word(self.device).data_ptr(),
                                            _lib.current_stream_ptr(self.device)), "forge_push_block")

    def linear(self, index: int, weight: torch.Tensor, full_output: bool = True) -> torch.Tensor:
        """``gather(X) W_r^T`` for the set's pushed input; ``weight``: this rank's ``(V / world, H)`` rows.
        ``full_output``: the ``(BT, V)`` output gathered over the ranks (every rank gets the same), else this
        rank's ``(BT, V / world)`` columns."""
        bt, h, v = self.sets[index]
        vr = v // self.world
        if weight.dtype != torch.bfloat16 or tuple(weight.shape) != (vr, h) or weight.stride(1) != 1:
            raise ValueError(f"expected this rank's bf16 ({vr}, {h}) rows of the weight")
        a = _lib.ForgeLinearGatheredArgs()
        a.X = self.x_buf.data_ptr() + self._x_off[index]
        a.W = weight.data_ptr()
        a.BT, a.H, a.V_r, a.ld_x, a.ld_w = bt, h, vr, h, weight.stride(0)
        a.x_arrivals = self.arrivals.data_ptr() + 4 * (2 * index) * self.world
        a.epoch = self.epoch.data_ptr()
        a.rank, a.world = self.rank, self.world
        status = _lib.status_word(self.device).data_ptr()
        a.status = status
        lib = _lib.load()
        with torch.cuda.device(self.device):
            stream = _lib.current_stream_ptr(self.device)
            if not full_output:
                out = torch.empty(bt, vr, dtype=torch.bfloat16, device=self.device)
                a.y, a.ld_y = out.data_ptr(), vr
                _lib.check(lib.forge_linear_gathered(ctypes.byref(a), stream), "forge_linear_gathered")
                return out
            a.y = None
            a.y_dst, a.y_col, a.y_pitch = self._y_dst[index], self.rank * vr, v
            a.y_arrivals = self._y_arr[index]
            a.y_counter = self.counters.data_ptr() + 4 * (2 * index + 1)
            _lib.check(lib.forge_linear_gathered(ctypes.byref(a), stream), "forge_linear_gathered")
            out = torch.empty(bt, v, dtype=torch.bfloat16, device=self.device)
            _lib.check(lib.forge_collect(self.y_buf.data_ptr() + self._y_off[index], v,
                                         self.arrivals.data_ptr() + 4 * (2 * index + 1) * self.world,
                                         self.epoch.data_ptr(), out.data_ptr(), bt, v, v, self.world, status, stream),
                       "forge_collect")
        return out
