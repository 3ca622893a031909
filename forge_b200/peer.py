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


def _share(t: torch.Tensor, group=None) -> list[torch.Tensor]:
    """Views of every rank's tensor `t` (same shape everywhere) mapped into this process."""
    from torch.multiprocessing.reductions import reduce_tensor
    world, rank = dist.get_world_size(group), dist.get_rank(group)
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
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
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

    def run(self, index: int, members, out: torch.Tensor | None = None, reduce_stream=None) -> torch.Tensor:
        """``reduce_stream``: run the owner's wait-and-sum there (after the GEMM, by an event) so that the
        current stream can go on while the peers' tiles are still arriving; the caller orders its use of
        the result after that stream."""
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
