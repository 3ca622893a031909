"""Row-sharded tensor parallelism for the fused weight-gradient + optimizer path.

The reference has no distributed code (no ``torch.distributed`` call site anywhere in its tree); this
mode is new.  It shards every weight along its OUTPUT rows V -- the only axis along which
``dW[v, :] = sum_bt dY[bt, v] X[bt, :]`` and its optimizer update need no gradient reduction -- so rank
``r`` of ``R`` owns rows ``[r V/R, (r+1) V/R)`` of W, of the moments and of their per-row scale arrays
(``row_range``).  Activations travel feature-sharded between linears:

    before a linear   all-gather X          (BT, H/R) per rank -> (BT, H) in local memory  [NCCL]
    forward           Y_r = X W_r^T         (BT, V/R), stays sharded
    backward          dW_r = dY_r^T X       local fused kernel, no communication
                      dX = sum_r dY_r W_r   reduce-scatter over ranks -> (BT, H/R)          [NCCL]

One process per GPU; ``torch.distributed`` (NCCL over NVLink / NVSwitch on GPUs, gloo on CPU for the
host-logic tests).  A gathered tensor always lands in this rank's own memory before any kernel reads
it; no kernel of this package dereferences a peer's memory.

Parity: results equal the single-GPU run row for row, because each row's update depends on no other
row.  The one exception is ``state_mode="fp8"`` (one scale per tensor): each rank keeps the scale
of its own shard, so codes differ from a single-GPU run; use ``"fp8_block"`` where they must match.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from forge_b200.module import FusedLinear


def row_range(V: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of a (V, H) weight owned by `rank`: contiguous blocks, sizes differing by at most one
    8-row group so that every shard keeps the 16-byte row-pitch alignment of its dY slice."""
    if V % 8 != 0:
        raise ValueError(f"V ({V}) must be a multiple of 8 to be row-sharded")
    groups = V // 8
    base, extra = divmod(groups, world)
    start = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return start * 8, (start + count) * 8


def feature_range(H: int, rank: int, world: int) -> tuple[int, int]:
    """Columns of a feature-sharded activation held by `rank` (equal shards; H % world == 0)."""
    if H % world != 0:
        raise ValueError(f"feature dimension {H} is not divisible by the world size {world}")
    s = H // world
    return rank * s, (rank + 1) * s


def all_gather_features(x_shard: torch.Tensor, group=None) -> torch.Tensor:
    """(…, H/R) per rank -> (…, H) on every rank (feature-concatenated)."""
    world = dist.get_world_size(group)
    if world == 1:
        return x_shard
    x_shard = x_shard.contiguous()
    lead = x_shard.shape[:-1]
    flat = torch.empty((world * x_shard.shape[0],) + tuple(x_shard.shape[1:]), dtype=x_shard.dtype,
                       device=x_shard.device)
    dist.all_gather_into_tensor(flat, x_shard, group=group)     # rank blocks concatenated along dim 0
    out = flat.view((world,) + tuple(x_shard.shape))
    # (R, …, H/R) -> (…, R, H/R) -> (…, H)
    nd = x_shard.dim()
    perm = tuple(range(1, nd)) + (0, nd)
    return out.permute(*perm).reshape(*lead, world * x_shard.shape[-1])


def reduce_scatter_features(x_full: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the ranks' (…, H) partial results, scattered by feature block: returns (…, H/R)."""
    world = dist.get_world_size(group)
    if world == 1:
        return x_full
    lead = x_full.shape[:-1]
    H = x_full.shape[-1]
    s = H // world
    # (…, R, H/R) -> (R, …, H/R) so that block r is contiguous
    nd = x_full.dim()
    blocks = x_full.reshape(*lead, world, s).permute(nd - 1, *range(nd - 1), nd).contiguous()
    if dist.get_backend(group) == "gloo":
        # gloo (CPU host-logic tests) has no reduce-scatter: all-reduce and keep this rank's block
        dist.all_reduce(blocks, op=dist.ReduceOp.SUM, group=group)
        return blocks[dist.get_rank(group)].clone()
    out = torch.empty(tuple(lead) + (s,), dtype=x_full.dtype, device=x_full.device)
    dist.reduce_scatter_tensor(out, blocks.view((world * blocks.shape[1],) + tuple(blocks.shape[2:])),
                               op=dist.ReduceOp.SUM, group=group)
    return out


class _GatherX(torch.autograd.Function):
    """all-gather in forward, reduce-scatter of the gradient in backward."""

    @staticmethod
    def forward(ctx, x_shard, group):
        ctx.group = group
        return all_gather_features(x_shard, group)

    @staticmethod
    def backward(ctx, grad_full):
        return reduce_scatter_features(grad_full.contiguous(), ctx.group), None


class _ShardedLinearFusedScatter(torch.autograd.Function):
    """A row-sharded linear whose backward forms the reduce-scattered input gradient in one step:
    forward = all-gather of the feature shards + ``F.linear`` on the local rows; backward = this
    library's dX GEMM with the reduce-scatter fused into its epilogue (``forge_b200.peer``: tiles go
    straight into the owner ranks' receive buffers over peer memory, the owner sums them in rank order)
    followed by the fused update of the local rows.  Only the plain fused branch; the module falls back
    to gather + ``FusedLinearFunction`` + NCCL reduce-scatter for everything else."""

    @staticmethod
    def forward(ctx, x_shard, weight, local, scatter, index, group):
        x = all_gather_features(x_shard, group)
        ctx.save_for_backward(x, weight)
        ctx.local, ctx.scatter, ctx.index, ctx.shard_shape = local, scatter, index, x_shard.shape
        return torch.nn.functional.linear(x, weight)

    @staticmethod
    def backward(ctx, grad_output):
        from forge_b200.autograd import _apply_fused
        x, weight = ctx.saved_tensors
        local = ctx.local
        dy2d = grad_output.reshape(-1, grad_output.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        x2d = x.reshape(-1, x.shape[-1])
        # before the in-place update of `weight` on this stream
        dx_shard = ctx.scatter.run(ctx.index, [(dy2d, weight.data)]).view(ctx.shard_shape)
        if local._update_group is not None:
            local._update_group.add(weight, lambda: _apply_fused(dy2d, x2d, weight, local._state, local._config))
        else:
            _apply_fused(dy2d, x2d, weight, local._state, local._config)
        return dx_shard, None, None, None, None, None


class _ShardedLinearFusedGather(torch.autograd.Function):
    """A row-sharded linear on a feature-sharded input whose forward has both of its all-gathers fused in
    (``forge_b200.peer.GatheredLinear``): the input block is pushed to every rank, the GEMM consumes the
    blocks as they arrive and stores its output tiles into every rank's gathered output.  Input
    ``(…, H / R)``, output the full ``(…, V)`` (the same on every rank).  Backward: this rank's columns
    of the output gradient, then as ``_ShardedLinearFusedScatter`` (or library GEMM + NCCL
    reduce-scatter when no fused scatter is attached)."""

    @staticmethod
    def forward(ctx, x_shard, weight, layer):
        fwd, idx = layer._gather, layer._gather_index
        x2d = x_shard.reshape(-1, x_shard.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        fwd.push(idx, x2d)
        y = fwd.linear(idx, weight.data, full_output=True)
        # the gathered input lives in the set's buffer until the next step begins: the backward reads it there
        ctx.save_for_backward(fwd.gathered_input(idx), weight)
        ctx.layer, ctx.shard_shape = layer, x_shard.shape
        return y.view(*x_shard.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, grad_full):
        from forge_b200.autograd import _apply_fused
        x2d, weight = ctx.saved_tensors
        layer = ctx.layer
        local = layer.local
        vr = weight.shape[0]
        dy2d = grad_full.reshape(-1, grad_full.shape[-1])[:, layer.rank * vr:(layer.rank + 1) * vr].contiguous()
        # before the in-place update of `weight` on this stream
        if layer._scatter is not None:
            dx_shard = layer._scatter.run(layer._scatter_index, [(dy2d, weight.data)])
        else:
            dx_shard = reduce_scatter_features(dy2d @ weight.data, layer.group)
        if local._update_group is not None:
            local._update_group.add(weight, lambda: _apply_fused(dy2d, x2d, weight, local._state, local._config))
        else:
            _apply_fused(dy2d, x2d, weight, local._state, local._config)
        return dx_shard.view(ctx.shard_shape), None, None


class _ShardedSetFusedAllReduce(torch.autograd.Function):
    """Several row-sharded linears on one REPLICATED input (q / k / v; gate / up).  Forward: one
    ``F.linear`` per member.  Backward: ONE launch of this library's dX GEMM accumulates
    ``sum_i dY_i W_i`` over the members and stores every tile into every rank's receive buffer; each
    rank then adds the ranks' partial sums itself (a fused all-reduce over peer memory: no per-linear
    GEMMs, no autograd additions, no NCCL all-reduce); the members' fused updates follow."""

    @staticmethod
    def forward(ctx, x, scatter, index, locals_, *weights):
        ctx.save_for_backward(x, *weights)
        ctx.locals_, ctx.scatter, ctx.index = locals_, scatter, index
        return tuple(torch.nn.functional.linear(x, w) for w in weights)

    @staticmethod
    def backward(ctx, *grads):
        from forge_b200.autograd import _apply_fused
        x, *weights = ctx.saved_tensors
        x2d = x.reshape(-1, x.shape[-1])
        dys = []
        for g, w in zip(grads, weights):
            d = g.reshape(-1, w.shape[0])
            dys.append(d if d.is_contiguous() else d.contiguous())
        # before the in-place updates of the weights on this stream
        dx = ctx.scatter.run(ctx.index, [(d, w.data) for d, w in zip(dys, weights)]).view(x.shape)
        for d, w, loc in zip(dys, weights, ctx.locals_):
            if loc._update_group is not None:
                loc._update_group.add(w, lambda d=d, w=w, loc=loc: _apply_fused(d, x2d, w, loc._state, loc._config))
            else:
                _apply_fused(d, x2d, w, loc._state, loc._config)
        return (dx, None, None, None) + (None,) * len(weights)


class RowShardedLinearSet(nn.Module):
    """Row-sharded linears that consume the same replicated activation.  Without a fused scatter attached
    (or outside its conditions) it runs the members one by one; ``partial_input_grad`` tells the caller
    whether the input gradient it gets back still has to be summed over the ranks.  The set does not
    own its members (no parameters of its own), so a model that also holds them by name keeps one entry
    per layer in its state dict."""

    def __init__(self, members):
        super().__init__()
        if any(m.gather_input for m in members):
            raise ValueError("the members of a set take a replicated input (gather_input=False)")
        if len({m.in_features for m in members}) != 1:
            raise ValueError("the members of a set share one input")
        self.members = tuple(members)       # not registered here: the members stay owned by whoever built them
        self._scatter, self._scatter_index = None, None

    def attach_fused_scatter(self, scatter, index: int):
        self._scatter, self._scatter_index = scatter, index

    def fused(self, x) -> bool:
        if self._scatter is None or not x.is_cuda or x.dtype != torch.bfloat16 or len(self.members) > 4:
            return False
        for m in self.members:
            loc = m.local
            if not (m.world > 1 and loc.training and loc._config is not None and not loc._is_accumulating
                    and loc.use_fused_backward and loc.bias is None and loc.weight.dtype == torch.bfloat16):
                return False
            loc._ensure_state()
            if loc._state._pending_grad is not None:
                return False
        return True

    def forward(self, x):
        """Returns ``(outputs, complete)``: the members' outputs and whether the input gradient that will
        come back is already summed over the ranks (fused path) or still partial (plain path)."""
        if self.fused(x):
            locals_ = [m.local for m in self.members]
            outs = _ShardedSetFusedAllReduce.apply(x, self._scatter, self._scatter_index, locals_,
                                                   *[loc.weight for loc in locals_])
            return outs, True
        return tuple(m(x) for m in self.members), False


class RowShardedFusedLinear(nn.Module):
    """A ``FusedLinear`` holding only this rank's rows of the weight (and of its optimizer state).

    ``forward`` takes the feature-sharded activation (…, H/R), gathers it, and returns this rank's
    slice (…, V_r) of the output.  Its backward runs the fused update on the local rows and returns
    the reduce-scattered input gradient (…, H/R).  With ``gather_input=False`` the caller passes an
    already gathered (…, H) activation (several linears sharing one gather, e.g. q/k/v or gate/up)
    and receives the full-width partial dX, to be summed once and reduce-scattered by the caller.
    """

    def __init__(self, in_features, out_features, rank=None, world=None, group=None, gather_input=True,
                 dtype=None, device=None, **fused_kwargs):
        super().__init__()
        self.group = group
        self.world = world if world is not None else dist.get_world_size(group)
        self.rank = rank if rank is not None else dist.get_rank(group)
        self.in_features, self.out_features = in_features, out_features
        self.row_start, self.row_end = row_range(out_features, self.rank, self.world)
        self.gather_input = gather_input
        # the shard is created where it will live: a large shard is never materialised on the host
        if device is not None:
            with torch.device(device):
                self.local = FusedLinear(in_features, self.row_end - self.row_start, **fused_kwargs)
        else:
            self.local = FusedLinear(in_features, self.row_end - self.row_start, **fused_kwargs)
        if dtype is not None:
            self.local = self.local.to(dtype=dtype)
        self._scatter, self._scatter_index = None, None      # see attach_fused_scatter
        self._gather, self._gather_index = None, None        # see attach_fused_gather

    @classmethod
    def from_full_weight(cls, weight: torch.Tensor, rank=None, world=None, group=None, **kw):
        """Build from the full (V, H) weight: keeps a copy of this rank's rows only."""
        V, H = weight.shape
        m = cls(H, V, rank=rank, world=world, group=group, **kw)
        with torch.no_grad():
            m.local.weight.data = weight[m.row_start:m.row_end].detach().clone()
        return m

    @property
    def weight(self):
        return self.local.weight

    def attach_fused_scatter(self, scatter, index: int):
        """Use ``scatter`` (a ``forge_b200.peer.DgradReduceScatter``), set ``index``, for this layer's input
        gradient instead of a library GEMM followed by an NCCL reduce-scatter.  For layers that gather
        their input (``gather_input=True``) with bf16 weights and no bias."""
        self._scatter, self._scatter_index = scatter, index

    def attach_fused_gather(self, gather, index: int):
        """Use ``gather`` (a ``forge_b200.peer.GatheredLinear``), set ``index``, for this layer's forward:
        the all-gather of its input and of its output are fused into the GEMM.  The layer then takes the
        feature-sharded input and returns the FULL ``(…, V)`` output (``returns_full_output``), so the
        caller must not gather it again.  Same conditions as ``attach_fused_scatter``.  One training forward
        per step and set (``GatheredLinear.begin_step`` between steps): the gathered input stays in the set's
        buffer for the backward pass, so a second forward before it -- activation recomputation, two
        micro-batches -- is refused rather than allowed to overwrite it."""
        self._gather, self._gather_index = gather, index

    def _fused_conditions(self, x) -> bool:
        loc = self.local
        if not (self.gather_input and self.world > 1 and loc.training and loc._config is not None
                and not loc._is_accumulating and loc.use_fused_backward and loc.bias is None and x.is_cuda
                and x.dtype == torch.bfloat16 and loc.weight.dtype == torch.bfloat16):
            return False
        loc._ensure_state()
        return loc._state._pending_grad is None

    def returns_full_output(self, x) -> bool:
        return self._gather is not None and self._fused_conditions(x)

    def forward(self, x):
        sc = self._scatter
        loc = self.local
        if self._gather is not None and self._fused_conditions(x):
            return _ShardedLinearFusedGather.apply(x, loc.weight, self)
        if sc is not None and self._fused_conditions(x):
            return _ShardedLinearFusedScatter.apply(x, loc.weight, loc, sc, self._scatter_index, self.group)
        if self.gather_input and self.world > 1:
            x = _GatherX.apply(x, self.group)
        return self.local(x)

    def gather_full_weight(self) -> torch.Tensor:
        """Reassemble the (V, H) weight on every rank (checkpointing / parity checks)."""
        return gather_rows(self.local.weight.data, self.out_features, self.rank, self.world, self.group)


def gather_rows(shard: torch.Tensor, V: int, rank: int, world: int, group=None) -> torch.Tensor:
    """All-gather row shards of possibly unequal height into the full (V, …) tensor."""
    if world == 1:
        return shard.clone()
    sizes = [row_range(V, r, world) for r in range(world)]
    tallest = max(e - s for s, e in sizes)
    padded = torch.zeros((tallest,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    padded[: shard.shape[0]] = shard
    flat = torch.empty((world * tallest,) + tuple(shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    dist.all_gather_into_tensor(flat, padded, group=group)
    out = flat.view((world, tallest) + tuple(shard.shape[1:]))
    return torch.cat([out[r, : e - s] for r, (s, e) in enumerate(sizes)], dim=0)


# ---------------------------------------------------------------------------------------------
# Checkpoints of row shards.  Every row-indexed tensor (the weight, the moments or their codes, the
# per-(row, block) scale arrays) is saved with the row range it covers, so a checkpoint written by R
# ranks can be loaded by any other number of ranks: a rank assembles its rows from the overlapping
# pieces.  The reference's state_dict (``state.py:179-205``) has neither shards nor fp8 state.
# ---------------------------------------------------------------------------------------------
_SCALAR_KEYS = ("optimizer_type", "step", "quantize_state", "state_mode")


def shard_state_dict(layer: "RowShardedFusedLinear") -> dict:
    """This rank's piece of a sharded checkpoint (tensors cloned to the CPU)."""
    opt = layer.local.get_optimizer_state_dict()
    if opt is not None:
        opt = {k: (v.detach().cpu().clone() if torch.is_tensor(v) else v) for k, v in opt.items()}
    return {"rows": (layer.row_start, layer.row_end), "out_features": layer.out_features,
            "in_features": layer.in_features, "world": layer.world,
            "weight": layer.local.weight.detach().cpu().clone(),
            "bias": None if layer.local.bias is None else layer.local.bias.detach().cpu().clone(),
            "optimizer": opt}


def _rows_from_pieces(pieces, start: int, end: int) -> torch.Tensor:
    """Rows [start, end) cut out of [(row0, row1, tensor with row1 - row0 rows), ...]."""
    parts, at = [], start
    for r0, r1, t in sorted(pieces, key=lambda p: p[0]):
        lo, hi = max(r0, at), min(r1, end)
        if lo < hi:
            if lo != at:
                raise ValueError(f"rows {at}..{lo} are missing from the checkpoint")
            parts.append(t[lo - r0:hi - r0])
            at = hi
    if at != end:
        raise ValueError(f"rows {at}..{end} are missing from the checkpoint")
    return torch.cat(parts, dim=0) if len(parts) > 1 else parts[0].clone()


def load_resharded(layer: "RowShardedFusedLinear", shards: list) -> None:
    """Load this rank's rows from the pieces of a sharded checkpoint (``shard_state_dict`` of every
    rank that wrote it, in any order, written with any world size)."""
    if not shards:
        raise ValueError("no shards given")
    for s in shards:
        if s["out_features"] != layer.out_features or s["in_features"] != layer.in_features:
            raise ValueError("checkpoint belongs to a layer of another shape")
    a, b = layer.row_start, layer.row_end
    dev = layer.local.weight.device
    with torch.no_grad():
        w = _rows_from_pieces([(s["rows"][0], s["rows"][1], s["weight"]) for s in shards], a, b)
        layer.local.weight.data.copy_(w.to(dev))
        if layer.local.bias is not None and shards[0].get("bias") is not None:
            bias = _rows_from_pieces([(s["rows"][0], s["rows"][1], s["bias"]) for s in shards], a, b)
            layer.local.bias.data.copy_(bias.to(dev))
    opts = [s["optimizer"] for s in shards]
    if all(o is None for o in opts):
        return
    if any(o is None for o in opts):
        raise ValueError("some shards carry optimizer state and some do not")
    first = opts[0]
    for o in opts[1:]:
        for k in _SCALAR_KEYS:
            if o.get(k) != first.get(k):
                raise ValueError(f"shards disagree on {k!r}: {o.get(k)!r} vs {first.get(k)!r}")
    merged = {k: first[k] for k in _SCALAR_KEYS if k in first}
    for key, val in first.items():
        if not torch.is_tensor(val):
            continue
        if val.dim() >= 2:      # row-indexed: moments, codes, per-(row, block) scales
            merged[key] = _rows_from_pieces([(s["rows"][0], s["rows"][1], s["optimizer"][key]) for s in shards], a, b)
        else:
            # one scale per tensor (fp8 mode): the codes of a shard are relative to that shard's own
            # scale, so they can only be taken over whole
            exact = [s for s in shards if tuple(s["rows"]) == (a, b)]
            if not exact:
                raise ValueError("per-tensor fp8 state can only be loaded with the sharding it was saved with; "
                                 "use state_mode='fp8_block' for checkpoints that must reshard")
            merged[key] = exact[0]["optimizer"][key].clone()
    layer.local.load_optimizer_state_dict(merged)
