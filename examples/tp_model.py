"""A decoder-only transformer (Llama-3.1 / Qwen3 architecture) whose linears are row-sharded over the
ranks of a tensor-parallel group, for the whole-model runs of ``examples/llama_step.py --tp N``.

The reference has no distributed code; this is the harness of the row-sharded mode that
``forge_b200.tensor_parallel`` defines.  Every weight is sharded along its OUTPUT rows -- the one axis
along which the fused weight-gradient + optimizer update needs no gradient reduction -- so rank r holds
rows [r V/R, (r+1) V/R) of q, k, v, o, gate, up, down and lm_head with their optimizer moments, and
updates them locally inside its backward pass.  Data flow of one block (h is replicated):

    x1 = norm(h)                         replicated
    q_r, k_r, v_r = x1 Wq_r^T, ...       this rank's heads; backward: all-reduce of the partial dX
    a_r = attention(q_r, k_r, v_r)       head-local
    a = all-gather(a_r)                  backward: reduce-scatter of the partial dX of o
    o_r = a Wo_r^T                       (BT, hidden / R)
    h = h + all-gather(o_r)              backward: each rank keeps its slice, no communication
    x2 = norm(h); g_r, u_r = x2 Wg_r^T, x2 Wu_r^T; t_r = silu(g_r) u_r
    t = all-gather(t_r); d_r = t Wd_r^T; h = h + all-gather(d_r)

and the head: logits_r = norm(h) Wlm_r^T over this rank's vocabulary rows, with a vocabulary-parallel
cross entropy (all-reduce of the row maxima, of the sums of exponentials and of the target logits).
Embedding and norm weights are replicated; the gradients that reach them are complete on every rank
(every dX that enters the replicated part has been summed over the ranks first), so they need no
all-reduce -- except the per-head q / k norm weights of Qwen3, whose gradients are sums over heads that
live on different ranks.  Collectives: NCCL through ``torch.distributed``; every kernel reads local
memory only.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from forge_b200.tensor_parallel import (RowShardedFusedLinear, RowShardedLinearSet, all_gather_features, feature_range,
                                        reduce_scatter_features)


class _ToShardedLinears(torch.autograd.Function):
    """A replicated activation entering row-sharded linears: identity forward; the linears return
    partial input gradients (each from its own rows), summed over the ranks in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _GatherForShardedLinear(torch.autograd.Function):
    """Feature shards -> full activation consumed by a row-sharded linear: the gradient that comes
    back is a partial sum per rank, so backward is a reduce-scatter."""

    @staticmethod
    def forward(ctx, x_shard, group):
        ctx.group = group
        return all_gather_features(x_shard, group)

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_features(g.contiguous(), ctx.group), None


class _GatherIntoReplicated(torch.autograd.Function):
    """Feature shards -> full activation consumed by replicated computation (the residual stream):
    every rank then holds the same full gradient and keeps the slice of its own shard."""

    @staticmethod
    def forward(ctx, x_shard, group):
        ctx.group = group
        ctx.width = x_shard.shape[-1]
        return all_gather_features(x_shard, group)

    @staticmethod
    def backward(ctx, g):
        r = dist.get_rank(ctx.group)
        return g[..., r * ctx.width:(r + 1) * ctx.width].contiguous(), None


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Mean next-token cross entropy from this rank's slice of the logits (rows [v0, v1) of the
    vocabulary): three small all-reduces (max, sum of exponentials, target logit)."""

    @staticmethod
    def forward(ctx, logits_r, targets, v0, group):
        lf = logits_r.float()
        m = lf.max(dim=-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m[:, None])
        s = e.sum(dim=-1)
        dist.all_reduce(s, group=group)
        local = (targets >= v0) & (targets < v0 + lf.shape[-1])
        idx = (targets - v0).clamp(0, lf.shape[-1] - 1)
        t = torch.where(local, lf.gather(1, idx[:, None])[:, 0], torch.zeros_like(m))
        dist.all_reduce(t, group=group)
        loss = (torch.log(s) + m - t).mean()
        p = e / s[:, None]
        p.scatter_add_(1, idx[:, None], -local.to(p.dtype)[:, None])      # minus one at the target, where it is local
        ctx.save_for_backward(p)
        ctx.dtype = logits_r.dtype
        return loss

    @staticmethod
    def backward(ctx, gout):
        (p,) = ctx.saved_tensors
        return (p * (gout / p.shape[0])).to(ctx.dtype), None, None, None


class _LibraryRMSNorm(torch.autograd.Function):
    """RMSNorm through the library's kernels (one launch forward, two backward) instead of a chain of
    elementwise torch kernels on fp32 copies of the activation."""

    @staticmethod
    def forward(ctx, x, gamma, eps):
        from forge_b200.rmsnorm_linear import rmsnorm_forward
        ctx.save_for_backward(x, gamma)
        ctx.eps = eps
        return rmsnorm_forward(x, gamma, eps)

    @staticmethod
    def backward(ctx, g):
        from forge_b200.rmsnorm_linear import rmsnorm_backward
        x, gamma = ctx.saved_tensors
        dx, dgamma = rmsnorm_backward(x, gamma, g.contiguous(), ctx.eps)
        return dx, dgamma, None


class RMSNorm(nn.Module):
    library_kernels = True      # False: torch ops everywhere

    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        if (RMSNorm.library_kernels and x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and x.shape[-1] >= 1024 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384):
            return _LibraryRMSNorm.apply(x, self.weight, self.eps)
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


def _rope(x, cos, sin):
    # x: (B, heads, T, D); rotate-half convention
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return x * cos + rot * sin


class Block(nn.Module):
    def __init__(self, cfg, group, state_mode, dtype, device):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group)
        hid, hd = cfg["hidden"], cfg["head_dim"]
        self.hd = hd
        self.nq, self.nkv = cfg["q_heads"] // self.world, cfg["kv_heads"] // self.world
        if cfg["q_heads"] % self.world or cfg["kv_heads"] % self.world:
            raise ValueError("the head counts must be divisible by the tensor-parallel size")
        kw = dict(group=group, gather_input=False, dtype=dtype, device=device, optimizer_type="adamw", state_mode=state_mode,
                  weight_decay=0.01)
        self.norm1 = RMSNorm(hid, cfg["eps"])
        self.q = RowShardedFusedLinear(hid, cfg["q_heads"] * hd, **kw)
        self.k = RowShardedFusedLinear(hid, cfg["kv_heads"] * hd, **kw)
        self.v = RowShardedFusedLinear(hid, cfg["kv_heads"] * hd, **kw)
        self.o = RowShardedFusedLinear(cfg["q_heads"] * hd, hid, **kw)
        self.norm2 = RMSNorm(hid, cfg["eps"])
        self.gate = RowShardedFusedLinear(hid, cfg["ffn"], **kw)
        self.up = RowShardedFusedLinear(hid, cfg["ffn"], **kw)
        self.down = RowShardedFusedLinear(cfg["ffn"], hid, **kw)
        # the members that share a replicated input, for the fused input gradient (use_fused_scatter)
        self.qkv_set = RowShardedLinearSet([self.q, self.k, self.v])
        self.gu_set = RowShardedLinearSet([self.gate, self.up])
        self.qk_norm = cfg.get("qk_norm", False)
        if self.qk_norm:
            self.q_norm, self.k_norm = RMSNorm(hd, cfg["eps"]), RMSNorm(hd, cfg["eps"])

    def forward(self, h, cos, sin):
        B, T, _ = h.shape
        x = self.norm1(h)
        if self.qkv_set.fused(x):
            (q, k, v), _ = self.qkv_set(x)           # its backward returns the input gradient summed over the ranks
        else:
            x = _ToShardedLinears.apply(x, self.group)
            q, k, v = self.q(x), self.k(x), self.v(x)
        q = q.view(B, T, self.nq, self.hd)
        k = k.view(B, T, self.nkv, self.hd)
        v = v.view(B, T, self.nkv, self.hd)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.nq != self.nkv)
        a = a.transpose(1, 2).reshape(B, T, self.nq * self.hd)
        # (with a fused scatter attached, o and down gather their own input and return the scattered gradient)
        if self.o.returns_full_output(a):        # fused gathers: sharded input in, full output out
            h = h + self.o(a)
        else:
            o = self.o(a) if self.o.gather_input else self.o(_GatherForShardedLinear.apply(a, self.group))
            h = h + _GatherIntoReplicated.apply(o, self.group)
        x = self.norm2(h)
        if self.gu_set.fused(x):
            (gate, up), _ = self.gu_set(x)
        else:
            x = _ToShardedLinears.apply(x, self.group)
            gate, up = self.gate(x), self.up(x)
        t = F.silu(gate) * up
        if self.down.returns_full_output(t):
            return h + self.down(t)
        d = self.down(t) if self.down.gather_input else self.down(_GatherForShardedLinear.apply(t, self.group))
        return h + _GatherIntoReplicated.apply(d, self.group)


class TPDecoder(nn.Module):
    """``cfg``: dict with vocab, hidden, ffn, layers, q_heads, kv_heads, head_dim, eps, rope_theta, qk_norm."""

    def __init__(self, cfg, group=None, state_mode="bf16", dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg, self.group = cfg, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.embed = nn.Embedding(cfg["vocab"], cfg["hidden"], dtype=dtype, device=device)
        self.layers = nn.ModuleList([Block(cfg, group, state_mode, dtype, device) for _ in range(cfg["layers"])])
        self.norm = RMSNorm(cfg["hidden"], cfg["eps"])
        self.lm_head = RowShardedFusedLinear(cfg["hidden"], cfg["vocab"], group=group, gather_input=False, dtype=dtype,
                                             device=device, optimizer_type="adamw", state_mode=state_mode, weight_decay=0.01)
        self.to(device)
        for m in self.modules():
            if isinstance(m, RMSNorm):
                m.weight.data = m.weight.data.to(dtype)
        self._init_weights()

    def _init_weights(self):
        # the replicated parameters get the same values on every rank, the shards their own
        g = torch.Generator(device=self.embed.weight.device).manual_seed(1234)
        self.embed.weight.data.normal_(0.0, 0.02, generator=g)
        gs = torch.Generator(device=self.embed.weight.device).manual_seed(99 + self.rank)
        for m in self.modules():
            if isinstance(m, RowShardedFusedLinear):
                m.local.weight.data.normal_(0.0, 0.02, generator=gs)

    def use_fused_scatter(self, tokens: int, replicated_sets: bool = True):
        """Form the input gradients of o and down with the reduce-scatter fused into this library's dX
        GEMM (``forge_b200.peer``) instead of a library GEMM + NCCL reduce-scatter, and those of q / k / v
        and gate / up (replicated input) with one GEMM launch per set whose tiles go to every rank, instead
        of one library GEMM per linear, autograd's additions and an NCCL all-reduce.  ``tokens`` = batch x
        sequence length of the steps to come (the receive buffers are sized for it); ``replicated_sets=False``
        leaves q / k / v and gate / up on the library path.  Collective."""
        from forge_b200.peer import DgradReduceScatter
        sets, layers = [], []
        for blk in self.layers:
            for lin in (blk.o, blk.down):                 # input gathered from feature shards: reduce-scatter
                sets.append((tokens, lin.in_features))
                layers.append(lin)
            for group in (blk.qkv_set, blk.gu_set) if replicated_sets else ():       # replicated input: all-reduce
                sets.append((tokens, group.members[0].in_features, "allreduce"))
                layers.append(group)
        self.fused_scatter = DgradReduceScatter(sets, group=self.group, device=self.embed.weight.device)
        for i, lin in enumerate(layers):
            if isinstance(lin, RowShardedFusedLinear):
                lin.gather_input = True
            lin.attach_fused_scatter(self.fused_scatter, i)
        return self

    def use_fused_gather(self, tokens: int):
        """Form the outputs of o and down with both all-gathers (of the feature-sharded input and of the
        row-sharded output) fused into this library's forward GEMM (``forge_b200.peer.GatheredLinear``)
        instead of NCCL all-gather + library GEMM + NCCL all-gather.  Collective."""
        from forge_b200.peer import GatheredLinear
        layers = [lin for blk in self.layers for lin in (blk.o, blk.down)]
        self.fused_gather = GatheredLinear([(tokens, lin.in_features, lin.out_features) for lin in layers],
                                           group=self.group, device=self.embed.weight.device)
        for i, lin in enumerate(layers):
            lin.gather_input = True
            lin.attach_fused_gather(self.fused_gather, i)
        return self

    def head_sharded_norm_params(self):
        """Replicated parameters whose gradients are partial sums per rank (per-head q / k norms)."""
        return [p for blk in self.layers if blk.qk_norm for p in (blk.q_norm.weight, blk.k_norm.weight)]

    def forward(self, ids):
        B, T = ids.shape
        hd, theta = self.cfg["head_dim"], self.cfg["rope_theta"]
        inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=ids.device, dtype=torch.float32) / hd))
        ang = torch.arange(T, device=ids.device, dtype=torch.float32)[:, None] * inv[None, :]
        ang = torch.cat([ang, ang], dim=-1)
        cos, sin = ang.cos().to(self.embed.weight.dtype), ang.sin().to(self.embed.weight.dtype)
        if getattr(self, "fused_scatter", None) is not None and self.training:
            self.fused_scatter.begin_step()      # this step's arrivals are told from the last one's by the epoch
        if getattr(self, "fused_gather", None) is not None and self.training:
            self.fused_gather.begin_step()
        h = self.embed(ids)
        for blk in self.layers:
            h = blk(h, cos, sin)
        x = _ToShardedLinears.apply(self.norm(h), self.group)
        logits_r = self.lm_head(x)                               # (B, T, vocab / R)
        v0 = self.lm_head.row_start
        flat = logits_r[:, :-1].reshape(-1, logits_r.shape[-1])
        return _VocabParallelCrossEntropy.apply(flat, ids[:, 1:].reshape(-1), v0, self.group)


CONFIGS = {
    "llama3.1-8b": dict(vocab=128256, hidden=4096, ffn=14336, layers=32, q_heads=32, kv_heads=8, head_dim=128, eps=1e-5,
                        rope_theta=500000.0, qk_norm=False),
    "qwen3-32b": dict(vocab=151936, hidden=5120, ffn=25600, layers=64, q_heads=64, kv_heads=8, head_dim=128, eps=1e-6,
                      rope_theta=1000000.0, qk_norm=True),
}
