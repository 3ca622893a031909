"""Sharded checkpoints of the row-parallel layer: a checkpoint written by R ranks loads on any other
number of ranks (host logic only; no process group is needed because every rank is built explicitly)."""

import pytest
import torch

from forge_b200.tensor_parallel import RowShardedFusedLinear, load_resharded, row_range, shard_state_dict

V, H = 136, 128   # ragged: 17 groups of 8 rows


def _layers(world, mode, full_w):
    out = []
    for r in range(world):
        m = RowShardedFusedLinear.from_full_weight(full_w, rank=r, world=world, state_mode=mode)
        m.local._ensure_state()
        m.local._state.ensure_buffers()
        m.local._state.step = 7
        out.append(m)
    return out


def _fill_state(layers, mode, gen):
    """Give every row-indexed buffer the values of one global tensor, so shards can be compared."""
    names = {"bf16": ("m", "v"), "int8": ("m_q", "v_q", "m_scale", "v_scale"),
             "fp8_block": ("m_q", "v_q", "m_scale", "v_scale")}[mode]
    full = {}
    for n in names:
        proto = getattr(layers[0].local._state, n)
        shape = (V,) + tuple(proto.shape[1:])
        vals = torch.randint(-100, 100, shape, generator=gen).float()
        full[n] = vals.to(proto.dtype) if proto.dtype != torch.float8_e4m3fn else (vals / 64).to(proto.dtype)
        for m in layers:
            getattr(m.local._state, n).copy_(full[n][m.row_start:m.row_end])
    return full


@pytest.mark.parametrize("mode", ["bf16", "int8", "fp8_block"])
@pytest.mark.parametrize("src_world,dst_world", [(4, 2), (2, 3), (1, 4), (3, 1)])
def test_reshard_round_trip(mode, src_world, dst_world):
    gen = torch.Generator().manual_seed(3)
    full_w = torch.randn(V, H, generator=gen)
    src = _layers(src_world, mode, full_w)
    full = _fill_state(src, mode, gen)
    shards = [shard_state_dict(m) for m in src]
    dst = _layers(dst_world, mode, torch.zeros(V, H))
    for m in dst:
        load_resharded(m, list(reversed(shards)))     # order must not matter
        a, b = row_range(V, m.rank, dst_world)
        assert torch.equal(m.local.weight.data, full_w[a:b])
        assert m.local._state.step == 7
        for n, t in full.items():
            got = getattr(m.local._state, n)
            assert got.shape[0] == b - a
            assert torch.equal(got.view(torch.uint8) if got.dtype == torch.float8_e4m3fn else got,
                               t[a:b].view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t[a:b]), n


def test_missing_rows_and_shape_mismatch_are_errors():
    full_w = torch.randn(V, H)
    src = _layers(4, "bf16", full_w)
    shards = [shard_state_dict(m) for m in src]
    dst = _layers(2, "bf16", full_w)[0]
    with pytest.raises(ValueError, match="missing"):
        load_resharded(dst, shards[1:])
    other = RowShardedFusedLinear.from_full_weight(torch.randn(V + 8, H), rank=0, world=1)
    with pytest.raises(ValueError, match="another shape"):
        load_resharded(other, shards)


def test_per_tensor_fp8_only_loads_with_the_same_sharding():
    full_w = torch.randn(V, H)
    src = _layers(2, "fp8", full_w)
    for i, m in enumerate(src):
        m.local._state.m_scale.fill_(0.5 + i)
    shards = [shard_state_dict(m) for m in src]
    same = _layers(2, "fp8", torch.zeros(V, H))
    for m in same:
        load_resharded(m, shards)
        assert float(m.local._state.m_scale) == 0.5 + m.rank
    with pytest.raises(ValueError, match="fp8_block"):
        load_resharded(_layers(4, "fp8", full_w)[1], shards)
