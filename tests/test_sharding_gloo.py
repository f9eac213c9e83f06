"""Batch x head sharding across ranks: partition arithmetic and the optional all-gather, on CPU
ranks with the gloo backend (world size 2 and 3)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sageattention.sharding import gather_units, partition_units, sageattn_sharded


def test_partition_covers_all_units_once():
    for units in (1, 7, 48, 192):
        for world in (1, 2, 3, 4, 8):
            spans = [partition_units(units, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == units
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a1 >= a0
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert [partition_units(192, 8, r) for r in (0, 7)] == [(0, 24), (168, 192)]
    with pytest.raises(ValueError):
        partition_units(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_attn(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None, smooth_k=True):
    # stands in for the CUDA call on CPU ranks: exact softmax attention per unit
    if k.shape[1] != q.shape[1]:                       # grouped-query heads
        g = q.shape[1] // k.shape[1]
        k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    return torch.nn.functional.scaled_dot_product_attention(
        q.float(), k.float(), v.float(), is_causal=is_causal).to(q.dtype)


def _worker(rank, world, port, units, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        q, k, v = (torch.randn(1, units, 40, 128, generator=g).half() for _ in range(3))
        lo, hi = partition_units(units, world, rank)
        local = sageattn_sharded(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], attn_fn=_fake_attn)
        assert local.shape == (1, hi - lo, 40, 128)
        full = sageattn_sharded(q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], gather=True, attn_fn=_fake_attn)
        want = _fake_attn(q, k, v)
        assert full.shape == want.shape
        assert torch.equal(full, want)
        assert torch.equal(gather_units(local), want)
        # grouped-query heads: key/value units are partitioned, each carries `grp` query units
        grp = 2
        qg = torch.randn(1, grp * units, 24, 128, generator=g).half()
        out = sageattn_sharded(qg[:, grp * lo:grp * hi], k[:, lo:hi], v[:, lo:hi], gather=True, attn_fn=_fake_attn)
        assert torch.equal(out, _fake_attn(qg, k, v))
        ret[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,units", [(2, 6), (3, 7)])
def test_sharded_call_and_gather(world, units):
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, units, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        for p in procs:
            if p.is_alive():
                p.terminate()
            assert p.exitcode == 0
        assert all(ret.get(r) for r in range(world))


def test_scaling_configuration_partition():
    """The 192 (batch, head) units of the B=4, H=48 scaling configuration split evenly over
    1, 2, 4 and 8 ranks: 192 / 96 / 48 / 24 units each, contiguous, covering every unit once."""
    from sageattention.sharding import partition_units
    for world, per in ((1, 192), (2, 96), (4, 48), (8, 24)):
        ranges = [partition_units(192, world, r) for r in range(world)]
        assert all(hi - lo == per for lo, hi in ranges)
        assert ranges[0][0] == 0 and ranges[-1][1] == 192
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
