"""Batch x head sharding on real GPUs: each rank runs the CUDA path on its units, outputs are
all-gathered over NCCL only because the test asks for the whole tensor.  Needs two GPUs (skipped
otherwise); ranks are child processes, rendezvous on 127.0.0.1."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import sageattention
        from sageattention.sharding import partition_units, sageattn_sharded
        g = torch.Generator().manual_seed(0)                       # the same tensors on every rank
        units, grp = 6, 2
        q = torch.randn(1, grp * units, 300, 128, generator=g).half()
        k = torch.randn(1, units, 300, 128, generator=g).half()
        v = torch.randn(1, units, 300, 128, generator=g).half()
        lo, hi = partition_units(units, world, rank)
        dev = torch.device("cuda", rank)
        out = sageattn_sharded(q[:, grp * lo:grp * hi].to(dev), k[:, lo:hi].to(dev), v[:, lo:hi].to(dev),
                               is_causal=True, gather=True)
        whole = sageattention.sageattn(q.to(dev), k.to(dev), v.to(dev), is_causal=True)
        assert out.shape == whole.shape
        assert torch.equal(out, whole)                              # units are independent: bit-identical
        ret[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_call_with_nccl_gather():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        for p in procs:
            if p.is_alive():
                p.terminate()
            assert p.exitcode == 0
        assert all(ret.get(r) for r in range(world))
