"""Peer-memory collectives against NCCL on 2+ GPUs (skipped with fewer): bitwise all-gather,
deterministic rank-order reduce-scatter, and a missing peer signal that must time out cleanly."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import ops
        from flex_shard_b200.parallel.comm import Comm, plan_reduction
        from flex_shard_b200.parallel.symm import SymmComm
        from flex_shard_b200.placement_contract import GradientReduction

        dev = torch.device("cuda", rank)
        g = dist.group.WORLD
        sc, nc = SymmComm(g, rank, world, dev), Comm(g, rank, world, dev)
        torch.manual_seed(rank)
        res = {}
        for n in (1024, 1 << 20, 3 * (1 << 20) + 16):
            x = torch.randn(n, device=dev).bfloat16()
            a = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
            b = torch.empty_like(a)
            sc.all_gather_into_tensor(a, x)
            nc.all_gather_into_tensor(b, x)
            res[f"ag{n}"] = bool(torch.equal(a, b))
        plan = plan_reduction(GradientReduction(), world, torch.float32)
        for n in (4096, 1 << 20):
            gsend = torch.randn(world * n, device=dev)
            o1 = torch.empty(n, device=dev)
            o2 = torch.empty(n, device=dev)
            o3 = torch.empty(n, device=dev)
            sc.reduce_scatter_tensor(o1, gsend.clone(), plan)
            sc.reduce_scatter_tensor(o3, gsend.clone(), plan)
            nc.reduce_scatter_tensor(o2, gsend.clone(), plan)
            res[f"rs{n}_close"] = float((o1 - o2).abs().max())
            res[f"rs{n}_deterministic"] = bool(torch.equal(o1, o3))
        torch.cuda.synchronize()
        ops.check_status()
        # a flag that nothing sets: the wait gives up after its (shortened) limit and reports it
        reg = sc._ag
        reg.max_polls = 2000
        reg.wait(900, 1)
        torch.cuda.synchronize()
        try:
            ops.check_status()
            res["timeout_reported"] = False
        except ops.NativeError as e:
            res["timeout_reported"] = "peer" in str(e)
        # the context is still usable afterwards
        res["alive"] = float(torch.ones(4, device=dev).sum()) == 4.0
        dist.barrier()
        torch.save(res, os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symm_collectives_match_nccl(tmp_path):
    import torch.multiprocessing as mp

    from tests.common import free_port

    world = 2
    mp.spawn(_worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        for k, v in res.items():
            if k.startswith("ag") or k.endswith("deterministic") or k in ("timeout_reported", "alive"):
                assert v is True, (k, v)
            elif k.endswith("_close"):
                assert v < 1e-5, (k, v)
