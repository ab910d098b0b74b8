"""Allocator and stream lifetime under injected delays, on 2 GPUs with the NCCL path (skipped with fewer):
collectives are slowed down with ``torch.cuda._sleep`` on their streams and the results must not change,
the packed reduce-scatter input of one bucket must reuse the block the previous bucket freed
(``max_pending_reduce_grads = 1`` bounds memory like FSDP2 does), and no gather buffer may stay allocated
after a step.  Behaviours restated from ``src/flex_shard/tests/test_flex_shard_training.py:379-597,1511-1533``."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    import torch.distributed as dist
    import torch.nn as nn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import BucketSpec, flex_shard
        from flex_shard_b200.parallel import comm as comm_mod
        from flex_shard_b200.parallel.comm import set_default_backend

        set_default_backend("nccl")
        dev = torch.device("cuda", rank)

        def build():
            torch.manual_seed(0)
            m = nn.Sequential(*[nn.Linear(512, 512) for _ in range(4)]).to(dev)
            flex_shard(m, [BucketSpec([str(i)]) for i in range(4)])
            return m

        def run(m, steps=3):
            outs = []
            for s in range(steps):
                x = torch.randn(8, 512, generator=torch.Generator().manual_seed(10 * s + rank)).to(dev)
                m(x).square().mean().backward()
                outs.append([p.grad.detach().clone() for p in m.parameters()])
                for p in m.parameters():
                    p.grad = None
            torch.cuda.synchronize()
            return outs

        base = run(build())
        # slow every collective down on its own stream (about a millisecond each) and record the reduce inputs
        rs, ag = comm_mod.Comm.reduce_scatter_tensor, comm_mod.Comm.all_gather_into_tensor
        send_ptrs = []

        def slow_rs(self, out_t, inp, plan, async_op=False):
            send_ptrs.append(inp.data_ptr())
            torch.cuda._sleep(2_000_000)
            return rs(self, out_t, inp, plan, async_op)

        def slow_ag(self, out_t, inp, async_op=False):
            torch.cuda._sleep(2_000_000)
            return ag(self, out_t, inp, async_op)

        comm_mod.Comm.reduce_scatter_tensor, comm_mod.Comm.all_gather_into_tensor = slow_rs, slow_ag
        try:
            m = build()
            delayed = run(m)
        finally:
            comm_mod.Comm.reduce_scatter_tensor, comm_mod.Comm.all_gather_into_tensor = rs, ag
        res = {"equal": all(torch.equal(a, b) for sa, sb in zip(base, delayed) for a, b in zip(sa, sb))}
        # equal-sized buckets, one reduction pending at a time: every send buffer of a step after the first
        # reuses the block its predecessor gave back
        per_step = [send_ptrs[i:i + 4] for i in range(0, len(send_ptrs), 4)]
        res["reuse"] = [len(set(ptrs)) for ptrs in per_step]
        # nothing of the gathers is left: resharded parameters hold no storage, the runtime is idle
        ctx = m._fsb_ctx()
        res["idle"] = ctx.idle()
        res["unsharded_bytes"] = sum(p.untyped_storage().size() for st in m.sharded_bucket_storages
                                     for p in st.runtime.unsharded_params)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        run(m, 2)
        res["growth"] = torch.cuda.memory_allocated() - before
        torch.save(res, os.path.join(out, f"d{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_delayed_collectives_change_nothing_and_buffers_are_reused(tmp_path):
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"d{r}.pt")
        assert res["equal"], "gradients changed when the collectives were delayed"
        assert all(n <= 2 for n in res["reuse"]), res["reuse"]      # at most two blocks alternate
        assert res["idle"] and res["unsharded_bytes"] == 0 and res["growth"] == 0, res
