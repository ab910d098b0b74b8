"""Times ONE collective of the library on every rank of a real multi-GPU job: the workloads behind the
NVLink figures in the profile summaries.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node W --master-addr 127.0.0.1 --master-port P \
        -m flex_shard_b200.utils.comm_cases <case> [--iters N]

Cases (sizes are one Llama-3-8B layer bucket, 218.1 M parameters):

``gather``        bf16 parameter all-gather of the bucket into ``[W, shard]``: this library's copy-engine
                  gather and its SM pull kernel, both reading the peers' resident shards in place, against
                  ``dist.all_gather_into_tensor`` (NCCL).
``reduce_adamw``  fp32 gradient reduce-scatter of the bucket fused with the sharded AdamW update: rank-order
                  peer loads and the in-switch (multimem) sum, against NCCL ``reduce_scatter_tensor`` followed
                  by the fused AdamW kernel.

Every figure is the median over ``iters`` launches of the CUDA-event time on each rank, then the maximum
over ranks; rank 0 prints one JSON line.  ``*_gbs`` is the NVLink payload entering each GPU divided by
that time.  Nothing here runs under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # before CUDA initialises: peer waits must not meet lazy kernel loading

import torch
import torch.distributed as dist

LAYER_PARAMS = 218_112_000   # wqkv + wo + w13 + w2 + two norms of one block, rounded to a multiple of 64 * 16


def _median_max(fn, iters, world):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gather", "reduce_adamw"])
    ap.add_argument("--iters", type=int, default=7)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from flex_shard_b200 import ops
    from flex_shard_b200.parallel.symm import PeerBucket, SymmComm

    g = dist.group.WORLD
    out = {"case": args.case, "world": world, "iters": args.iters, "params": LAYER_PARAMS}
    shard = LAYER_PARAMS // world
    try:
        if args.case == "gather":
            comm = SymmComm(g, rank, world, dev)
            nbytes = shard * 2
            src = comm.alloc_storage(nbytes)           # resident shard: the peers read it in place
            src.view(torch.bfloat16).normal_()
            dst = torch.empty(world * nbytes, dtype=torch.uint8, device=dev)
            segs = [(r, 0, dst.data_ptr() + r * nbytes, nbytes) for r in range(world)]
            inbound = (world - 1) * nbytes
            for engine in ("dma", "sm"):
                comm.gather_engine = engine
                ms = _median_max(lambda: comm.all_gather_segments(src, segs), args.iters, world)
                out[f"{engine}_ms"], out[f"{engine}_inbound_gbs"] = ms, inbound / ms / 1e6
            ref = torch.empty_like(dst)
            ms = _median_max(lambda: dist.all_gather_into_tensor(ref, src), args.iters, world)
            out["nccl_ms"], out["nccl_inbound_gbs"] = ms, inbound / ms / 1e6
            comm.all_gather_segments(src, segs)
            torch.cuda.synchronize()
            out["bitwise_equal_to_nccl"] = bool(torch.equal(dst, ref))
            comm.fence_resident()
        else:
            comm = SymmComm(g, rank, world, dev)
            row = shard - shard % 4
            ring = comm.grad_ring(world * row * 4)
            # every rank's contribution to every owner, as the weight-gradient epilogues leave it (pull layout)
            for k in range(ring.entries):
                ring.region.payload[k * ring.entry_bytes:k * ring.entry_bytes + world * row * 4].view(torch.float32).normal_()
            p = torch.randn(row, device=dev).bfloat16()
            m = torch.zeros(row, device=dev)
            v = torch.zeros(row, device=dev)
            adam = dict(p=p, m=m, v=v, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1)
            out["multicast_mapped"] = bool(ring.region.mc_base)

            def fused():
                k, u = ring.acquire()
                comm.reduce_incoming(PeerBucket(ring, k, u, row), 1.0 / world, None, adam)

            inbound_peer = (world - 1) * row * 4
            for name, mc in (("peer_loads", False), ("multimem", True)):
                if mc and not ring.region.mc_base:
                    continue
                comm.multimem_reduce = mc
                ms = _median_max(fused, args.iters, world)
                out[f"{name}_ms"] = ms
                out[f"{name}_inbound_gbs"] = (row * 4 if mc else inbound_peer) / ms / 1e6
                out[f"{name}_reduced_gbs"] = world * row * 4 / ms / 1e6
            send = torch.randn(world * row, device=dev)
            red = torch.empty(row, device=dev)
            from flex_shard_b200.ops.elementwise import adamw_step_

            def nccl():
                dist.reduce_scatter_tensor(red, send, op=dist.ReduceOp.AVG)
                adamw_step_(p, red, m, v, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=1)

            ms = _median_max(nccl, args.iters, world)
            out["nccl_then_adamw_ms"], out["nccl_reduced_gbs"] = ms, world * row * 4 / ms / 1e6
        torch.cuda.synchronize()
        ops.check_status()
        dist.barrier()
        if rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
