"""Optimizer-step time of the Muon configuration: the Llama-3-8B-shaped decoder with every 2-D weight
stored whole on an owner rank (``BucketedOwned``, owners chosen greedily by Newton-Schulz cost and
carried across buckets) and updated by Muon (momentum 0.95, 5 Newton-Schulz iterations, bf16
tcgen05 GEMMs on the owner GPU, no communication); embeddings, head and norms are ``Shard(0)`` +
fused AdamW.

``python bench_muon.py [--gpus N] [--steps K] [--warmup W] [--impl owned|shard|torch]`` (torchrun for N > 1)
prints one JSON line: optimizer-step milliseconds (max over ranks, CUDA events, gradients are synthetic random
tensors in the shards' own layout, so no forward/backward runs).

Arms: ``owned`` (default) owner storage, no communication; ``shard`` the same matrices stored as ``Shard(0)`` rows
and moved to their owners and back by the pipelined redistribution runtime every step (the layout the
reference's published 527 ms figure belongs to; ``--comm nccl`` uses ``all_to_all_single``, ``symm`` peer pulls);
``torch`` the baseline: ``torch.optim.Muon`` (library GEMMs) on the same owner-stored matrices.
"""
from __future__ import annotations

import argparse
import json
import os

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")   # before CUDA initialises: peer waits must not meet lazy kernel loading

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--impl", choices=["owned", "shard", "torch"], default="owned")
    ap.add_argument("--comm", choices=["symm", "nccl"], default="symm")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from flex_shard_b200 import BucketSpec, flex_shard, ops
    from flex_shard_b200.bucket_storage import MixedPrecisionPolicy
    from flex_shard_b200.dist_muon import DistMuon, build_local_dist_muon, get_flex_shard_muon_compute_layouts
    from flex_shard_b200.dist_muon import BucketConfig
    from flex_shard_b200.models.llama import Llama, LlamaConfig
    from flex_shard_b200.optim.adamw import FusedAdamW
    from flex_shard_b200.placements import Shard, make_bucketed_owned_full_param_placement_fn
    from flex_shard_b200.placements.mixed_bucket import make_mixed_placement_fn

    if world > 1:
        from flex_shard_b200.parallel.comm import set_default_backend

        set_default_backend(args.comm)
    cfg = LlamaConfig(n_layers=args.layers)
    with torch.device("meta"):
        model = Llama(cfg, dtype=torch.bfloat16, device="meta")
    mesh = None
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh("cuda", (world,))
    owned = make_bucketed_owned_full_param_placement_fn(carry_loads=True)

    def layer_fn(named, m):
        mats = [(f, p) for f, p in named if p.dim() >= 2]
        out = dict(owned(mats, m))
        out.update({f: Shard(0) for f, p in named if p.dim() < 2})
        return out

    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    specs = [BucketSpec(["tok_embeddings"], mesh=mesh, mp_policy=mp)]
    for i in range(cfg.n_layers):
        specs.append(BucketSpec([f"layers.{i}"], mesh=mesh, mp_policy=mp,
                                placement_fn=None if args.impl == "shard" else make_mixed_placement_fn(layer_fn)))
    specs.append(BucketSpec(["head"], mesh=mesh, mp_policy=mp))
    flex_shard(model, specs)
    model.to_empty(device=dev)
    with torch.no_grad():
        for p in model.parameters():
            p.normal_(0.0, 0.02)
    is_matrix = lambda n, p: n.startswith("layers.") and len(getattr(p, "_fsb_global_shape", p.shape)) >= 2
    if args.impl == "shard":
        lays = get_flex_shard_muon_compute_layouts(model)
        named = [(n, p) for n, p in model.named_parameters() if is_matrix(n, p)]
        muon = DistMuon([p for _, p in named], param_names=[n for n, _ in named],
                        compute_layouts={n: lays[n] for n, _ in named}, lr=0.02, momentum=0.95, ns_steps=5,
                        weight_decay=0.0,
                        bucket_configs=[BucketConfig((f"layers.{i}.*",), f"layers.{i}") for i in range(cfg.n_layers)])
    elif args.impl == "torch":
        mats = [p for n, p in model.named_parameters() if is_matrix(n, p) and p.numel() > 0]
        muon = torch.optim.Muon(mats, lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.0) if mats else None
    else:
        muon = build_local_dist_muon(model, is_muon_param=is_matrix, lr=0.02, momentum=0.95, ns_steps=5,
                                     weight_decay=0.0)
    rest = [p for n, p in model.named_parameters() if not is_matrix(n, p)]
    adamw = FusedAdamW(rest, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    params = list(model.parameters())
    local_elems = sum(p.numel() for p in params)

    def set_grads():
        for p in params:
            p.grad = torch.randn_like(p) * 1e-3 if p.numel() else torch.zeros_like(p)

    def step():
        if muon is not None:
            muon.step()
        adamw.step()

    for _ in range(args.warmup):
        set_grads()
        step()
    torch.cuda.synchronize()
    ops.check_status()
    times = []
    for _ in range(args.steps):
        set_grads()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    ops.check_status()
    ms = torch.tensor([sum(times) / len(times)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"metric": "optimizer-step ms, Muon config (Llama-3-8B-shaped, BucketedOwned, 5 Newton-Schulz steps)",
                          "value": float(ms), "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "higher_is_better": False, "dtype": "bf16", "data": "synthetic gradients",
                          "impl": args.impl, "local_param_elems_rank0": local_elems,
                          "collectives_issued": getattr(muon, "collectives_issued", None),
                          "peer_pull_exchanges": getattr(muon, "p2p_exchanges", None),
                          "config": {"model": f"llama3-8b-shaped ({cfg.n_layers} layers)", "parallelism": f"dp{world}"}}),
              flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
