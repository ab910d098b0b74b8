"""Smallest end-to-end example: the tiny MoE transformer, AdamW, dense buckets on the data-parallel mesh and
expert buckets on a smaller "efsdp" sub-mesh.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 4 examples/train_adamw.py [--check]

Runs on CPU (gloo) or GPUs (nccl). ``--check`` asserts, from the runtime's own counters, what the reference's
``--trace`` asserts on a compiled graph: every bucket is gathered once for forward and once for backward and
reduced once per step, and the runtime is idle between steps.  Role parity: ``examples/train_adamw.py`` of the
reference (dp mesh + efsdp mesh ``:23-50``, collective check ``:52-81``).
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flex_shard_b200 import BucketSpec, flex_shard  # noqa: E402
from flex_shard_b200.models.tiny_moe import TinyMoEConfig, TinyMoETransformer, next_token_loss  # noqa: E402


def build_buckets(model, dp_mesh, efsdp_mesh):
    specs = [BucketSpec(["tok_embeddings"], mesh=dp_mesh)]
    for i in range(len(model.layers)):
        dense = [f"layers.{i}.{part}.*" for part in ("attention_norm", "attention", "ffn_norm", "moe.router")]
        specs.append(BucketSpec(dense, mesh=dp_mesh))
        # experts are sharded over the (smaller) efsdp mesh; ranks at the same position of different efsdp
        # groups hold replicas of the same shard
        specs.append(BucketSpec([f"layers.{i}.moe.experts.*"], mesh=efsdp_mesh))
    specs.append(BucketSpec(["norm", "output"], mesh=dp_mesh, reshard_after_forward=False))
    return specs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--check", action="store_true", help="assert one gather per pass and one reduction per bucket per step")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    dev = torch.device("cuda") if cuda else torch.device("cpu")
    # efsdp: pairs of neighbouring ranks when the world is even (every rank must create every group)
    efsdp = None
    if world % 2 == 0 and world > 2:
        groups = [dist.new_group([r, r + 1]) for r in range(0, world, 2)]
        efsdp = groups[rank // 2]
    model = TinyMoETransformer(TinyMoEConfig()).to(dev)
    model.init_weights(0)
    flex_shard(model, build_buckets(model, dist.group.WORLD, efsdp if efsdp is not None else dist.group.WORLD))
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    ctx = model._fsb_ctx()
    n_buckets = len(model.sharded_bucket_storages)
    for step in range(args.steps):
        # with an efsdp sub-mesh the replicas of an expert shard (ranks r and r + 2, ...) must see the same
        # gradient: this example gives them the same tokens, so the two efsdp groups stay identical without
        # an extra all-reduce over the replica group
        seed = 1000 * step + (rank % 2 if efsdp is not None else rank)
        tok = torch.randint(0, 1024, (4, 128), generator=torch.Generator().manual_seed(seed)).to(dev)
        before = dict(ctx.stats)
        loss = next_token_loss(model(tok), tok)
        loss.backward()
        opt.step()
        opt.zero_grad()
        if args.check:
            d = {k: ctx.stats[k] - before[k] for k in before}
            kept = sum(1 for st in model.sharded_bucket_storages if not st.reshard_after_forward)
            assert d["unshards"] == 2 * n_buckets - kept, d      # a bucket kept after forward is gathered once
            assert d["reduces"] == n_buckets, d
            assert ctx.idle()
        if rank == 0:
            print(f"step {step} loss {loss.item():.4f}")
    if args.check and rank == 0:
        print(f"check ok: {n_buckets} buckets, one gather per pass and one reduction per bucket per step")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
