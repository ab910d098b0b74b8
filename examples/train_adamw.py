"""Smallest end-to-end example: the tiny MoE transformer, Shard(0) buckets per layer, AdamW.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/train_adamw.py

Runs on CPU (gloo) or GPUs (nccl). Role parity: ``examples/train_adamw.py`` of the reference.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flex_shard_b200 import BucketSpec, flex_shard  # noqa: E402
from flex_shard_b200.models.tiny_moe import TinyMoEConfig, TinyMoETransformer, next_token_loss  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    dev = torch.device("cuda") if cuda else torch.device("cpu")
    model = TinyMoETransformer(TinyMoEConfig()).to(dev)
    model.init_weights(0)
    specs = [BucketSpec(["tok_embeddings"])] + [BucketSpec([f"layers.{i}.*"]) for i in range(len(model.layers))]
    specs.append(BucketSpec(["norm", "output"], reshard_after_forward=False))
    flex_shard(model, specs)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4)
    for step in range(10):
        tok = torch.randint(0, 1024, (4, 128), generator=torch.Generator().manual_seed(1000 * step + rank)).to(dev)
        loss = next_token_loss(model(tok), tok)
        loss.backward()
        opt.step()
        opt.zero_grad()
        if rank == 0:
            print(f"step {step} loss {loss.item():.4f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
