"""Train the DeepSeek-V3-style MoE model with flex_shard_b200 on one host.

    python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc-per-node 8 \
        examples/deepseek_v3/train.py --steps 100 --ep 8 --optimizer muon

Flags follow the reference's example (``examples/deepseek_v3/train.py:61-111``): ``--ep`` sets the
expert-parallel degree, ``--optimizer {adamw,muon}``, ``--checkpoint-dir`` saves and resumes,
``--deterministic`` fixes seeds, ``--profile-dir`` writes a Chrome trace of step 5 per rank.
``--small`` shrinks the model for smoke runs (also on CPU with the gloo backend).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from data import PackedDocumentBatches, SyntheticBatches  # noqa: E402
from muon import build_muon, store_heads_blockwise, store_on_owners  # noqa: E402

from flex_shard_b200 import (checkpoint, flex_shard, register_optimizer_checkpoint_hook,  # noqa: E402
                             set_state_dict_global_layouts)
from flex_shard_b200.dist_muon import load_muon_checkpoint_state, muon_checkpoint_state  # noqa: E402
from flex_shard_b200.dist_muon.placement import get_mesh_rank_groups, get_strided_rank_groups  # noqa: E402
from flex_shard_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config, deepseek_buckets  # noqa: E402
from flex_shard_b200.optim.adamw import FusedAdamW  # noqa: E402
from flex_shard_b200.parallel.expert_parallel import apply_expert_parallel  # noqa: E402
from flex_shard_b200.utils.training import JsonMetrics, clip_grad_norm_, lr_lambda  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--local-batch-size", type=int, default=2)
    ap.add_argument("--ep", type=int, default=0, help="expert-parallel degree (0: all ranks, 1: off)")
    ap.add_argument("--optimizer", choices=["adamw", "muon"], default="adamw")
    ap.add_argument("--data", choices=["synthetic", "files"], default="synthetic",
                    help="synthetic: resumable random tokens; files: documents packed from local token files "
                         "(--data-files), labels stop at document ends and positions restart per document")
    ap.add_argument("--data-files", default=None, help="file, directory or glob of .npy / .pt token files (--data files)")
    ap.add_argument("--bos-id", type=int, default=0)
    ap.add_argument("--eos-id", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--warmup-steps", type=int, default=2)
    ap.add_argument("--decay-ratio", type=float, default=0.1)
    ap.add_argument("--min-lr-factor", type=float, default=0.1)
    ap.add_argument("--max-norm", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--checkpoint-interval", type=int, default=0)
    ap.add_argument("--profile-dir", default=None)
    ap.add_argument("--no-activation-checkpointing", action="store_true",
                    help="keep every block's activations instead of recomputing the block in backward")
    ap.add_argument("--init-checkpoint", default=None,
                    help="checkpoint directory to take the initial weights from (model only; optimizers start fresh)")
    ap.add_argument("--document-length", type=int, default=0,
                    help="> 0: synthetic sequences are packed documents of this many tokens; attention stays inside them")
    ap.add_argument("--aux-loss-coeff", type=float, default=0.0, help="weight of the sequence-wise router balance loss")
    ap.add_argument("--no-explicit-prefetch", action="store_true",
                    help="leave prefetching to the learned order instead of block-by-block prefetch lists")
    ap.add_argument("--attention", choices=["sdpa"], default="sdpa",
                    help="attention implementation: PyTorch SDPA with a block-diagonal mask for packed documents (the "
                         "reference's other choice, FlexAttention, needs torch.compile, which this library does not use)")
    ap.add_argument("--muon-split", choices=["head", "role"], default="head",
                    help="Muon's matrices inside the attention projections: one per head, or one per head and role "
                         "(no-position / rotary / value rows apart, the Kimi-K2 recipe)")
    ap.add_argument("--muon-storage", choices=["owners", "heads"], default="owners",
                    help="owners: every matrix whole on an owner rank; heads: per-head matrices in head blocks "
                         "spread over the ranks (BlockShard by attention head), the rest on owners")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--comm", choices=["nccl", "symm"], default="nccl")
    return ap.parse_args()


def prefetch_blocks_in_order(model) -> None:
    """Explicit prefetch lists: the first bucket of a block (the one that runs first) prefetches every bucket
    of the next block in forward and of the previous block in backward; expert buckets prefetch nothing.
    With expert parallelism the learned one-bucket-ahead order would issue the next gathers only after the
    dispatcher's host-visible step. Parity: ``examples/deepseek_v3/train.py:178-200`` of the reference."""
    storages = list(model.sharded_bucket_storages)
    embedding, head = storages[0], storages[-1]
    blocks: dict[int, list] = {}
    for st in storages[1:-1]:
        layer = int(st.infos[0].fqn.split(".")[1])
        blocks.setdefault(layer, []).append(st)
    order = [blocks[i] for i in sorted(blocks)]
    for group in order:
        for st in group[1:]:
            st.set_buckets_to_forward_prefetch([])
            st.set_buckets_to_backward_prefetch([])
    embedding.set_buckets_to_forward_prefetch(order[0] if order else [head])
    head.set_buckets_to_backward_prefetch(order[-1] if order else [embedding])
    for i, group in enumerate(order):
        group[0].set_buckets_to_forward_prefetch(order[i + 1] if i + 1 < len(order) else [head])
        group[0].set_buckets_to_backward_prefetch(order[i - 1] if i > 0 else [embedding])


def main():
    args = parse()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if args.deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
    torch.manual_seed(args.seed)
    if args.comm == "symm" and cuda:
        from flex_shard_b200.parallel.comm import set_default_backend

        set_default_backend("symm")

    cfg = DeepSeekV3Config(max_seq_len=args.seq_len)
    if args.small:
        cfg = DeepSeekV3Config(vocab_size=2048, d_model=256, n_layers=3, n_heads=2, q_lora_rank=128, kv_lora_rank=64,
                               qk_nope_dim=64, qk_rope_dim=32, v_dim=64, dense_hidden=512, n_experts=8,
                               expert_hidden=128, top_k=2, max_seq_len=args.seq_len)
    cfg.activation_checkpointing = not args.no_activation_checkpointing
    cfg.aux_loss_coeff = args.aux_loss_coeff
    ep = world if args.ep == 0 else args.ep
    model = DeepSeekV3(cfg, dtype=torch.bfloat16 if cuda else torch.float32, device=dev)
    model.init_weights(args.seed)

    dp_group = dist.group.WORLD
    expert_mesh = None
    if ep > 1:
        # EP groups of `ep` consecutive ranks; experts are then sharded over ranks holding the same ones
        ep_groups = [dist.new_group(ranks) for ranks in get_mesh_rank_groups(world, ep)]
        efsdp_groups = [dist.new_group(ranks) for ranks in get_strided_rank_groups(world, ep)]
        apply_expert_parallel(model, ep_groups[rank // ep])
        expert_mesh = efsdp_groups[rank % ep]
    flex_shard(model, deepseek_buckets(model, mesh=dp_group, expert_mesh=expert_mesh))
    if not args.no_explicit_prefetch:
        prefetch_blocks_in_order(model)
    if args.init_checkpoint:
        sd = model.state_dict()
        set_state_dict_global_layouts(model, sd)
        checkpoint.load({"model": sd}, args.init_checkpoint)
        model.load_state_dict(sd)

    if args.optimizer == "muon":
        (store_heads_blockwise if args.muon_storage == "heads" else store_on_owners)(model)
        muon, adam = build_muon(model, args.lr, args.weight_decay, split=args.muon_split)
        opts = [muon, adam]
    else:
        adam = FusedAdamW(model.parameters(), lr=args.lr, betas=(0.9, 0.95), weight_decay=args.weight_decay)
        opts = [adam]
    register_optimizer_checkpoint_hook(adam, model)
    scheds = [torch.optim.lr_scheduler.LambdaLR(o, lambda s: lr_lambda(s, args.warmup_steps, args.steps,
                                                                       args.decay_ratio, args.min_lr_factor))
              for o in opts]
    if args.data == "files":
        if not args.data_files:
            raise SystemExit("--data files needs --data-files")
        data = PackedDocumentBatches(args.data_files, args.local_batch_size, args.seq_len, rank=rank, world_size=world,
                                     bos_id=args.bos_id, eos_id=args.eos_id)
    else:
        data = SyntheticBatches(cfg.vocab_size, args.local_batch_size, args.seq_len, args.seed, rank, pin_memory=cuda)
    steps_done = [0]
    positions = None
    if args.document_length > 0:
        positions = (torch.arange(args.seq_len, device=dev) % args.document_length).expand(args.local_batch_size, -1)

    def state():
        sd = model.state_dict()
        set_state_dict_global_layouts(model, sd)
        # the data position differs between ranks (each reads its own files): saved per rank
        out = {"model": sd, "adam": adam.state_dict(), "data": checkpoint.PerRank(data.state_dict()),
               "sched": [s.state_dict() for s in scheds], "step": steps_done[0]}
        if args.optimizer == "muon":    # momentum buffers, tagged with their parameters' layouts
            out["muon"] = muon_checkpoint_state(muon, model)
        return out

    start = 0
    if args.checkpoint_dir and os.path.isdir(args.checkpoint_dir) and os.listdir(args.checkpoint_dir):
        last = sorted(os.listdir(args.checkpoint_dir))[-1]
        # optimizer state must exist before it can be filled: one step with zero gradients and zero lr
        for p in model.parameters():
            p.grad = torch.zeros_like(p, dtype=getattr(p, "grad_dtype", None) or p.dtype)
        saved_lr = [g["lr"] for g in adam.param_groups]
        for g in adam.param_groups:
            g["lr"] = 0.0
        adam.step()
        adam.zero_grad(set_to_none=True)
        for g, lr in zip(adam.param_groups, saved_lr):
            g["lr"] = lr
        sd = state()
        checkpoint.load(sd, os.path.join(args.checkpoint_dir, last))
        model.load_state_dict(sd["model"])
        adam.load_state_dict(sd["adam"])
        if args.optimizer == "muon":
            load_muon_checkpoint_state(muon, sd["muon"])
        data.load_state_dict(sd["data"].value)
        for s_, ssd in zip(scheds, sd["sched"]):
            s_.load_state_dict(ssd)
        start = int(sd.get("step", getattr(data, "step", 0)))

    metrics = JsonMetrics(rank=rank, module=model)
    for step in range(start, args.steps):
        prof = None
        if args.profile_dir and step == 5:
            prof = torch.profiler.profile()
            prof.__enter__()
        metrics.start_step()
        batch = next(data)
        if isinstance(batch, dict):      # packed documents: inputs, next-token labels and per-document positions
            inputs, labels = batch["input"].to(dev, non_blocking=True), batch["labels"].to(dev, non_blocking=True)
            step_positions = batch["positions"].to(dev, non_blocking=True)
        else:
            tok = batch.to(dev, non_blocking=True)
            inputs, labels, step_positions = tok[:, :-1], tok[:, 1:], positions
        ntok = torch.tensor([labels.numel()], dtype=torch.float32, device=dev)
        dist.all_reduce(ntok)
        # sum of token losses divided by the global token count (buckets sum gradients)
        if args.aux_loss_coeff > 0:
            for moe in model.moe_layers():
                moe.aux_loss_denominator = float(ntok)
        loss = model.loss(inputs, labels, loss_is_root=False, positions=step_positions) * (
            labels.numel() / ntok.squeeze())
        loss.backward()
        gnorm = clip_grad_norm_(model, args.max_norm)
        for m in model.moe_layers():
            m.update_expert_bias()
        for o in opts:
            o.step()
        for s in scheds:
            s.step()
        for o in opts:
            o.zero_grad(set_to_none=True)
        red = loss.detach().clone()
        dist.all_reduce(red)
        metrics.end_step(step, labels.numel(), loss=red, grad_norm=gnorm, lr=scheds[0].get_last_lr()[0])
        steps_done[0] = step + 1
        if prof is not None:
            prof.__exit__(None, None, None)
            os.makedirs(args.profile_dir, exist_ok=True)
            prof.export_chrome_trace(os.path.join(args.profile_dir, f"rank{rank}.json"))
        if args.checkpoint_dir and args.checkpoint_interval and (step + 1) % args.checkpoint_interval == 0:
            checkpoint.save(state(), os.path.join(args.checkpoint_dir, f"step{step + 1:08d}"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
