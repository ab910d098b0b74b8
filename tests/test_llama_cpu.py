"""The Llama-shaped model through the ops' CPU reference paths: sharded (gloo, 2 ranks, gradient
buckets written in reduce-scatter layout) against the unsharded model."""
import torch

from tests.common import run_ranks

CFG = dict(vocab_size=512, d_model=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_hidden=384, max_seq_len=128)


def _tokens(step, rank):
    g = torch.Generator().manual_seed(77 * step + rank)
    return torch.randint(0, CFG["vocab_size"], (2, 129), generator=g)


def _sharded(rank, world, steps, grad_bucket):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.models.llama import Llama, LlamaConfig
    from flex_shard_b200.optim.adamw import FusedAdamW
    from flex_shard_b200.placements.shard import shard_placement_fn

    model = Llama(LlamaConfig(**CFG), dtype=torch.float32)
    model.init_weights(0)
    fn = shard_placement_fn(0, grad_bucket=grad_bucket)
    specs = [BucketSpec(["tok_embeddings"], placement_fn=fn)]
    specs += [BucketSpec([f"layers.{i}"], placement_fn=fn) for i in range(CFG["n_layers"])]
    specs += [BucketSpec(["head"], placement_fn=fn, reshard_after_forward=False)]
    flex_shard(model, specs)
    opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
    losses = []
    for s in range(steps):
        tok = _tokens(s, rank)
        loss = model.loss(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()))
    return losses


def _unsharded(steps, world):
    from flex_shard_b200.models.llama import Llama, LlamaConfig

    model = Llama(LlamaConfig(**CFG), dtype=torch.float32)
    model.init_weights(0)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
    losses = []
    for s in range(steps):
        tot = 0.0
        for r in range(world):
            tok = _tokens(s, r)
            loss = model.loss(tok[:, :-1], tok[:, 1:], loss_is_root=False) / world
            loss.backward()
            tot += float(loss.detach())
        opt.step()
        opt.zero_grad()
        losses.append(tot)
    return losses


def test_llama_sharded_matches_unsharded_with_grad_bucket():
    steps, world = 4, 2
    ref = _unsharded(steps, world)
    for grad_bucket in (True, False):
        res = run_ranks(_sharded, world, steps, grad_bucket)
        mean = [sum(r[i] for r in res) / world for i in range(steps)]
        for a, b in zip(mean, ref):
            assert abs(a - b) < 5e-4 * max(1.0, abs(b)), (grad_bucket, mean, ref)


def test_llama_trains_with_quantised_gather_buckets():
    """The same model with its blocks' 2-D weights gathered as FP8 128x128 blocks or as MXFP8 (the
    weights arrive as quantised wrappers and ``linear`` runs the block-scaled products) follows the
    bf16 run closely."""
    import torch

    from flex_shard_b200 import flex_shard
    from flex_shard_b200.models.llama import Llama, LlamaConfig, llama_buckets, llama_quantized_buckets

    cfg = LlamaConfig(vocab_size=512, d_model=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_hidden=512, max_seq_len=64)
    runs = {}
    for kind in ("bf16", "fp8", "mxfp8"):
        torch.manual_seed(0)
        m = Llama(cfg, dtype=torch.bfloat16, device="cpu")
        m.init_weights(0)
        flex_shard(m, llama_buckets(m) if kind == "bf16" else llama_quantized_buckets(m, kind=kind))
        opt = torch.optim.SGD(m.parameters(), lr=0.1)
        losses = []
        for s in range(3):
            tok = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(s))
            loss = m.loss(tok[:, :-1], tok[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad()
            losses.append(float(loss.detach()))
        runs[kind] = losses
    for kind in ("fp8", "mxfp8"):
        for a, b in zip(runs[kind], runs["bf16"]):
            assert abs(a - b) < 2e-2, runs
    assert runs["bf16"][-1] < runs["bf16"][0]
