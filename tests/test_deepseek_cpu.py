"""DeepSeek-V3-style MoE model on CPU: sharded vs unsharded on one rank group, and expert
parallelism (2 gloo ranks, experts split, all-to-all dispatch) against the non-EP model."""
import torch

from tests.common import run_ranks

CFG = dict(vocab_size=512, d_model=128, n_layers=2, n_dense_layers=1, n_heads=2, q_lora_rank=64, kv_lora_rank=32,
           qk_nope_dim=32, qk_rope_dim=16, v_dim=32, dense_hidden=256, n_experts=4, expert_hidden=64, top_k=2,
           n_shared_experts=1, max_seq_len=64)


def _tok(step, rank):
    return torch.randint(0, CFG["vocab_size"], (2, 33), generator=torch.Generator().manual_seed(17 * step + rank))


def _make():
    from flex_shard_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config

    torch.manual_seed(0)
    m = DeepSeekV3(DeepSeekV3Config(**CFG), dtype=torch.float32)
    m.init_weights(0)
    return m


def _ep_worker(rank, world, steps):
    import torch.distributed as dist

    from flex_shard_b200 import flex_shard
    from flex_shard_b200.models.deepseek_v3 import deepseek_buckets
    from flex_shard_b200.parallel.expert_parallel import apply_expert_parallel
    from flex_shard_b200.bucket_storage import MixedPrecisionPolicy

    model = _make()
    apply_expert_parallel(model, dist.group.WORLD)
    # experts are already split over the EP group: shard them over a 1-rank mesh (this rank alone)
    solo = dist.new_group([rank]) if False else None
    groups = [dist.new_group([r]) for r in range(world)]
    specs = deepseek_buckets(model, mesh=None, expert_mesh=groups[rank], mp_policy=MixedPrecisionPolicy())
    flex_shard(model, specs)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for s in range(steps):
        t = _tok(s, rank)
        loss = model.loss(t[:, :-1], t[:, 1:], loss_is_root=False) / world
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss.detach()) * world)
    return losses


def _reference(world, steps):
    model = _make()
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    out = []
    for s in range(steps):
        tot = 0.0
        for r in range(world):
            t = _tok(s, r)
            loss = model.loss(t[:, :-1], t[:, 1:], loss_is_root=False) / world
            loss.backward()
            tot += float(loss.detach())
        opt.step()
        opt.zero_grad()
        out.append(tot)
    return out


def test_expert_parallel_matches_single_process():
    steps, world = 3, 2
    ref = _reference(world, steps)
    res = run_ranks(_ep_worker, world, steps)
    mean = [sum(r[i] for r in res) / world for i in range(steps)]
    for a, b in zip(mean, ref):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (mean, ref)


def _tiny_cfg(**kw):
    from flex_shard_b200.models.deepseek_v3 import DeepSeekV3Config

    return DeepSeekV3Config(vocab_size=128, d_model=64, n_layers=2, n_dense_layers=1, n_heads=2, q_lora_rank=32,
                            kv_lora_rank=16, qk_nope_dim=16, qk_rope_dim=8, v_dim=16, dense_hidden=64, n_experts=4,
                            expert_hidden=32, top_k=2, n_shared_experts=1, max_seq_len=32, **kw)


def _grads(cfg, tokens, positions=None):
    import torch

    from flex_shard_b200.models.deepseek_v3 import DeepSeekV3

    torch.manual_seed(0)
    m = DeepSeekV3(cfg, dtype=torch.float32)
    m.init_weights(0)
    loss = m.loss(tokens[:, :-1], tokens[:, 1:], loss_is_root=False, positions=positions)
    loss.backward()
    return loss.detach(), {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}, m


def test_activation_checkpointing_document_mask_and_balance_loss():
    import torch

    tokens = torch.randint(0, 128, (2, 17), generator=torch.Generator().manual_seed(3))
    base_loss, base, _ = _grads(_tiny_cfg(), tokens)
    # per-block recompute: same loss, same gradients
    ac_loss, ac, _ = _grads(_tiny_cfg(activation_checkpointing=True), tokens)
    assert torch.equal(ac_loss, base_loss)
    assert all(torch.allclose(ac[n], base[n], atol=1e-6) for n in base)
    # balance loss: the reported loss is unchanged, the router gate's gradient is not
    aux_loss, aux, _ = _grads(_tiny_cfg(aux_loss_coeff=0.5), tokens)
    assert torch.equal(aux_loss, base_loss)
    gate = next(n for n in base if n.endswith(".gate"))
    assert not torch.allclose(aux[gate], base[gate])
    assert all(torch.allclose(aux[n], base[n], atol=1e-6) for n in base if "routed_experts" in n)
    # document mask: logits of the first document do not see the second one
    positions = (torch.arange(16) % 8).expand(2, -1)
    _, _, m = _grads(_tiny_cfg(), tokens, positions)
    other = tokens.clone()
    other[:, 8:16] = (other[:, 8:16] + 1) % 128
    with torch.no_grad():
        a = m(tokens[:, :-1], positions).view(2, 16, -1)
        b = m(other[:, :-1], positions).view(2, 16, -1)
        c = m(other[:, :-1]).view(2, 16, -1)
    assert torch.allclose(a[:, :8], b[:, :8], atol=1e-6) and not torch.allclose(a[:, 8:], b[:, 8:])
    assert torch.allclose(b[:, :8], c[:, :8], atol=1e-6)         # causal anyway: the first document never saw the second
    assert not torch.allclose(b[:, 8:], c[:, 8:], atol=1e-6)     # without the mask the second document sees the first
