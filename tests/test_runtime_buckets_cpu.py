"""Per-bucket behaviour of the runtime on 2 gloo ranks: module-name patterns, the per-bucket unshard / reshard calls,
one gathered bucket at a time with ``reshard_after_forward``, persistent unsharded parameters whose storage is freed
and refilled, a head applied chunk by chunk, and the per-bucket switches.
Parity: the behaviours pinned by the reference's ``tests/test_flex_shard_runtime.py:348-407,409-569,709-870,921-970``."""
import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


class Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.lin = nn.Linear(d, d)
        self.norm = nn.LayerNorm(d)

    def forward(self, x):
        return self.norm(torch.relu(self.lin(x)))


class Stack(nn.Module):
    def __init__(self, d=8, n=3, vocab=16):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList([Block(d) for _ in range(n)])
        self.head = nn.Linear(d, vocab, bias=False)

    def hidden(self, t):
        h = self.emb(t)
        for l in self.layers:
            h = l(h)
        return h

    def forward(self, t):
        return self.head(self.hidden(t))


def _work(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    out = {}
    torch.manual_seed(0)
    m, ref = Stack(), Stack()
    ref.load_state_dict(m.state_dict())
    # module names as patterns: "layers.0" takes every parameter below that module; two sibling modules form one
    # bucket that is hooked on both of them (gathered in the first one's forward, resharded after the last one's)
    flex_shard(m, [BucketSpec(["emb"]), BucketSpec(["layers.0"]), BucketSpec(["layers.1", "layers.2"]),
                   BucketSpec(["head"], reshard_after_forward=False)])
    sts = m.sharded_bucket_storages
    out["members"] = [[i.fqn for i in st.infos] for st in sts]
    # one gathered bucket at a time in forward (the kept head aside)
    gathered_at = []
    for i, l in enumerate(m.layers):
        l.register_forward_hook(lambda mod, a, o: gathered_at.append([st.runtime.is_unsharded for st in sts]))
    tok = torch.randint(0, 16, (4, 5), generator=torch.Generator().manual_seed(rank))
    with torch.no_grad():
        m(tok)
    out["one_at_a_time"] = all(sum(flags[:3]) <= 1 for flags in gathered_at) and len(gathered_at) == 3
    m.reshard()
    # per-bucket unshard / reshard, identity and storage of the persistent unsharded parameters
    st = sts[1]
    st.unshard()
    ups = list(st.runtime.unsharded_params)
    out["unsharded_shapes"] = [tuple(u.shape) for u in ups] == [tuple(i.global_shape) for i in st.infos]
    out["others_stay_sharded"] = not sts[2].runtime.is_unsharded
    full_ref = [p.detach().clone() for p in ref.layers[0].parameters()]
    out["values"] = all(torch.equal(u.detach(), f) for u, f in zip(ups, full_ref))
    st.reshard()
    out["freed"] = [u.untyped_storage().size() for u in ups] == [0] * len(ups)
    st.unshard()
    out["same_objects_refilled"] = ([id(u) for u in st.runtime.unsharded_params] == [id(u) for u in ups]
                                    and all(torch.equal(u.detach(), f) for u, f in zip(ups, full_ref)))
    st.reshard()
    # a head applied chunk by chunk (loss over sequence chunks): same gradients as one call, one reduction of the head
    ctx = sts[0].runtime.context
    before = ctx.stats["reduces"]
    h = m.hidden(tok)
    loss = sum(m.head(c).square().mean() for c in h.chunk(5, dim=1)) / 5
    loss.backward()
    out["reduces"] = ctx.stats["reduces"] - before
    toks = [torch.randint(0, 16, (4, 5), generator=torch.Generator().manual_seed(r)) for r in range(world)]
    sum(sum(ref.head(c).square().mean() for c in ref.hidden(t).chunk(5, dim=1)) / 5 for t in toks).div(world).backward()
    n = -(-ref.head.weight.shape[0] // world)
    want = ref.head.weight.grad[rank * n:(rank + 1) * n]
    out["chunked_head_grad"] = bool(torch.allclose(m.head.weight.grad, want, atol=1e-6))
    out["idle"] = ctx.idle()
    m.reshard()
    # per-bucket switches: one bucket keeps its gradients (no sync) while the others reduce
    for p in m.parameters():
        p.grad = None
    sts[2].set_requires_gradient_sync(False)
    before = ctx.stats["reduces"]
    m(tok).square().mean().backward()
    out["partial_sync_reduces"] = ctx.stats["reduces"] - before
    out["kept_bucket_has_no_sharded_grad"] = all(sp.grad is None for sp in sts[2].sharded_params)
    sts[2].set_requires_gradient_sync(True)
    m(tok).square().mean().backward()
    out["kept_bucket_reduced_later"] = all(sp.grad is not None for sp in sts[2].sharded_params)
    return out


def test_per_bucket_runtime_contracts():
    for r in run_ranks(_work, 2):
        assert r["members"] == [["emb.weight"],
                                ["layers.0.lin.weight", "layers.0.lin.bias", "layers.0.norm.weight", "layers.0.norm.bias"],
                                [f"layers.{i}.{n}" for i in (1, 2) for n in ("lin.weight", "lin.bias", "norm.weight", "norm.bias")],
                                ["head.weight"]]
        assert r["one_at_a_time"] and r["unsharded_shapes"] and r["others_stay_sharded"] and r["values"]
        assert r["freed"] and r["same_objects_refilled"]
        assert r["reduces"] == 4 and r["chunked_head_grad"] and r["idle"]
        assert r["partial_sync_reduces"] == 3 and r["kept_bucket_has_no_sharded_grad"] and r["kept_bucket_reduced_later"]


def _inference_first(rank, world, kind):
    import torch.nn as nn

    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import (make_bucketed_block_shard_placement_fn,
                                            make_bucketed_owned_full_param_placement_fn)

    fn = {"shard": None, "owned": make_bucketed_owned_full_param_placement_fn(),
          "flat": make_bucketed_block_shard_placement_fn()}[kind]
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))
    ref = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))
    ref.load_state_dict(m.state_dict())
    flex_shard(m, [BucketSpec(["0.*"], placement_fn=fn), BucketSpec(["2.*"], placement_fn=fn)])
    x = torch.randn(3, 8)
    with torch.inference_mode():
        first = m(x)                    # the first unshard of every bucket happens here
    ok = bool(torch.allclose(first, ref(x), atol=1e-6))
    for _ in range(2):                  # training afterwards saves and refills the same gathered parameters
        m(x).sum().backward()
    with torch.inference_mode():
        again = m(x)
    return ok, all(p.grad is not None for p in m.parameters()), bool(torch.allclose(again, first, atol=1e-6))


@pytest.mark.parametrize("kind", ["shard", "owned", "flat"])
def test_first_unshard_may_happen_under_inference_mode(kind):
    """An evaluation pass under ``torch.inference_mode()`` before training leaves ordinary gathered parameters behind
    (parity: ``tests/test_flex_shard_runtime.py:409-541`` of the reference)."""
    for world in (1, 2):
        for ok, grads, same in run_ranks(_inference_first, world, kind):
            assert ok and grads and same


class _WithUnused(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b, self.unused = nn.Linear(8, 8), nn.Linear(8, 4), nn.Linear(8, 8)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


def _user_hooks_and_freezing(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = _WithUnused()
    seen = []
    m.a.register_forward_pre_hook(lambda mod, args: seen.append(tuple(mod.weight.shape)))   # before flex_shard
    flex_shard(m, [BucketSpec(["a.*", "unused.*"]), BucketSpec(["b.*"])])
    x = torch.randn(3, 8)
    m(x).sum().backward()
    out = {"hook_saw": seen[:], "unused": [float(p.grad.abs().sum()) for p in m.unused.parameters()]}
    for p in m.parameters():
        p.grad = None
    m.a.weight.requires_grad_(False)            # freezing a local shard takes effect at the next unshard
    m(x).sum().backward()
    out["frozen_has_no_grad"] = m.a.weight.grad is None and m.a.bias.grad is not None
    out["repr"] = all("ShardedBucketStorage" in repr(st) for st in m.sharded_bucket_storages)   # while resharded
    return out


def test_user_hooks_unused_parameters_and_freezing_after_wrap():
    """A pre-forward hook registered before ``flex_shard`` sees the gathered parameter, trainable parameters that the
    forward does not use get zero gradients, a shard frozen after wrapping stops getting one, and ``repr`` of a
    resharded bucket reads no freed storage (parity: ``tests/test_flex_shard_runtime.py:409-541, 921-971`` of the
    reference)."""
    for out in run_ranks(_user_hooks_and_freezing, 2):
        assert out["hook_saw"] == [(8, 8)] and out["unused"] == [0.0, 0.0]
        assert out["frozen_has_no_grad"] and out["repr"]
