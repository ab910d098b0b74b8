"""Training-time contracts on 2 gloo ranks: deferred post-backward for late weight gradients, parameters that
only some ranks use, per-parameter compute dtypes, tied weights, an asynchronous unshard that the forward
finishes, shared version counters, prefetch-target validation.
Parity: the behaviours pinned by the reference's ``tests/test_flex_shard_training.py:1155-1205,1275-1325,
1722-1833,2439-2480`` and ``tests/test_flex_shard_runtime.py:233-254,697-707``."""
import copy

import torch
import torch.nn as nn

from tests.common import run_ranks


def _expected_shard(full, rank, world):
    n = -(-full.shape[0] // world)
    return full[rank * n:(rank + 1) * n]


class _LateWgrad(torch.autograd.Function):
    """y = x W^T whose weight gradient is not produced by this node: the owner computes it later in the same
    backward (as a delayed-wgrad layer does) and then tells the sharding runtime."""

    @staticmethod
    def forward(ctx, x, w, owner):
        ctx.save_for_backward(x, w)
        ctx.owner = owner
        return x @ w.t()

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        ctx.owner.pending = (x.detach(), dy.detach(), w)
        return dy @ w, None, None


class LateLinear(nn.Module):
    def __init__(self, owner):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(8, 8) * 0.3)
        self._owner = [owner]                     # in a list: not registered as a submodule

    def forward(self, x):
        return _LateWgrad.apply(x, self.weight, self._owner[0])


class DelayedWgradModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.inp = nn.Linear(8, 8)
        self.layer = LateLinear(self)
        self.out = nn.Linear(8, 4)
        self.pending = None
        self.on_wgrad = lambda: None

    def __deepcopy__(self, memo):
        new = DelayedWgradModel()
        new.load_state_dict(self.state_dict())
        return new

    def forward(self, x):
        h = self.inp(x)
        if h.requires_grad:
            h.register_hook(self._late)           # runs after the layer's own backward node
        return self.out(torch.relu(self.layer(h)))

    def _late(self, g):
        x, dy, w = self.pending
        late = dy.t() @ x
        w.grad = late if w.grad is None else w.grad + late
        self.on_wgrad()
        return g


def _deferred(rank, world):
    import torch.distributed as dist

    from flex_shard_b200 import BucketSpec, flex_shard

    out = {}
    for reshard_after_forward, no_sync in ((True, False), (False, True)):
        torch.manual_seed(0)
        model = DelayedWgradModel()
        ref = copy.deepcopy(model)
        flex_shard(model, [BucketSpec([f"{n}.*"], reshard_after_forward=reshard_after_forward,
                                      defer_post_backward=(n == "layer")) for n in ("inp", "layer", "out")])
        model.on_wgrad = lambda model=model: model.finish_deferred_backward(model.layer.weight)
        ref.on_wgrad = lambda: None
        try:
            model.finish_deferred_backward(model.out.weight)
            out["non_deferring"] = ""
        except ValueError as e:
            out["non_deferring"] = str(e)
        torch.manual_seed(1 + rank)
        for step in range(2 if no_sync else 1):
            model.set_requires_gradient_sync(step == int(no_sync))
            x = torch.randn(4, 8)
            model(x).sum().backward()
            ref(x).sum().backward()
        ok = True
        for p, q in zip(model.parameters(), ref.parameters()):
            want = q.grad.clone()
            dist.all_reduce(want)
            want /= world
            ok = ok and torch.allclose(p.grad, _expected_shard(want, rank, world), atol=1e-6)
        out[f"grads_{reshard_after_forward}_{no_sync}"] = ok
    # a syncing backward that ends with the deferring bucket unfinished raises
    model.on_wgrad = lambda: None
    try:
        model(torch.randn(4, 8)).sum().backward()
        out["unfinished"] = ""
    except RuntimeError as e:
        out["unfinished"] = str(e)
    return out


def test_deferred_post_backward_waits_for_the_late_weight_gradient():
    for r in run_ranks(_deferred, 2):
        assert "does not defer" in r["non_deferring"]
        assert r["grads_True_False"] and r["grads_False_True"], r
        assert "finish_deferred_backward" in r["unfinished"]


class RankRoutedExperts(nn.Module):
    """Two experts in one bucket, of which a call uses one, and a side module whose output may go unused."""

    class Experts(nn.Module):
        def __init__(self):
            super().__init__()
            self.w0 = nn.Parameter(torch.randn(8, 8) * 0.3)
            self.w1 = nn.Parameter(torch.randn(8, 8) * 0.3)

        def forward(self, x, which):
            return x @ (self.w0 if which == 0 else self.w1).t()

    def __init__(self):
        super().__init__()
        self.experts = RankRoutedExperts.Experts()
        self.side = nn.Linear(8, 8)

    def forward(self, x, which, use_side_output):
        h = self.experts(x, which)
        s = self.side(x)                       # runs on every rank ...
        return h + s if use_side_output else h  # ... but its output may not reach the loss


def _unused(rank, world):
    import torch.distributed as dist

    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    model = RankRoutedExperts()
    ref = copy.deepcopy(model)
    # the buckets stay gathered between forward and backward: a rank that skips a bucket's backward must not
    # miss an all-gather that the other rank issues there
    flex_shard(model, [BucketSpec(["experts.*"], reshard_after_forward=False),
                       BucketSpec(["side.*"], reshard_after_forward=False)])
    ctx = model.sharded_bucket_storages[0].runtime.context
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(1 + rank))
    # three microbatches: without sync (each rank its own expert), then syncing with the ranks swapped and the side
    # output unused everywhere, then syncing with the side output unused on rank 1 only
    plan = [(False, rank, True), (True, 1 - rank, False), (True, rank, rank == 0)]
    reduces = []
    for sync, which, use_side in plan:
        model.set_requires_gradient_sync(sync)
        before = ctx.stats["reduces"]
        model(x, which, use_side).sum().backward()
        ref(x, which, use_side).sum().backward()
        reduces.append(ctx.stats["reduces"] - before)
    ok = True
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        want = q.grad.clone() if q.grad is not None else torch.zeros_like(q)
        dist.all_reduce(want)
        want /= world
        ok = ok and p.grad is not None and torch.allclose(p.grad, _expected_shard(want, rank, world), atol=1e-6)
    return {"ok": ok, "idle": ctx.idle(), "reduces": reduces}


def test_parameters_used_on_some_ranks_only():
    res = run_ranks(_unused, 2)
    assert all(r["ok"] and r["idle"] for r in res), res
    # every rank issues the same reductions: none without sync, both buckets in each syncing backward
    assert res[0]["reduces"] == res[1]["reduces"] == [0, 2, 2]


def _per_param_dtypes(rank, world):
    from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(8, 8)
            self.router = nn.Linear(8, 4, bias=False)

        def forward(self, x):
            return self.lin(x).float().sum() + self.router(x.float()).sum()

    torch.manual_seed(0)
    m = Net()
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, param_dtype_overrides={"router.*": torch.float32})
    flex_shard(m, [BucketSpec(["*"], mp_policy=mp)])
    seen = {}
    m.lin.register_forward_pre_hook(lambda mod, a: seen.__setitem__("lin", mod.weight.dtype))
    m.router.register_forward_pre_hook(lambda mod, a: seen.__setitem__("router", mod.weight.dtype))
    m(torch.randn(4, 8).bfloat16()).backward()
    return {"seen": {k: str(v) for k, v in seen.items()},
            "shard_dtypes": sorted({str(p.dtype) for p in m.parameters()}),
            "grad_dtypes": sorted({str(p.grad.dtype) for p in m.parameters()})}


def test_per_parameter_compute_dtype_overrides():
    for r in run_ranks(_per_param_dtypes, 2):
        assert r["seen"] == {"lin": "torch.bfloat16", "router": "torch.float32"}
        assert r["shard_dtypes"] == ["torch.float32"] and r["grad_dtypes"] == ["torch.float32"]


class TiedLM(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(16, 8)
        self.mid = nn.Linear(8, 8)
        self.out = nn.Linear(8, 16, bias=False)
        self.out.weight = self.emb.weight

    def forward(self, t):
        return self.out(torch.tanh(self.mid(self.emb(t))))


def _tied(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    model = TiedLM()
    ref = copy.deepcopy(model)
    flex_shard(model, [BucketSpec(["emb.*", "out.*"]), BucketSpec(["mid.*"])])
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for s in range(3):
        toks = [torch.randint(0, 16, (4, 6), generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)]
        model(toks[rank]).square().mean().backward()
        opt.step()
        opt.zero_grad()
        sum(ref(t).square().mean() for t in toks).div(world).backward()
        ropt.step()
        ropt.zero_grad()
    model.unshard()
    same_object = model.out.weight is model.emb.weight
    err = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(model.parameters(), ref.parameters()))
    model.reshard()
    return {"same": same_object and model.out.weight is model.emb.weight, "err": err,
            "n_params": len(list(model.parameters()))}


def test_tied_weights_train_like_the_unsharded_model():
    for r in run_ranks(_tied, 2):
        assert r["same"] and r["n_params"] == 3 and r["err"] < 1e-5, r


def _misc(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))
    flex_shard(m, [BucketSpec(["0.*"]), BucketSpec(["2.*"])])
    out = {}
    # an asynchronous unshard need not be waited for: the forward finishes it
    h = m.unshard(async_op=True)
    y = m(torch.randn(2, 8))
    h.wait()
    out["async_forward"] = tuple(y.shape) == (2, 4)
    y.sum().backward()
    # the sharded parameter and its view of the bucket storage share one version counter
    st = m.sharded_bucket_storages[0]
    sp = st.sharded_params[0]
    view = st.local_view(st.infos[0])
    before = view._version
    with torch.no_grad():
        sp.add_(1.0)
    out["version_shared"] = view._version == sp._version and sp._version > before
    # prefetch targets must be bucket storages
    try:
        st.set_buckets_to_forward_prefetch([m[2]])
        out["prefetch_type"] = ""
    except TypeError as e:
        out["prefetch_type"] = str(e)
    st.set_buckets_to_forward_prefetch([m.sharded_bucket_storages[1]])
    m(torch.randn(2, 8)).sum().backward()
    out["idle"] = st.runtime.context.idle()
    return out


def test_async_unshard_version_counter_and_prefetch_targets():
    for r in run_ranks(_misc, 2):
        assert r["async_forward"] and r["version_shared"] and r["idle"], r
        assert "ShardedBucketStorage" in r["prefetch_type"]
