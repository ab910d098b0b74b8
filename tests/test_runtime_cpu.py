"""Runtime scheduling contracts on 2 gloo ranks: learned prefetch counts, persistent unsharded
parameters, no-sync accumulation, manual finalisation, unshard-in-backward, separate
reduce-scatter group, bucket lookup, and poisoning after a raising backward.

The asserted numbers are the reference's own goldens (``tests/test_flex_shard_runtime.py``:
6 unshards for 3 buckets per step with 4 prefetch hits from the second step on; storage size 0
while resharded; "cannot run in backward"; "wait on the previous"; "a previous backward raised")."""
import torch
import torch.nn as nn

from tests.common import run_ranks


class Stack(nn.Sequential):
    def __init__(self):
        super().__init__(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 4))


class Boom(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a):
        return a.clone()

    @staticmethod
    def backward(ctx, g):
        raise RuntimeError("boom")


def _work(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    out = {}
    torch.manual_seed(0)
    m = Stack()
    # listed in reverse order on purpose: the schedule follows execution order, not the spec order
    flex_shard(m, [BucketSpec(["4.*"]), BucketSpec(["2.*"]), BucketSpec(["0.*"])])
    storages = m.sharded_bucket_storages
    ctx = storages[0].runtime.context
    x = torch.randn(4, 8)

    def step():
        before = dict(ctx.stats)
        m(x).square().mean().backward()
        return {k: ctx.stats[k] - before[k] for k in before}

    out["steps"] = [step() for _ in range(3)]
    rt = storages[0].runtime
    out["resharded_storage"] = [p.untyped_storage().size() for p in rt.unsharded_params]
    ids = [id(p) for s in storages for p in s.runtime.unsharded_params]
    step()
    out["identity_stable"] = ids == [id(p) for s in storages for p in s.runtime.unsharded_params]
    out["idle_between_steps"] = ctx.idle()

    def grads():
        return [p.grad.clone() for p in m.parameters()]

    def clear():
        for p in m.parameters():
            p.grad = None

    clear()
    step()
    g1 = grads()
    # no-sync microbatch then a syncing one: one reduction per bucket, gradient of both microbatches
    clear()
    m.set_requires_gradient_sync(False)
    out["nosync"] = step()
    out["nosync_has_sharded_grads"] = any(p.grad is not None for p in m.parameters())
    m.set_requires_gradient_sync(True)
    out["sync"] = step()
    out["accumulated_is_2x"] = all(torch.allclose(a, 2 * b, atol=1e-6) for a, b in zip(grads(), g1))
    # unshard() from inside backward
    msgs = []

    def hook(g):
        try:
            m.unshard()
        except RuntimeError as e:
            msgs.append(str(e))
        return g

    clear()
    y = m(x)
    y.register_hook(hook)
    y.square().mean().backward()
    out["unshard_in_backward"] = msgs
    # manual finalisation
    clear()
    m.set_manual_backward_finalization(True)
    out["manual_backward"] = step()
    h = m.finalize_backward(async_op=True)
    try:
        m.finalize_backward(async_op=True)
        out["second_finalize"] = ""
    except RuntimeError as e:
        out["second_finalize"] = str(e)
    before = ctx.stats["reduces"]
    h.wait()
    out["manual_grads_equal"] = all(torch.allclose(p.grad, b, atol=1e-6) for p, b in zip(m.parameters(), g1))
    m.set_manual_backward_finalization(False)
    # bucket lookup by either face of a parameter
    st = storages[1]
    out["storage_of"] = (m.bucket_storage_of(st.sharded_params[0]) is st,
                         m.bucket_storage_of(st.runtime.unsharded_params[0]) is st)
    # separate reduce-scatter group: same bits
    clear()
    m.set_separate_reduce_scatter_group(True)
    step()
    out["separate_rs_group_bitwise"] = all(torch.equal(p.grad, b) for p, b in zip(m.parameters(), g1))
    m.set_separate_reduce_scatter_group(True)   # idempotent
    m.set_separate_reduce_scatter_group(False)
    # a backward that raises half-way poisons the runtime
    clear()
    try:
        m[4](torch.relu(Boom.apply(m[2](torch.relu(m[0](x)))))).square().mean().backward()
        out["boom"] = ""
    except RuntimeError as e:
        out["boom"] = str(e)
    for name, fn in (("forward_after", lambda: m(x)), ("reshard_after", lambda: m.reshard())):
        try:
            fn()
            out[name] = ""
        except RuntimeError as e:
            out[name] = str(e)
    return out


def test_runtime_contracts():
    for r in run_ranks(_work, 2):
        assert r["steps"][0] == {"unshards": 6, "prefetch_hits": 0, "reduces": 3}
        assert r["steps"][1] == {"unshards": 6, "prefetch_hits": 4, "reduces": 3}
        assert r["steps"][2] == r["steps"][1]
        assert r["resharded_storage"] == [0, 0] and r["identity_stable"] and r["idle_between_steps"]
        assert r["nosync"]["reduces"] == 0 and not r["nosync_has_sharded_grads"]
        assert r["sync"]["reduces"] == 3 and r["accumulated_is_2x"]
        assert r["unshard_in_backward"] and all("cannot run in backward" in s for s in r["unshard_in_backward"])
        assert r["manual_backward"]["reduces"] == 0
        assert "wait on the previous" in r["second_finalize"] and r["manual_grads_equal"]
        assert r["storage_of"] == (True, True)
        assert r["separate_rs_group_bitwise"]
        assert r["boom"] == "boom"
        assert "a previous backward raised" in r["forward_after"]
        assert "a previous backward raised" in r["reshard_after"]
