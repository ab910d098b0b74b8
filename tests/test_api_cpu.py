"""The module-level control surface on a one-rank CPU mesh (no worker processes): bucket validation, class
swizzle, meta materialisation, state dicts, explicit unshard handles, setters, frozen parameters, and the rule
that a one-rank mesh issues no collective.  Parity: the role of the reference's ``tests/test_flex_shard_api.py``
and ``tests/test_flex_shard_state_dict.py`` (single-rank harness, ``tests/common.py:31-51``)."""
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(8, 16)
        self.b = nn.Linear(16, 4)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


@pytest.fixture(scope="module", autouse=True)
def one_rank_group():
    if dist.is_initialized():
        yield
        return
    store = dist.FileStore(tempfile.NamedTemporaryFile(delete=False).name, 1)
    dist.init_process_group("gloo", store=store, rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def _sharded(buckets=None, **kw):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = Net()
    flex_shard(m, buckets or [BucketSpec(["a.*"], **kw), BucketSpec(["b.*"], **kw)])
    return m


def test_every_parameter_belongs_to_exactly_one_bucket():
    from flex_shard_b200 import BucketSpec, flex_shard

    with pytest.raises(ValueError, match="matches no BucketSpec"):
        flex_shard(Net(), [BucketSpec(["a.*"])])
    with pytest.raises(ValueError, match="more than one BucketSpec"):
        flex_shard(Net(), [BucketSpec(["a.*"]), BucketSpec(["*"])])
    with pytest.raises((ValueError, TypeError)):
        flex_shard(Net(), [])


def test_dtype_overrides_span_the_buckets_that_share_the_policy():
    """An override may name a parameter of any bucket whose policy is equal; one that no such bucket holds is an
    error that names it (parity: ``tests/test_flex_shard_api.py:153-187`` of the reference), and nested wrapping
    is refused in both orders (``:53-109``)."""
    from dataclasses import replace

    from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard

    bf16 = MixedPrecisionPolicy(param_dtype=torch.bfloat16)
    override = replace(bf16, param_dtype_overrides={"b.weight": torch.float32})

    def shard(*policies):
        return flex_shard(Net(), [BucketSpec([f"{name}.*"], mp_policy=p) for name, p in zip("ab", policies)])

    m = shard(override, replace(bf16, param_dtype_overrides={"b.weight": torch.float32}))
    dtypes = {i.fqn: i.param_dtype for st in m.sharded_bucket_storages for i in st.infos}
    assert dtypes == {"a.weight": torch.bfloat16, "a.bias": torch.bfloat16,
                      "b.weight": torch.float32, "b.bias": torch.bfloat16}
    with pytest.raises(ValueError, match=r"buckets \[0\].*\['b\.weight'\]"):
        shard(override, bf16)

    child_first = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    flex_shard(child_first[0], [BucketSpec(["*"])])
    with pytest.raises(ValueError, match="already applied to submodule"):
        flex_shard(child_first, [BucketSpec(["*"])])
    root_first = flex_shard(nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2)), [BucketSpec(["*"])])
    with pytest.raises(ValueError, match="ancestor or descendant"):
        flex_shard(root_first[0], [BucketSpec(["*"])])


def test_bucket_hooks_receive_named_unsharded_parameters():
    """Hooks are called with the bucket's ``(fqn, unsharded parameter)`` pairs, as in the reference
    (``flex_shard/bucket_storage.py:48-49, 207-227`` there); the argument also answers for the storage, and
    ``alloc_grads_in_param_layout`` can be the pre-backward hook as it is."""
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.utils.validation import alloc_grads_in_param_layout

    seen = []

    def pre(named):
        seen.append(("pre", [(fqn, tuple(p.shape), p.grad is None) for fqn, p in named], named.name))
        for _, p in named:
            p.marker = "set in pre-backward"

    def post(named):
        seen.append(("post", [fqn for fqn, _ in named], [getattr(p, "marker", None) for _, p in named],
                     [p.grad is None for _, p in named]))

    torch.manual_seed(0)
    m = Net()
    flex_shard(m, [BucketSpec(["a.*"], pre_backward_hook=pre, post_reduce_hook=post),
                   BucketSpec(["b.*"], pre_backward_hook=alloc_grads_in_param_layout)])
    m(torch.randn(3, 8)).sum().backward()
    assert seen[0] == ("pre", [("a.weight", (16, 8), True), ("a.bias", (16,), True)], "a")
    assert seen[1] == ("post", ["a.weight", "a.bias"], ["set in pre-backward"] * 2, [True, True])
    assert all(p.grad is not None for p in m.parameters())


def test_reference_call_forms_are_accepted():
    """Setters take the reference's keyword names and ``recurse``; ``init_from_full(local, layout, init_fn)`` and
    ``set_sharding_info(tensor, placements, global_shape, global_stride, mesh)`` take its positional forms
    (``flex_shard/flex_shard.py:262-394``, ``param_init.py:18``, ``sharded_param.py:57`` there)."""
    from flex_shard_b200 import (GlobalLayout, get_flex_shard_global_layouts, get_global_shape, get_placements,
                                 init_from_full, is_flex_shard_param)
    from flex_shard_b200.placements import Shard
    from flex_shard_b200.sharded_param import set_sharding_info

    m = _sharded()
    m.set_requires_gradient_sync(requires_gradient_sync=False, recurse=True)
    assert not any(st.requires_gradient_sync for st in m.sharded_bucket_storages)
    m.set_requires_gradient_sync(True, recurse=False)
    m.set_reshard_after_backward(reshard_after_backward=False)
    m.set_gradient_divide_factor(2.0, recurse=True)
    m.set_gradient_divide_factor(None)
    m.set_gradient_reduce_op(dist.ReduceOp.SUM, recurse=True)
    m.set_separate_reduce_scatter_group(enable=False)
    m.set_max_pending_reduce_grads(max_pending_reduce_grads=2, recurse=True)
    m.set_max_pending_reduce_grads()
    m.unshard(async_op=False)
    m.reshard()

    layouts = get_flex_shard_global_layouts(m)
    w = dict(m.named_parameters())["a.weight"]
    init_from_full(w, layouts["a.weight"], lambda full: full.fill_(3.0))
    assert bool((w.detach() == 3.0).all())
    init_from_full(w, lambda full: full.fill_(4.0))
    assert bool((w.detach() == 4.0).all())
    half = torch.zeros(2, 4)      # rows 2..3 of a [4, 4] tensor
    init_from_full(half, GlobalLayout((4, 4), ((2, 0),), ((0, 0),), ((2, 4),)),
                   lambda full: full.copy_(torch.arange(16.0).view(4, 4)))
    assert half.tolist() == [[8, 9, 10, 11], [12, 13, 14, 15]]
    with pytest.raises(TypeError):
        init_from_full(half, "not a layout", lambda full: None)

    t = torch.zeros(2, 3)
    set_sharding_info(t, (Shard(0),), torch.Size((4, 3)), (3, 1), None)
    assert is_flex_shard_param(t) and get_placements(t) == (Shard(0),) and tuple(get_global_shape(t)) == (4, 3)
    with pytest.raises(TypeError):
        set_sharding_info(t, (Shard(0),), (4, 3), (3, 1), None, placement=Shard(0))
    with pytest.raises(ValueError, match="1-D"):
        set_sharding_info(t, (Shard(0), Shard(1)), (4, 3), (3, 1), None)


def test_storage_and_param_info_answer_to_the_reference_names():
    """Read-only names of the reference's ``ShardedBucketStorage`` and ``ParamInfo``
    (``flex_shard/bucket_storage.py:283-340, 742-800, 961-969`` there)."""
    from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard

    m = Net()
    m.a.weight.grad_dtype = torch.float64
    flex_shard(m, [BucketSpec(["a.*"], mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16)),
                   BucketSpec(["b.*"], gradient_divide_factor=4.0)])
    a, b = m.sharded_bucket_storages
    assert a.flat_storage is a.byte_storage and a.numel == a.total_bytes == a.byte_storage.numel()
    assert list(a.param_infos) == ["a.weight", "a.bias"] and a.world_size == 1
    assert b.gradient_reduce_op == dist.ReduceOp.AVG and b.gradient_divide_factor == 4.0
    assert b.gradient_reduction.divide_factor == 4.0 and a.gradient_divide_factor is None
    assert a.reduce_mesh is a.mesh
    assert a.get_local_view("a.bias").shape == (16,) and a.get_local_view("a.bias").data_ptr() == m.a.bias.data_ptr()
    info = a.param_infos["a.weight"]
    assert info.placements == (info.placement,) and info.dtype == torch.float32
    assert info.unsharded_dtype == torch.bfloat16 and info.has_explicit_grad_dtype
    assert info.grad_dtype_override == torch.float64 and info.grad_reduce_dtype == torch.float64
    plain = b.param_infos["b.weight"]
    assert not plain.has_explicit_grad_dtype and plain.grad_dtype_override is None
    assert plain.unsharded_dtype == plain.grad_reduce_dtype == torch.float32


def test_flex_shard_applies_once():
    from flex_shard_b200 import BucketSpec, flex_shard

    m = _sharded()
    with pytest.raises(ValueError, match="already applied"):
        flex_shard(m, [BucketSpec(["*"])])


def test_class_swizzle_keeps_the_original_class():
    from flex_shard_b200 import FlexShardModule

    m = _sharded()
    assert isinstance(m, Net) and isinstance(m, FlexShardModule)
    assert type(m).__name__ == "FlexShardNet"
    assert [st.name for st in m.sharded_bucket_storages] == ["a", "b"]
    assert [[i.fqn for i in st.infos] for st in m.sharded_bucket_storages] == [["a.weight", "a.bias"], ["b.weight", "b.bias"]]


def test_training_step_matches_the_plain_module():
    m = _sharded()
    torch.manual_seed(0)
    ref = Net()
    opt, ropt = torch.optim.SGD(m.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    ids = [id(p) for p in m.parameters()]
    for s in range(3):
        x = torch.randn(4, 8, generator=torch.Generator().manual_seed(s))
        for mod, o in ((m, opt), (ref, ropt)):
            mod(x).square().mean().backward()
            o.step()
            o.zero_grad()
    assert ids == [id(p) for p in m.parameters()]            # the optimizer keeps seeing the same parameters
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        assert torch.equal(p.detach(), q.detach()), n


def test_one_rank_mesh_issues_no_collective(monkeypatch):
    def boom(*a, **k):
        raise AssertionError("a one-rank mesh must not call a collective")

    for name in ("all_gather_into_tensor", "reduce_scatter_tensor", "all_reduce", "all_gather", "all_to_all_single"):
        monkeypatch.setattr(dist, name, boom)
    m = _sharded()
    m(torch.randn(4, 8)).square().mean().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_state_dict_has_the_plain_keys_and_reshards_first():
    m = _sharded()
    plain = Net().state_dict()
    m.unshard()
    assert m.sharded_bucket_storages[0].runtime.is_unsharded
    sd = m.state_dict()
    assert not m.sharded_bucket_storages[0].runtime.is_unsharded      # the pre-hook put the shards back
    assert list(sd) == list(plain) and all(sd[k].shape == plain[k].shape for k in sd)
    other = _sharded()
    with torch.no_grad():
        for p in other.parameters():
            p.zero_()
    other.load_state_dict(sd)
    x = torch.randn(4, 8)
    assert torch.equal(other(x), m(x))


def test_explicit_unshard_returns_a_handle_and_rejects_backward():
    m = _sharded()
    h = m.unshard(async_op=True)
    assert type(h).__name__ == "ModuleUnshardHandle"
    h.wait()
    assert all(st.runtime.is_unsharded for st in m.sharded_bucket_storages)
    m.reshard()
    assert not any(st.runtime.is_unsharded for st in m.sharded_bucket_storages)
    assert m.unshard() is None
    m.reshard()
    seen = []

    def hook(g):
        try:
            m.unshard()
        except RuntimeError as e:
            seen.append(str(e))
        return g

    y = m(torch.randn(4, 8))
    y.register_hook(hook)
    y.square().mean().backward()
    assert seen and "cannot run in backward" in seen[0]


def test_setters_validate_their_arguments():
    m = _sharded()
    with pytest.raises(ValueError, match=">= 1"):
        m.set_max_pending_reduce_grads(0)
    with pytest.raises(ValueError, match="AVG or SUM"):
        m.set_gradient_reduce_op("sum")
    m.set_gradient_reduce_op(dist.ReduceOp.SUM)
    m.set_gradient_divide_factor(4.0)
    m.set_max_pending_reduce_grads(2)
    m.set_reshard_after_backward(False)
    m.set_reshard_after_forward(False)
    m.set_requires_gradient_sync(True)
    assert m.sharded_bucket_storages[0].runtime.context.max_pending_reduce_grads == 2
    with pytest.raises(ValueError, match="not managed"):
        m.bucket_storage_of(nn.Parameter(torch.zeros(1)))
    st = m.sharded_bucket_storages[1]
    assert m.bucket_storage_of(st.sharded_params[0]) is st


def test_divide_factor_scales_the_reduced_gradient():
    """With SUM and a divide factor f the sharded gradient is the local gradient / f (one rank)."""
    m, ref = _sharded(), _sharded()
    m.set_gradient_reduce_op(dist.ReduceOp.SUM)
    m.set_gradient_divide_factor(4.0)
    x = torch.randn(4, 8)
    for mod in (m, ref):
        mod(x).square().mean().backward()
    for p, q in zip(m.parameters(), ref.parameters()):
        torch.testing.assert_close(p.grad, q.grad / 4.0)


def test_meta_module_is_materialised_by_to_empty():
    from flex_shard_b200 import BucketSpec, flex_shard

    with torch.device("meta"):
        m = Net()
    flex_shard(m, [BucketSpec(["*"])])
    with pytest.raises(RuntimeError, match="to_empty"):
        m.unshard()
    assert all(p.device.type == "meta" for p in m.parameters())
    m.to_empty(device="cpu")
    assert all(p.device.type == "cpu" for p in m.parameters())
    with torch.no_grad():
        for p in m.parameters():
            p.normal_()
    assert m(torch.randn(2, 8)).shape == (2, 4)
    m(torch.randn(2, 8)).sum().backward()
    assert all(p.grad is not None for p in m.parameters())


def test_frozen_parameters_get_no_gradient_and_no_reduction():
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = Net()
    for p in m.a.parameters():
        p.requires_grad_(False)
    flex_shard(m, [BucketSpec(["a.*"]), BucketSpec(["b.*"])])
    ctx = m.sharded_bucket_storages[0].runtime.context
    before = ctx.stats["reduces"]
    m(torch.randn(4, 8)).square().mean().backward()
    assert all(p.grad is None for p in m.a.parameters()) and all(p.grad is not None for p in m.b.parameters())
    assert ctx.stats["reduces"] - before == 1          # only the trainable bucket reduced
    assert ctx.idle()


def test_shared_parameter_is_stored_once():
    """Tied weights (one Parameter under two names) land in one bucket slot and stay tied after sharding."""
    from flex_shard_b200 import BucketSpec, flex_shard

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(10, 8)
            self.out = nn.Linear(8, 10, bias=False)
            self.out.weight = self.emb.weight

        def forward(self, t):
            return self.out(self.emb(t))

    m = Tied()
    flex_shard(m, [BucketSpec(["*"])])
    assert m.out.weight is m.emb.weight
    assert len(list(m.parameters())) == 1
    m(torch.randint(0, 10, (3, 5))).square().mean().backward()
    assert m.emb.weight.grad is not None and m.out.weight is m.emb.weight
