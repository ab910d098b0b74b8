"""Bucket and placement validation before anything is materialised (one-rank CPU mesh, no worker processes).
Parity: the behaviours pinned by the reference's ``tests/test_flex_shard_buckets.py:91-440`` (assignment of
parameters to buckets, tied parameters, placement-function contract, mixed dtypes / placements, shard dims)."""
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


class Tied(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(10, 8)
        self.norm = nn.LayerNorm(8)
        self.out = nn.Linear(8, 10, bias=False)
        self.out.weight = self.emb.weight

    def forward(self, t):
        return self.out(self.norm(self.emb(t)))


@pytest.fixture(scope="module", autouse=True)
def one_rank_group():
    if dist.is_initialized():
        yield
        return
    dist.init_process_group("gloo", store=dist.FileStore(tempfile.NamedTemporaryFile(delete=False).name, 1),
                            rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def _spec(patterns, **kw):
    from flex_shard_b200 import BucketSpec

    return BucketSpec(patterns, **kw)


def _untouched(m):
    """Validation failed before materialisation: the module still holds its own plain parameters."""
    from flex_shard_b200 import FlexShardModule

    return not isinstance(m, FlexShardModule) and all(type(p) is nn.Parameter for p in m.parameters())


def test_patterns_must_be_a_sequence_and_the_module_a_module():
    from flex_shard_b200 import BucketSpec, flex_shard

    with pytest.raises(TypeError, match="not a string"):
        BucketSpec("a.*")
    with pytest.raises(TypeError, match="nn.Module"):
        flex_shard([1], [BucketSpec(["*"])])


def test_tied_parameter_names_must_share_one_bucket():
    from flex_shard_b200 import flex_shard

    m = Tied()
    flex_shard(m, [_spec(["emb.*", "norm.*", "out.*"])])                     # every name in one bucket: accepted
    assert [i.fqn for i in m.sharded_bucket_storages[0].infos] == ["emb.weight", "norm.weight", "norm.bias"]
    m = Tied()
    with pytest.raises(ValueError, match=r"(?s)'emb\.weight' is shared with.*out\.weight -> bucket 1.*same BucketSpec"):
        flex_shard(m, [_spec(["emb.*"]), _spec(["norm.*", "out.*"])])
    assert _untouched(m)
    m = Tied()
    with pytest.raises(ValueError, match=r"out\.weight -> no bucket"):
        flex_shard(m, [_spec(["emb.*", "norm.*"])])
    assert _untouched(m)


def test_placement_fn_must_cover_exactly_the_bucket():
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.placements import Shard

    m = Net()
    with pytest.raises(ValueError, match="no placement for"):
        flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {named[0][0]: Shard(0)})])
    assert _untouched(m)
    with pytest.raises(ValueError, match="not in the bucket"):
        flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {**{f: Shard(0) for f, _ in named}, "zzz": Shard(0)})])
    assert _untouched(m)
    with pytest.raises(TypeError, match="is not a Placement"):
        flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {f: "Shard(0)" for f, _ in named})])
    assert _untouched(m)


def test_incomplete_placement_contract_is_rejected():
    """A Placement subclass that leaves the abstract hooks out cannot be instantiated at all."""
    from flex_shard_b200.placement_contract import Placement

    class Half(Placement):
        def compute_local_shape(self, shape, rank, world_size):
            return tuple(shape)

    with pytest.raises(TypeError, match="abstract"):
        Half()


def test_shard_dim_and_uneven_nonzero_dim_are_rejected():
    from flex_shard_b200.placements import Shard

    with pytest.raises(ValueError, match="does not apply"):
        Shard(3).compute_local_shape((16, 8), 0, 2)
    assert Shard(0).compute_local_shape((5, 8), 0, 2) == (3, 8)          # dim 0 may be uneven (padded slot)
    assert Shard(0).compute_local_shape((5, 8), 1, 2) == (2, 8)
    assert Shard(1).compute_local_shape((16, 8), 1, 2) == (16, 4)
    with pytest.raises(ValueError):
        Shard(1).compute_local_shape((16, 7), 0, 2)                      # only dim 0 pads


def test_bucket_rejects_mixed_dtypes_and_mixed_placements():
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.placements import BlockShard, Shard

    m = Net()
    m.b.to(torch.bfloat16)
    with pytest.raises(ValueError, match="mixes parameter dtypes"):
        flex_shard(m, [_spec(["*"])])
    assert _untouched(m)
    flex_shard(m, [_spec(["a.*"]), _spec(["b.*"])])                      # one dtype per bucket is fine
    m = Net()
    with pytest.raises(ValueError, match="mixes incompatible placements"):
        flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {
            f: (Shard(0) if i % 2 else BlockShard((1,), 0)) for i, (f, _) in enumerate(named)})])
    assert _untouched(m)


def test_shard_dims_may_mix_in_one_bucket():
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.placements import Shard

    torch.manual_seed(0)
    m, ref = Net(), Net()
    ref.load_state_dict(m.state_dict())
    flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {f: Shard(1 if p.dim() == 2 else 0) for f, p in named})])
    x = torch.randn(4, 8)
    assert torch.equal(m(x), ref(x))


def test_fsdp2_compatible_needs_shard_and_offload_is_refused():
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.placements import BlockShard

    m = Net()
    with pytest.raises(ValueError, match="requires Shard placements"):
        flex_shard(m, [_spec(["*"], fsdp2_compatible=True,
                             placement_fn=lambda named, mesh: {f: BlockShard((1,), 0) for f, _ in named})])
    with pytest.raises(ValueError, match="offload_policy is not supported"):
        flex_shard(m, [_spec(["*"], offload_policy=object())])
    assert _untouched(m)


def test_multi_dim_mesh_is_rejected():
    from torch.distributed.device_mesh import init_device_mesh

    from flex_shard_b200 import flex_shard

    mesh = init_device_mesh("cpu", (1, 1), mesh_dim_names=("a", "b"))
    with pytest.raises(ValueError, match="1-D mesh"):
        flex_shard(Net(), [_spec(["*"], mesh=mesh)])
    m = Net()
    flex_shard(m, [_spec(["*"], mesh=mesh["b"])])                           # a 1-D slice of it is fine
    assert m(torch.randn(2, 8)).shape == (2, 4)


def test_sharded_parameters_are_views_of_the_bucket_storage():
    from flex_shard_b200 import flex_shard

    m = Net()
    flex_shard(m, [_spec(["a.*"]), _spec(["b.*"])])
    for st in m.sharded_bucket_storages:
        base = st.byte_storage.untyped_storage().data_ptr()
        assert all(sp.untyped_storage().data_ptr() == base for sp in st.sharded_params)
        # writing through the storage is writing the parameters
        st.byte_storage.zero_()
        assert all(float(sp.detach().abs().sum()) == 0.0 for sp in st.sharded_params)


def test_reference_style_placement_functions_are_accepted():
    """The reference's factory names exist, and a placement function that returns one-element tuples
    ``{fqn: (placement,)}`` (its convention for a 1-D mesh) is accepted like one that returns bare placements."""
    from flex_shard_b200 import flex_shard
    from flex_shard_b200 import placements as P

    assert P.make_shard_placement_fn is P.shard_placement_fn
    assert P.make_bucketed_block_placement_fn is P.make_bucketed_block_shard_placement_fn
    assert P.make_fp8_bucketed_block_placement_fn is P.make_fp8_bucketed_block_shard_placement_fn
    assert P.make_mxfp8_bucketed_block_placement_fn is P.make_mxfp8_bucketed_block_shard_placement_fn
    named = [("w", nn.Parameter(torch.zeros(4, 4)))]
    assert P.per_param_placements(named, None) == {"w": P.Shard(0)}
    torch.manual_seed(0)
    m, ref = Net(), Net()
    ref.load_state_dict(m.state_dict())
    flex_shard(m, [_spec(["*"], placement_fn=lambda named, mesh: {f: (P.Shard(0),) for f, _ in named})])
    x = torch.randn(3, 8)
    assert torch.equal(m(x), ref(x))


def test_module_name_patterns_may_not_mix_with_parameter_patterns_or_name_containers():
    from flex_shard_b200 import flex_shard

    seq = nn.Sequential(nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 8), nn.ReLU(), nn.Linear(8, 8))
    with pytest.raises(ValueError, match="mixes module names and parameter patterns"):
        flex_shard(seq, [_spec(["0", "2.*"]), _spec(["4.*"])])
    with pytest.raises(ValueError, match="without a forward"):
        flex_shard(nn.Sequential(nn.ModuleList([nn.Linear(8, 8)])), [_spec(["0"])])
    flex_shard(seq, [_spec(["0", "2"]), _spec(["4"])])            # sibling modules in one bucket
    assert [[i.fqn for i in st.infos] for st in seq.sharded_bucket_storages] == [
        ["0.weight", "0.bias", "2.weight", "2.bias"], ["4.weight", "4.bias"]]
    assert seq(torch.randn(2, 8)).shape == (2, 8)
