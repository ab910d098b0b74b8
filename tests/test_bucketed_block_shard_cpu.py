"""``BucketedBlockShard`` (flat parameter-major buckets): plan geometry, identity of placements, rejected
configurations, views into the bucket, local shapes that keep the parameter's rank.  One-rank mesh or no mesh at all.
Parity: the behaviours pinned by the reference's ``tests/test_flex_shard_block_shard.py:60-380``."""
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from tests.common import FakeMesh


@pytest.fixture(scope="module", autouse=True)
def one_rank_group():
    if dist.is_initialized():
        yield
        return
    dist.init_process_group("gloo", store=dist.FileStore(tempfile.NamedTemporaryFile(delete=False).name, 1),
                            rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def test_equality_hash_and_repr_follow_the_blocks():
    from flex_shard_b200.placements import BlockShard, BucketedBlockShard

    a, b, c = BucketedBlockShard((1, 1)), BucketedBlockShard((1, 1)), BucketedBlockShard((1, 3))
    assert a == b and hash(a) == hash(b) and a != c
    assert a != BlockShard((1, 1), 0)                                 # a per-parameter block shard is another placement
    assert "blocks_per_rank=(1, 3)" in repr(c)
    assert a.bucket_compatibility_key() != c.bucket_compatibility_key()


def test_invalid_configurations_are_rejected():
    from flex_shard_b200.placements import BucketedBlockShard

    with pytest.raises(ValueError, match="dims"):
        BucketedBlockShard((1, 1), dims=(1,))
    with pytest.raises(ValueError, match="positive sum"):
        BucketedBlockShard((0, 0))
    with pytest.raises(ValueError, match="non-negative"):
        BucketedBlockShard((2, -1))
    with pytest.raises(ValueError, match="mesh has 4"):
        BucketedBlockShard((1, 1)).compute_local_shape((8, 4), 0, 4)
    with pytest.raises(RuntimeError, match="bucket plan"):
        BucketedBlockShard((1, 1)).extract_local_shard(torch.zeros(8, 4), 0, 2)


def test_placement_fn_uses_the_mesh_size():
    from flex_shard_b200.placements import make_bucketed_block_shard_placement_fn

    named = [("w", nn.Parameter(torch.zeros(8, 4))), ("b", nn.Parameter(torch.zeros(8)))]
    for W in (2, 4):
        pls = make_bucketed_block_shard_placement_fn()(named, FakeMesh(W))
        assert all(pl.blocks_per_rank == (1,) * W for pl in pls.values())
    uneven = make_bucketed_block_shard_placement_fn((1, 3))(named, FakeMesh(2))
    assert all(pl.blocks_per_rank == (1, 3) for pl in uneven.values())
    with pytest.raises(ValueError):
        make_bucketed_block_shard_placement_fn((1, 3))(named, FakeMesh(4))      # blocks for 2 ranks on a 4-rank mesh


def test_plan_cuts_fall_on_whole_rows_of_every_parameter():
    from flex_shard_b200.placements.bucketed_block_shard import FlatBucketPlan

    shapes = [(5, 6), (7,), (3, 4)]
    plan = FlatBucketPlan(shapes, (1, 1, 2))
    assert plan.align == 12                                            # lcm of the row sizes 6, 1, 4
    assert all(off % plan.align == 0 for off in plan.param_off)       # parameters start on aligned offsets
    assert plan.padded_total % (plan.align * 4) == 0 and plan.padded_total >= plan.total
    assert [plan.rank_range(r) for r in range(3)] == [(0, plan.block), (plan.block, 2 * plan.block),
                                                      (2 * plan.block, 4 * plan.block)]
    for i, s in enumerate(shapes):
        covered = []
        for r in range(3):
            r0, r1 = plan.local_rows(i, r)
            assert 0 <= r0 <= r1 <= s[0]
            covered += list(range(r0, r1))
        assert covered == list(range(s[0]))                            # every row on exactly one rank, in order
    assert not plan.uniform and FlatBucketPlan(shapes, (1, 1)).uniform


def test_a_rank_may_hold_padding_only():
    """More ranks than rows: the last ranks' ranges lie in the padding and hold no parameter rows."""
    from flex_shard_b200.placements.bucketed_block_shard import FlatBucketPlan

    plan = FlatBucketPlan([(2, 8)], (1, 1, 1, 1))
    rows = [plan.local_rows(0, r) for r in range(4)]
    assert sum(b - a for a, b in rows) == 2 and any(a == b for a, b in rows)


def test_sharded_parameters_are_views_into_one_flat_bucket_and_keep_their_rank():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import make_bucketed_block_shard_placement_fn

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(6, 5), nn.Linear(5, 3))
    ref = nn.Sequential(nn.Linear(6, 5), nn.Linear(5, 3))
    ref.load_state_dict(m.state_dict())
    flex_shard(m, [BucketSpec(["*"], placement_fn=make_bucketed_block_shard_placement_fn())])
    st = m.sharded_bucket_storages[0]
    base = st.byte_storage.untyped_storage().data_ptr()
    for sp, info in zip(st.sharded_params, st.infos):
        assert sp.untyped_storage().data_ptr() == base
        assert sp.dim() == len(info.global_shape)                       # a matrix stays a matrix, a vector a vector
    # view-in / view-out: the gathered parameters alias one bucket too
    m.unshard()
    ups = st.runtime.unsharded_params
    assert len({u.untyped_storage().data_ptr() for u in ups}) == 1
    m.reshard()
    x = torch.randn(4, 6)
    assert torch.equal(m(x), ref(x))
    m(x).square().mean().backward()
    ref(x).square().mean().backward()
    for p, q in zip(m.parameters(), ref.parameters()):
        assert p.grad.shape == p.shape and torch.allclose(p.grad, q.grad, atol=1e-6)
    # the reduced gradients come back as views of one local gradient buffer
    assert len({p.grad.untyped_storage().data_ptr() for p in m.parameters()}) == 1


def test_mixed_block_configurations_cannot_share_a_bucket():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import BucketedBlockShard

    m = nn.Sequential(nn.Linear(6, 5), nn.Linear(5, 3))
    with pytest.raises(ValueError, match="mixes incompatible placements"):
        flex_shard(m, [BucketSpec(["*"], placement_fn=lambda named, mesh: {
            f: BucketedBlockShard((1,) if i % 2 else (2,)) for i, (f, _) in enumerate(named)})])


def _padding_only_ranks(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.placements import make_bucketed_block_shard_placement_fn

    torch.manual_seed(0)
    m, ref = nn.Linear(8, 1, bias=False), nn.Linear(8, 1, bias=False)
    ref.load_state_dict(m.state_dict())
    flex_shard(m, [BucketSpec(["*"], placement_fn=make_bucketed_block_shard_placement_fn())])
    held = m.weight.numel()
    opt, ropt = torch.optim.SGD(m.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for s in range(2):
        xs = [torch.randn(3, 8, generator=torch.Generator().manual_seed(10 * s + r)) for r in range(world)]
        m(xs[rank]).square().mean().backward()
        opt.step()
        opt.zero_grad()
        sum(ref(x).square().mean() for x in xs).div(world).backward()
        ropt.step()
        ropt.zero_grad()
    m.unshard()
    err = float((m.weight.detach() - ref.weight.detach()).abs().max())
    m.reshard()
    return held, err


def test_ranks_that_hold_only_padding_train_with_the_others():
    """One row on four ranks: three ranks store nothing and still take part in every collective; the result equals
    the unsharded model (the reference refuses such a rank, ``tests/test_flex_shard_block_shard.py:203-246`` there)."""
    from tests.common import run_ranks

    res = run_ranks(_padding_only_ranks, 4)
    assert sorted(h for h, _ in res) == [0, 0, 0, 8]
    assert all(err < 1e-6 for _, err in res)
