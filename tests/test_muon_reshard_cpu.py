"""DistMuon's redistribution machinery without GPUs: validated region plans, packed all-to-all schedules,
the cross-rank plan digest, compute-layout resolution and its validator, and the two-slot pipelined
runtime on gloo ranks (restating the behaviours of ``src/flex_shard/tests/test_optimizer_reshard_schedule.py``
and ``test_dist_muon_optimizer.py`` of the reference for plain local tensors)."""
import math

import pytest
import torch

from tests.common import run_ranks


# --------------------------------------------------------------------------- plans
def test_row_plan_routes_tile_exactly_and_invert():
    from flex_shard_b200.dist_muon.reshard_plan import plan_rows

    # 10 x 3 matrix, Shard(0) over 4 ranks (chunk 3: rows 0-3, 3-6, 6-9, 9-10), whole matrix owned by rank 2
    plan = plan_rows((10, 3), [(0, 3), (3, 6), (6, 9), (9, 10)], [(0, 10, 2)])
    assert [p.tensor_shape for p in plan.storage] == [(3, 3), (3, 3), (3, 3), (1, 3)]
    assert [p.tensor_shape for p in plan.compute] == [(0, 3), (0, 3), (10, 3), (0, 3)]
    assert [(r.src_rank, r.dst_rank, r.dst_region.offsets[0], r.logical.shape[0]) for r in plan.routes] == [
        (0, 2, 0, 3), (1, 2, 3, 3), (2, 2, 6, 3), (3, 2, 9, 1)]
    assert not plan.is_local
    back = plan.back_routes
    assert all(b.src_rank == f.dst_rank and b.src_region == f.dst_region and b.dst_region == f.src_region
               for f, b in zip(plan.routes, back))


def test_head_blocks_split_across_storage_boundaries():
    from flex_shard_b200.dist_muon.reshard_plan import plan_rows

    # 12 rows in heads of 4, stored 5/5/2 (uneven on purpose), heads owned by ranks 1, 0, 1
    plan = plan_rows((12, 2), [(0, 5), (5, 10), (10, 12)], [(0, 4, 1), (4, 8, 0), (8, 12, 1)])
    assert plan.compute[1].tensor_shape == (8, 2) and plan.compute[0].tensor_shape == (4, 2)
    # head 1 (rows 4-8) straddles ranks 0 and 1: one row from rank 0, three from rank 1
    h1 = [(r.src_rank, r.logical.offsets[0], r.logical.shape[0]) for r in plan.routes if r.dst_rank == 0]
    assert h1 == [(0, 4, 1), (1, 5, 3)]
    # rank 1's compute tensor stacks head 0 then head 2
    tops = sorted((r.dst_region.offsets[0], r.logical.offsets[0]) for r in plan.routes if r.dst_rank == 1)
    assert tops == [(0, 0), (4, 8), (6, 10)]


def test_plan_validation_names_the_defect():
    from flex_shard_b200.dist_muon.reshard_plan import (Partition, PlanError, RedistributionPlan, Region, Route,
                                                        plan_rows, rows_region)

    good = plan_rows((4, 2), [(0, 2), (2, 4)], [(0, 4, 0)])
    shape = (4, 2)
    with pytest.raises(PlanError, match="cover"):     # a storage region is missing
        RedistributionPlan(2, shape, (good.storage[0], Partition(1, (0, 2), ())), good.compute, good.routes)
    with pytest.raises(PlanError, match="overlap"):
        RedistributionPlan(2, shape, (Partition(0, (2, 2), (rows_region(0, 2, shape),)),
                                      Partition(1, (2, 2), (rows_region(1, 3, shape),))), good.compute, good.routes)
    bad_route = Route(rows_region(0, 2, shape), 0, rows_region(0, 2, shape), 0, Region((0, 0), (1, 2)))
    with pytest.raises(PlanError, match="differ in size"):
        RedistributionPlan(2, shape, good.storage, good.compute, (bad_route, good.routes[1]))
    with pytest.raises(PlanError, match="outside the group"):
        plan_rows(shape, [(0, 2), (2, 4)], [(0, 4, 5)])
    with pytest.raises(PlanError, match="routes"):    # a route missing: the routes no longer tile the tensor
        RedistributionPlan(2, shape, good.storage, good.compute, good.routes[:1])


def test_packed_schedule_splits_and_spans():
    from flex_shard_b200.dist_muon.reshard_plan import pack, packed_schedule, plan_rows, unpack

    W = 3
    rows = [(0, 4), (4, 8), (8, 10)]
    plans = [plan_rows((10, 2), rows, [(0, 10, 1)]),                      # whole matrix -> rank 1
             plan_rows((10, 1), rows, [(0, 5, 2), (5, 10, 0)])]           # two blocks -> ranks 2 and 0
    scheds = [packed_schedule(plans, r, True) for r in range(W)]
    # rank 0 sends 8 elements of the first parameter to rank 1 and 4 of the second to rank 2
    assert scheds[0].send_splits == (0, 8, 4) and scheds[0].recv_splits == (0, 3, 2)
    assert scheds[1].recv_splits == (8, 8, 4)
    assert all(s.table == scheds[0].table for s in scheds)
    assert sum(map(sum, scheds[0].table)) == 30
    # simulate the all-to-all in one process and check every element lands where the plan says
    full = [torch.arange(20.).view(10, 2), 100 + torch.arange(10.).view(10, 1)]
    sends = []
    for r, (lo, hi) in enumerate(rows):
        buf = torch.zeros(scheds[r].send_numel)
        pack(buf, [t[lo:hi] for t in full], scheds[r].send_spans)
        sends.append(buf)
    for d in range(W):
        recv = torch.cat([sends[s][sum(scheds[s].send_splits[:d]):sum(scheds[s].send_splits[:d + 1])] for s in range(W)])
        assert recv.numel() == scheds[d].recv_numel
        outs = [torch.full(p.compute[d].tensor_shape, -1.0) for p in plans]
        unpack(recv, outs, scheds[d].recv_spans)
        if d == 1:
            assert torch.equal(outs[0], full[0])
        if d == 2:
            assert torch.equal(outs[1], full[1][0:5])
        if d == 0:
            assert torch.equal(outs[1], full[1][5:10])
    # the way back is the transposed traffic matrix
    back = packed_schedule(plans, 0, False)
    assert back.table == tuple(tuple(scheds[0].table[s][d] for s in range(W)) for d in range(W))


def test_plan_digest_is_stable_and_sensitive():
    from flex_shard_b200.dist_muon.reshard_plan import plan_digest, plan_rows

    a = plan_rows((8, 2), [(0, 4), (4, 8)], [(0, 8, 0)])
    b = plan_rows((8, 2), [(0, 4), (4, 8)], [(0, 8, 0)])
    c = plan_rows((8, 2), [(0, 4), (4, 8)], [(0, 8, 1)])
    assert plan_digest([a], ["w"]) == plan_digest([b], ["w"]) < 2 ** 56
    assert plan_digest([a], ["w"]) != plan_digest([c], ["w"])
    assert plan_digest([a], ["w"]) != plan_digest([a], ["v"])


def _digest_mismatch(rank, world):
    from flex_shard_b200.dist_muon.reshard_plan import check_plans_across_ranks

    check_plans_across_ranks(1234)            # agreement passes
    try:
        check_plans_across_ranks(1234 + (rank == 1))
        return "passed"
    except RuntimeError as e:
        return str(e)


def test_plan_digest_mismatch_raises_on_every_rank():
    res = run_ranks(_digest_mismatch, 2)
    assert all("differ across ranks" in r for r in res), res


# --------------------------------------------------------------------------- resolution + validator
def test_resolution_and_validator():
    from flex_shard_b200.dist_muon import BlockShard, ComputeLayout, LocalMuonComputeLayout, Owned
    from flex_shard_b200.dist_muon.compute_resolution import contiguous_owners, resolve_compute
    from flex_shard_b200.placements import Shard

    rs = LocalMuonComputeLayout("row_shard", global_shape=(12, 4), row_range=(0, 6))
    r = resolve_compute("w", rs, None)
    assert r.mode == "redistributed" and r.blocks == ((0, 12),) and r.spread == "owned"
    r = resolve_compute("w", rs, ComputeLayout({"dp": BlockShard(0, (4,))}))
    assert r.blocks == ((0, 4), (4, 8), (8, 12)) and r.spread == "contiguous" and r.matrix_shapes() == [(4, 4)] * 3
    r = resolve_compute("w", rs, ComputeLayout({"dp": Owned((2, 4))}))       # q/k-style repeating pattern
    assert r.blocks == ((0, 2), (2, 6), (6, 8), (8, 12)) and r.spread == "owned"
    batch = LocalMuonComputeLayout("row_shard", global_shape=(6, 3, 5), row_range=(0, 3))
    r = resolve_compute("experts", batch, ComputeLayout({"dp": Shard(0)}))
    assert r.batch and len(r.blocks) == 6 and r.spread == "contiguous" and r.matrix_shape == (3, 5)
    assert contiguous_owners(6, 4) == [0, 0, 1, 1, 2, 2] and contiguous_owners(3, 4) == [0, 1, 2]
    # storage that already holds whole matrices stays local
    own = LocalMuonComputeLayout("owned", global_shape=(12, 4))
    assert resolve_compute("w", own, None).mode == "local"
    assert resolve_compute("w", own, ComputeLayout({"dp": Owned()})).mode == "local"
    with pytest.raises(ValueError, match="at most one mesh axis"):
        resolve_compute("w", rs, ComputeLayout({"dp": Owned(), "tp": BlockShard(0, (4,))}))
    with pytest.raises(ValueError, match="whole repetitions"):
        resolve_compute("w", rs, ComputeLayout({"dp": BlockShard(0, (5,))}))
    with pytest.raises(ValueError, match="dim 0"):
        resolve_compute("w", rs, ComputeLayout({"dp": BlockShard(1, (4,))}))
    with pytest.raises(ValueError, match="2-D"):
        resolve_compute("experts", batch, ComputeLayout({"dp": BlockShard(0, (1,))}))
    with pytest.raises(ValueError, match="block storage"):
        resolve_compute("w", own, ComputeLayout({"dp": BlockShard(0, (4,))}))
    with pytest.raises(ValueError, match="matrices or"):
        resolve_compute("v", LocalMuonComputeLayout("owned", global_shape=(12,)), None)
    with pytest.raises(ValueError, match="without a sharding"):
        resolve_compute("w", rs, ComputeLayout({"dp": Owned()}, shard_order_by_tensor_dim={0: ("ep", "dp")}))


def test_constructor_rejects_bad_configs():
    from flex_shard_b200.dist_muon import BucketConfig, ComputeLayout, DistMuon, Owned

    w = torch.nn.Parameter(torch.randn(8, 4))
    with pytest.raises(ValueError, match="does not hold"):
        DistMuon([w], param_names=["w"], compute_sharding_by_fqn={"nope": ComputeLayout({"dp": Owned()})})
    with pytest.raises(ValueError, match="one parameter group"):
        DistMuon([{"params": [w]}, {"params": []}])
    opt = DistMuon([w], param_names=["w"], bucket_configs=[BucketConfig(("a*",)), BucketConfig(("b*",))])
    w.grad = torch.zeros_like(w)
    with pytest.raises(ValueError, match="must match one bucket"):
        opt.step()
    with pytest.raises(RuntimeError, match="frozen"):
        opt.add_param_group({"params": [torch.nn.Parameter(torch.randn(2, 2))]})


# --------------------------------------------------------------------------- pipelined runtime on gloo ranks
def _ns_reference(u, steps, coeffs, eps):
    from flex_shard_b200.ops.newton_schulz import newton_schulz

    return newton_schulz(u, steps, coeffs, eps)


def _pipeline(rank, world):
    """Three buckets of Shard(0)-stored matrices (one with heads, one native batch) plus a local one:
    parameters after two steps equal the whole-tensor update bit for bit, the transfer order is the
    rolling A/B/C pattern, and owners are balanced with loads carried across buckets."""
    from flex_shard_b200.dist_muon import (BlockShard, BucketConfig, ComputeLayout, DistMuon, LocalMuonComputeLayout,
                                           Owned)
    from flex_shard_b200.ops.newton_schulz import NS_COEFFS, muon_apply_, newton_schulz
    from flex_shard_b200.placements import Shard

    torch.manual_seed(0)
    shapes = {"a.w": (10, 6), "a.heads": (12, 6), "b.w": (9, 8), "c.experts": (5, 4, 6), "d.local": (6, 4)}
    full = {n: torch.randn(s) for n, s in shapes.items()}
    grads = [{n: torch.randn(s, generator=torch.Generator().manual_seed(7 * t + i)) for i, (n, s) in enumerate(shapes.items())}
             for t in range(2)]
    sh = Shard(0)

    def local_of(n, t):
        if n == "d.local":
            return t.clone()
        lo, hi = sh._range(t.shape[0], rank, world)
        return t[lo:hi].clone()

    params = {n: torch.nn.Parameter(local_of(n, t)) for n, t in full.items()}
    lays = {n: LocalMuonComputeLayout("row_shard", global_shape=shapes[n], row_range=sh._range(shapes[n][0], rank, world))
            for n in shapes if n != "d.local"}
    lays["d.local"] = LocalMuonComputeLayout("owned", global_shape=shapes["d.local"])
    opt = DistMuon(list(params.values()), param_names=list(params), compute_layouts=lays, lr=0.05, weight_decay=0.1,
                   compute_sharding_by_fqn={"a.heads": ComputeLayout({"dp": BlockShard(0, (4,))}),
                                            "c.experts": ComputeLayout({"dp": Owned()})},
                   bucket_configs=[BucketConfig(("a.*",), "a"), BucketConfig(("d.*",), "d"), BucketConfig(("b.*",), "b"),
                                   BucketConfig(("c.*",), "c")], ranks_per_host=1)
    opt.bucket_plans  # plan now
    opt._runtime.record_trace = True
    for t in range(2):
        for n, p in params.items():
            p.grad = local_of(n, grads[t][n])
        opt.step()
    trace = list(opt._runtime.trace)
    # whole-tensor reference (every matrix orthogonalised from its full bf16 direction)
    ref = {n: t.clone() for n, t in full.items()}
    mom = {n: torch.zeros_like(t) for n, t in full.items()}
    for t in range(2):
        for n in shapes:
            g = grads[t][n]
            mom[n].lerp_(g, 1 - 0.95)
            u = g.lerp(mom[n], 0.95).to(torch.bfloat16)
            if n == "a.heads":
                x = torch.cat([newton_schulz(u[i:i + 4], 5, NS_COEFFS, 1e-7) for i in range(0, 12, 4)])
            elif n == "c.experts":
                x = torch.stack([newton_schulz(u[i], 5, NS_COEFFS, 1e-7) for i in range(5)])
            else:
                x = newton_schulz(u, 5, NS_COEFFS, 1e-7)
            muon_apply_(ref[n], x, 0.05, 0.1, 1.0)
    equal = {n: bool(torch.equal(params[n].detach(), local_of(n, ref[n]))) for n in shapes}
    return {"equal": equal, "trace": trace, "owners": dict(opt.owners), "collectives": opt.collectives_issued,
            "exchanges": opt._runtime.exchanges}


@pytest.mark.parametrize("world", [2, 3])
def test_pipelined_redistribution_matches_whole_tensor_update(world):
    res = run_ranks(_pipeline, world)
    for r in res:
        assert all(r["equal"].values()), r["equal"]
        # buckets a, (d is local), b, c: prefetch of the next exchange before each Newton-Schulz
        assert r["trace"][:10] == ["A0", "A2", "B0", "C0", "L1", "A3", "B2", "C2", "B3", "C3"], r["trace"]
        assert r["collectives"] == 2 * 3 * 2 and r["exchanges"] == 12
    assert all(r["owners"] == res[0]["owners"] for r in res)
    own = res[0]["owners"]
    assert own["a.heads"] == tuple(min(b // -(-3 // world), world - 1) for b in range(3))   # contiguous runs
    # the balancer spreads the whole matrices and the experts over different ranks (loads carried across buckets)
    assert len({own["a.w"][0], own["b.w"][0]} | set(own["c.experts"])) == world


def _state_roundtrip(rank, world):
    from flex_shard_b200.dist_muon import DistMuon, LocalMuonComputeLayout
    from flex_shard_b200.placements import Shard

    sh = Shard(0)
    torch.manual_seed(1)
    w = torch.randn(8, 6)
    lo, hi = sh._range(8, rank, world)

    def make(ns_steps):
        p = torch.nn.Parameter(w[lo:hi].clone())
        lay = {"w": LocalMuonComputeLayout("row_shard", global_shape=(8, 6), row_range=(lo, hi))}
        return p, DistMuon([p], param_names=["w"], compute_layouts=lay, lr=0.05, ns_steps=ns_steps)

    p1, o1 = make(5)
    g = [torch.randn(8, 6, generator=torch.Generator().manual_seed(s)) for s in range(3)]
    for s in range(2):
        p1.grad = g[s][lo:hi].clone()
        o1.step()
    import copy

    sd = copy.deepcopy(o1.state_dict())   # load_state_dict may alias tensors of the dict it is given
    p2, o2 = make(3)                      # built with other hyper-parameters: the loaded group overrides them
    p2.data.copy_(p1.data)
    o2.load_state_dict(sd)
    assert o2._buckets is None and o2.param_groups[0]["ns_steps"] == 5
    p1.grad = g[2][lo:hi].clone()
    p2.grad = g[2][lo:hi].clone()
    o1.step()
    o2.step()
    return bool(torch.equal(p1.detach(), p2.detach())) and o2.state[p2]["momentum_buffer"].dtype == torch.float32


def test_state_dict_reload_replans_and_continues():
    assert all(run_ranks(_state_roundtrip, 2))


def test_runtime_buffers_are_reserved_once_for_the_largest_bucket():
    from flex_shard_b200.dist_muon.reshard_plan import packed_schedule, plan_rows
    from flex_shard_b200.dist_muon.reshard_runtime import LocalBucket, RedistributedBucket, RedistributionRuntime

    def bucket(rows, cols):
        plan = plan_rows((rows, cols), [(0, rows)], [(0, rows, 0)])
        return RedistributedBucket(("x",), (plan,), packed_schedule([plan], 0, True), packed_schedule([plan], 0, False))

    rt = RedistributionRuntime(torch.device("cpu"))
    rt.reserve([bucket(4, 4), LocalBucket(()), bucket(8, 4)])
    assert all(s.send.numel() == 32 and s.back_recv.numel() == 32 and s.send.dtype == torch.bfloat16 for s in rt.slots)
    ptrs = [s.send.data_ptr() for s in rt.slots]
    rt.reserve([bucket(2, 2)])
    assert [s.send.data_ptr() for s in rt.slots] == ptrs and len(rt.slots) == 2
    assert math.prod((8, 4)) == rt._reserved[0]


def _identical_layers(rank, world):
    from unittest import mock

    from flex_shard_b200.dist_muon import BlockShard, BucketConfig, ComputeLayout, DistMuon, LocalMuonComputeLayout
    from flex_shard_b200.dist_muon import reshard_plan
    from flex_shard_b200.placements import Shard

    # three layers whose 12 x 4 weight holds three 4-row matrices: the 6-row storage shards cut the middle one, so
    # every layer needs the same redistribution
    names = [f"layers.{i}.weight" for i in range(3)]
    lo, hi = Shard(0)._range(12, rank, world)
    params = [torch.nn.Parameter(torch.randn(hi - lo, 4)) for _ in names]
    lays = {n: LocalMuonComputeLayout("row_shard", global_shape=(12, 4), row_range=(lo, hi)) for n in names}
    with mock.patch.object(reshard_plan, "plan_rows", wraps=reshard_plan.plan_rows) as build:
        opt = DistMuon(params, param_names=names, compute_layouts=lays,
                       compute_sharding_by_fqn={n: ComputeLayout({"dp": BlockShard(0, (4,))}) for n in names},
                       bucket_configs=[BucketConfig((n,)) for n in names])
        buckets = opt.bucket_plans
    return build.call_count, len(buckets), buckets[0].plans[0] is buckets[2].plans[0]


def test_identical_layers_share_one_row_plan():
    """Parity: ``tests/test_optimizer_reshard_schedule.py:23-70`` of the reference."""
    for calls, n_buckets, shared in run_ranks(_identical_layers, 2):
        assert calls == 1 and n_buckets == 3 and shared
