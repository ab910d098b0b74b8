"""Layout and scheduling facts of the reference restated as tests (no process group where a fake mesh is
enough): the 25-element uneven ``Shard(0)`` bucket whose byte storage is the all-gather send buffer, the
14-element mixed row, explicit prefetch lists (8 gathers per step, 12 prefetch hits over 2 steps),
gradient-accumulation collective counts, finalisation order, hook call order, and the dtype in which kept
gradients accumulate (256 + 1 = 257 only in fp32).
Sources: ``src/flex_shard/tests/test_flex_shard_training.py:622-657,1535-1637,1834-2025,2339-2436``,
``test_flex_shard_buckets.py:887-1013``, ``test_flex_shard_runtime.py:617-695`` of the reference."""
import torch
import torch.nn as nn

from tests.common import FakeMesh, run_ranks


class UnevenMLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.out_activation = nn.PReLU()          # 1 element: rank 1 holds nothing of it
        self.in_proj = nn.Linear(3, 5)            # 5 rows over 2 ranks: 3 + 2
        self.out_proj = nn.Linear(5, 3)           # 3 rows: 2 + 1

    def forward(self, x):
        return self.out_activation(self.out_proj(torch.relu(self.in_proj(x))))


def test_uneven_shard_bucket_reserves_rank0_sized_slots_and_aliases_the_send_buffer():
    from flex_shard_b200 import BucketSpec, flex_shard
    from flex_shard_b200.parallel.comm import Comm

    for rank in (0, 1):
        m = nn.Sequential(UnevenMLP(), UnevenMLP())
        flex_shard(m, [BucketSpec(["0"], mesh=FakeMesh(2, rank)), BucketSpec(["1"], mesh=FakeMesh(2, rank))])
        st = m.sharded_bucket_storages[0]
        assert {i.fqn: i.storage_nbytes // 4 for i in st.infos} == {
            "0.out_activation.weight": 1, "0.in_proj.weight": 9, "0.in_proj.bias": 3, "0.out_proj.weight": 10,
            "0.out_proj.bias": 2}
        assert st.total_bytes == 25 * 4                        # on both ranks
        assert sum(i.local_numel for i in st.infos) == (25 if rank == 0 else 14)
        assert st.infos[0].local_numel == (1 if rank == 0 else 0)
        comm = Comm(None, rank, 2, torch.device("cpu"))
        prep = st.placement.prepare_unshard_bucket(st.infos, st.byte_storage, comm, None)
        assert prep.send.numel() == 25 * 4
        assert prep.send.untyped_storage().data_ptr() == st.byte_storage.untyped_storage().data_ptr()
        # padding is deterministic zeros
        tail = st.byte_storage.view(torch.float32)
        if rank == 1:
            assert float(tail[0]) == 0.0                        # the empty slot of the 1-element weight


def test_mixed_bucket_row_is_owner_region_plus_regular_slots():
    from flex_shard_b200.placements import BlockShard, BucketedOwned, MixedBucketPlacement, Shard
    from flex_shard_b200.placements.sliced import plan_rows

    class Info:
        def __init__(self, shape, pl):
            self.global_shape, self.placement = shape, pl
            self.param_dtype = torch.float32

    infos = [Info((2, 3), MixedBucketPlacement(BucketedOwned(((0, 0, 2),)))),      # head, owned by rank 0
             Info((3, 2), MixedBucketPlacement(BlockShard((1, 0), 1))),            # wo, one dim-1 block on rank 0
             Info((3,), MixedBucketPlacement(Shard(0))),                           # norm
             Info((2, 2), MixedBucketPlacement(BucketedOwned(((1, 0, 2),))))]      # dense, owned by rank 1
    plan = plan_rows(infos, 2, lambda i: 1, align=1)
    assert plan.row == 14                       # the reference's golden: 6 + 6 on rank 0 (4 on rank 1), then the norm's slot of 2
    assert plan.offsets[0][0] == 0 and plan.offsets[3][1] == 0      # owners start their rows with their parameters
    assert plan.offsets[2][0] == plan.offsets[2][1] > 0             # the Shard group sits after the owner region
    assert not plan.owner_only
    aligned = plan_rows(infos, 2, lambda i: 1)  # default: every slot starts on a 4-element (16-byte fp32) boundary
    assert aligned.row == 20 and all(o % 4 == 0 for row in aligned.offsets for o in row if o is not None)


class FourBlocks(nn.Sequential):
    def __init__(self):
        super().__init__(*[nn.Linear(8, 8) for _ in range(4)])


def _explicit_prefetch(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = FourBlocks()
    flex_shard(m, [BucketSpec([str(i)]) for i in range(4)])
    sts = m.sharded_bucket_storages
    for i, st in enumerate(sts):                   # each bucket prefetches its successor (forward) / predecessor (backward)
        st.set_buckets_to_forward_prefetch([sts[i + 1]] if i + 1 < 4 else [])
        st.set_buckets_to_backward_prefetch([sts[i - 1]] if i > 0 else [])
    ctx = sts[0].runtime.context
    x = torch.randn(3, 8)
    per_step = []
    for _ in range(2):
        before = dict(ctx.stats)
        m(x).square().mean().backward()
        per_step.append({k: ctx.stats[k] - before[k] for k in before})
    return per_step, ctx.idle()


def test_explicit_prefetch_lists_hit_from_the_first_step():
    for per_step, idle in run_ranks(_explicit_prefetch, 2):
        assert [s["unshards"] for s in per_step] == [8, 8]           # 4 buckets, forward and backward
        assert sum(s["prefetch_hits"] for s in per_step) == 12       # 3 forward + 3 backward hits per step
        assert idle


def _accumulation_counts(rank, world):
    """``reshard_after_backward`` kept False while accumulating: one gather serves all microbatches."""
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = FourBlocks()
    flex_shard(m, [BucketSpec([str(i)]) for i in range(4)])
    ctx = m._fsb_ctx()
    x = torch.randn(3, 8)
    out = {}
    for mode in ("per_microbatch", "keep"):
        before = dict(ctx.stats)
        for mb in range(3):
            last = mb == 2
            m.set_requires_gradient_sync(last)
            if mode == "keep":
                for st in m.sharded_bucket_storages:
                    st.set_reshard_after_backward(last)
                    st.set_reshard_after_forward(False)
            m(x).square().mean().backward()
        out[mode] = {k: ctx.stats[k] - before[k] for k in before}
        for st in m.sharded_bucket_storages:
            st.set_reshard_after_forward(True)
            st.set_reshard_after_backward(True)
        for p in m.parameters():
            p.grad = None
    return out


def test_gradient_accumulation_collective_counts():
    for out in run_ranks(_accumulation_counts, 2):
        # resharding after every pass: 3 microbatches x (forward + backward) gathers per bucket, one reduction each
        assert out["per_microbatch"]["unshards"] == 3 * 2 * 4 and out["per_microbatch"]["reduces"] == 4
        # kept gathered while accumulating: one gather per bucket for the whole step
        assert out["keep"]["unshards"] == 4 and out["keep"]["reduces"] == 4


def _orders(rank, world):
    from flex_shard_b200 import BucketSpec, flex_shard

    torch.manual_seed(0)
    m = FourBlocks()
    calls = []
    # specs listed in an order unrelated to execution; hooks record (kind, bucket)
    specs = [BucketSpec([str(i)], pre_backward_hook=lambda st: calls.append(("pre", st.name)),
                        post_reduce_hook=lambda st: calls.append(("post", st.name))) for i in (2, 0, 3, 1)]
    flex_shard(m, specs)
    x = torch.randn(3, 8)
    m.set_requires_gradient_sync(False)
    m(x).square().mean().backward()
    m(x).square().mean().backward()
    m.set_requires_gradient_sync(True)
    m(x).square().mean().backward()
    hooks = list(calls)
    # manual finalisation: reductions run in reverse module order whatever the spec order
    calls.clear()
    for p in m.parameters():
        p.grad = None
    m.set_manual_backward_finalization(True)
    m(x).square().mean().backward()
    reduced = []
    ctx = m._fsb_ctx()
    for rt in ctx.runtimes:
        orig = rt._reduce_now

        def wrapped(orig=orig, rt=rt):
            reduced.append(rt.storage.name)
            return orig()

        rt._reduce_now = wrapped
    m.finalize_backward()
    return hooks, reduced


def test_hook_and_finalisation_order():
    for hooks, reduced in run_ranks(_orders, 2):
        names = ["3", "2", "1", "0"]
        pre = [("pre", n) for n in names]
        # two backwards without reduction call only the pre-backward hooks; the syncing one interleaves
        # pre (when the bucket's backward starts) and post (after its gradients are taken), last layer first
        assert hooks[:8] == pre + pre
        assert [h for h in hooks[8:] if h[0] == "pre"] == pre
        assert [h for h in hooks[8:] if h[0] == "post"] == [("post", n) for n in names]
        assert hooks[8] == ("pre", "3") and hooks[-1] == ("post", "0")
        assert reduced == names


def _accumulation_dtype(rank, world):
    """One parameter, two backwards without reduction with gradients 256 and 1: the kept gradient is 257 only
    if it accumulates in fp32 (bf16 has 8 bits of mantissa: 256 + 1 = 256)."""
    from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard

    out = {}
    cases = {"fp32_storage_bf16_compute": (torch.float32, MixedPrecisionPolicy(param_dtype=torch.bfloat16), None),
             "explicit_grad_dtype": (torch.bfloat16, MixedPrecisionPolicy(), torch.float32),
             "bf16_reduce": (torch.float32, MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16), None),
             "all_bf16": (torch.bfloat16, MixedPrecisionPolicy(), None)}
    for name, (storage_dtype, mp, grad_dtype) in cases.items():
        lin = nn.Linear(4, 4, bias=False).to(storage_dtype)
        if grad_dtype is not None:
            lin.weight.grad_dtype = grad_dtype
        m = nn.Sequential(lin)
        flex_shard(m, [BucketSpec(["*"], mp_policy=mp, gradient_reduce_op=torch.distributed.ReduceOp.SUM)])
        st = m.sharded_bucket_storages[0]
        m.set_requires_gradient_sync(False)
        for scale in (256.0, 1.0):
            x = torch.ones(1, 4, dtype=st.infos[0].param_dtype)
            (m(x).float().sum() * scale).backward()
        up = st.runtime.unsharded_params[0]
        kept = up.grad
        out[name] = (float(kept.flatten()[0]), str(kept.dtype), str(up.grad_dtype))
        # the syncing backward hands autograd's gradients on unwidened (deferred cast), then restores grad_dtype
        m.set_requires_gradient_sync(True)
        (m(torch.ones(1, 4, dtype=st.infos[0].param_dtype)).float().sum()).backward()
        out[name + "_after_sync"] = (str(up.grad_dtype), float(m[0].weight.grad.flatten()[0]), str(m[0].weight.grad.dtype))
    return out


def test_kept_gradients_accumulate_in_the_wide_dtype():
    for out in run_ranks(_accumulation_dtype, 2):
        assert out["fp32_storage_bf16_compute"][:2] == (257.0, "torch.float32")
        assert out["explicit_grad_dtype"][:2] == (257.0, "torch.float32")
        assert out["bf16_reduce"][:2] == (256.0, "torch.bfloat16")
        assert out["all_bf16"][:2] == (256.0, "torch.bfloat16")
        # summed over 2 ranks: (256 + 1 + 1) * 2 in fp32; the sharded gradient keeps the storage / explicit dtype
        assert out["fp32_storage_bf16_compute_after_sync"] == ("torch.float32", 516.0, "torch.float32")
        assert out["explicit_grad_dtype_after_sync"] == ("torch.float32", 516.0, "torch.float32")
