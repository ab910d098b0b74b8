"""Host-side planners and contracts that need no process group: owner-rows transport plan, layout
composition, adapters, reduce-op mapping, API validation errors, LPT balancing."""
import pytest
import torch
import torch.distributed as dist
import torch.nn as nn



def test_transport_plan_writes_every_position_once_and_counts_crossing():
    from flex_shard_b200.placements.owner_rows_transport import choose_transport, plan_chunks

    lens = [1000, 300, 0, 2500]
    plan = plan_chunks(lens, hosts=[0, 0, 1, 1])
    assert plan.chunk % 128 == 0 and plan.chunk * 4 >= sum(lens)
    cover = [0] * (plan.chunk * 4)
    for m in plan.moves:
        for i in range(m.length):
            cover[m.dst * plan.chunk + m.dst_off + i] += 1
    assert sum(cover) == sum(lens) and max(cover) == 1
    # cross-host elements = what host 1 owns beyond its chunk share, here host-1 rows landing on host-0 chunks
    assert plan.cross_host_elems == sum(m.length for m in plan.moves if (m.src < 2) != (m.dst < 2))
    assert all((m.via >= 0) == ((m.src < 2) != (m.dst < 2)) for m in plan.moves)
    assert plan.buffer_elems >= plan.chunk
    assert choose_transport(plan) == "chunks"


def test_transport_threshold(monkeypatch):
    from flex_shard_b200.placements.owner_rows_transport import ChunkPlan, choose_transport

    p = ChunkPlan(chunk=128, cross_host_elems=83, total_elems=100)
    assert choose_transport(p) == "grouped"
    monkeypatch.setenv("FLEX_SHARD_OWNER_ROWS_TRANSPORT", "chunks")
    assert choose_transport(p) == "chunks"
    monkeypatch.setenv("FLEX_SHARD_OWNER_ROWS_TRANSPORT", "auto")
    monkeypatch.setenv("FLEX_SHARD_OWNER_ROWS_MAX_CROSSING", "0.9")
    assert choose_transport(p) == "chunks"


def test_compose_global_layouts_multi_chunk():
    from flex_shard_b200 import GlobalLayout, compose_global_layouts

    outer = GlobalLayout((16, 4), ((8, 0),), ((0, 0),), ((8, 4),))       # EP rank 1 of 2 holds rows 8..16
    inner = GlobalLayout((8, 4), ((2, 0), (6, 0)), ((0, 0), (2, 0)), ((2, 4), (2, 4)))
    c = compose_global_layouts(outer, inner)
    assert c.global_shape == (16, 4)
    assert c.global_offsets == ((10, 0), (14, 0)) and c.local_offsets == ((0, 0), (2, 0))


def test_shard_layout_goldens_uneven_and_empty():
    from flex_shard_b200.placements import BlockShard, BucketedOwned, Shard

    s = Shard(0)
    assert s.compute_local_shape((10, 3), 0, 4) == (3, 3) and s.compute_local_shape((10, 3), 3, 4) == (1, 3)
    assert s.compute_local_shape((2, 3), 3, 4) == (0, 3)
    assert s.global_layout((2, 3), 3, 4).global_offsets == ()
    assert s.local_storage_layout((10, 3), 3, 4).storage_numel == 9      # rank-0-sized slot on every rank
    with pytest.raises(ValueError):
        Shard(1).compute_local_shape((4, 10), 0, 4)
    b = BlockShard((1, 0, 2, 1), 1)
    assert b.compute_local_shape((3, 8), 2, 4) == (3, 4)
    assert b.global_layout((3, 8), 2, 4).global_offsets == ((0, 2),)
    o = BucketedOwned(((1, 0, 6),))
    assert o.compute_local_shape((6, 5), 1, 2) == (6, 5) and o.compute_local_shape((6, 5), 0, 2) == (0, 5)


def test_reduce_plan_mapping():
    from flex_shard_b200 import GradientReduction
    from flex_shard_b200.parallel.comm import plan_reduction

    assert plan_reduction(GradientReduction(dist.ReduceOp.SUM), 8, torch.float32).op == "sum"
    assert plan_reduction(GradientReduction(), 8, torch.float32).op == "avg"
    p = plan_reduction(GradientReduction(dist.ReduceOp.AVG, 3.0), 8, torch.bfloat16)
    assert p.op == "premul_sum" and abs(p.premul - 1 / 3) < 1e-12
    h = plan_reduction(GradientReduction(dist.ReduceOp.AVG, 8.0), 8, torch.float16)
    assert (h.pre_divide, h.post_divide) == (4.0, 2.0)
    h = plan_reduction(GradientReduction(dist.ReduceOp.AVG, 6.0), 4, torch.float16)
    assert (h.pre_divide, h.post_divide) == (4.0, 1.5)
    one = plan_reduction(GradientReduction(), 1, torch.float32)
    assert one.op == "sum" and one.post_divide is None
    with pytest.raises(ValueError):
        GradientReduction(dist.ReduceOp.SUM, 2.0)
    with pytest.raises(ValueError):
        GradientReduction(dist.ReduceOp.AVG, -1.0)


def test_api_validation_errors():
    from flex_shard_b200 import BucketSpec, OffloadPolicy, flex_shard

    def net():
        return nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 2))

    with pytest.raises(ValueError, match="matches no BucketSpec"):
        flex_shard(net(), [BucketSpec(["0.*"])])
    with pytest.raises(ValueError, match="more than one BucketSpec"):
        flex_shard(net(), [BucketSpec(["*"]), BucketSpec(["0.*"])])
    with pytest.raises(ValueError, match="offload_policy"):
        flex_shard(net(), [BucketSpec(["*"], offload_policy=OffloadPolicy())])
    m = net()
    flex_shard(m, [BucketSpec(["*"])])
    with pytest.raises(ValueError, match="already applied"):
        flex_shard(m, [BucketSpec(["*"])])
    outer = nn.Sequential(m)
    with pytest.raises(ValueError, match="already"):
        flex_shard(outer, [BucketSpec(["*"])])
    tied = net()
    tied[2].weight = nn.Parameter(torch.zeros(2, 4))
    shared = nn.Linear(4, 4)
    tied2 = nn.Sequential(shared, shared)
    flex_shard(tied2, [BucketSpec(["*"])])
    assert tied2[0].weight is tied2[1].weight
    mixed = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4).to(torch.bfloat16))
    with pytest.raises(ValueError, match="mixes parameter dtypes"):
        flex_shard(mixed, [BucketSpec(["*"])])


def test_fsdp2_param_order_is_post_order():
    from flex_shard_b200.bucket_storage import fsdp2_param_order

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.own = nn.Parameter(torch.zeros(1))
            self.child = nn.Linear(2, 2)

    m = M()
    names = [n for n, _ in fsdp2_param_order(m, list(m.named_parameters()))]
    assert names == ["child.weight", "child.bias", "own"]


def test_lpt_even_positions_first_and_carry():
    from flex_shard_b200.utils.validation import assign_to_hosts_then_ranks

    hosts = [r // 8 for r in range(64)]
    assert [r // 8 for r in assign_to_hosts_then_ranks([1.0] * 4, hosts)] == [0, 2, 4, 6]
    loads = [0.0] * 8
    a = assign_to_hosts_then_ranks([1.0] * 4, [0] * 8, loads)
    assert a == [0, 2, 4, 6]
    b = assign_to_hosts_then_ranks([1.0] * 4, [0] * 8, loads)
    assert sorted(b) == [1, 3, 5, 7]


def test_adapters():
    from flex_shard_b200.layout_adapters import spmd_layout

    lay = spmd_layout((4, 8), {"tp": ("shard", 0), "ep": ("replicate",)}, {"tp": (1, 2), "ep": (0, 4)})
    assert lay.global_shape == (8, 8) and lay.global_offsets == ((4, 0),)
    lay = spmd_layout((2, 8), {"a": ("shard", 0), "b": ("shard", 0)}, {"a": (1, 2), "b": (0, 2)}, {0: ("a", "b")})
    assert lay.global_shape == (8, 8) and lay.global_offsets == ((4, 0),)


def test_spmd_annotations_on_a_module_become_layouts_and_partial_groups():
    """Parity: ``layout_adapters/spmd_types.py:20-127`` and ``tests/test_flex_shard_spmd_types_layout.py:34`` of the
    reference (annotations come from parameter attributes here)."""
    import pytest
    import torch
    import torch.nn as nn

    from flex_shard_b200 import get_global_layout, get_partial_grad_group
    from flex_shard_b200.layout_adapters import spmd_types_to_global_layout

    m = nn.Module()
    m.w = nn.Parameter(torch.zeros(4, 8))
    m.norm = nn.Parameter(torch.zeros(8))
    m.plain = nn.Parameter(torch.zeros(2))
    m.w.spmd_sharding, m.w.spmd_mesh = {"tp": ("shard", 0), "dp": ("replicate",)}, {"tp": (1, 2), "dp": (0, 4)}
    m.norm.spmd_sharding, m.norm.spmd_mesh = {"tp": ("partial",)}, {"tp": (1, 2)}
    with pytest.raises(ValueError, match="no group was given"):
        spmd_types_to_global_layout(m)
    group = object()
    assert spmd_types_to_global_layout(m, {"tp": group}) is m
    lay = get_global_layout(m.w)
    assert (lay.global_shape, lay.global_offsets, lay.local_sizes) == ((8, 8), ((4, 0),), ((4, 8),))
    assert get_partial_grad_group(m.norm) is group and get_global_layout(m.norm).global_shape == (8,)
    assert get_global_layout(m.plain) is None and get_partial_grad_group(m.w) is None


def test_router_reference_gradients_match_autograd_of_the_plain_formula():
    import torch
    from flex_shard_b200.ops import moe

    torch.manual_seed(0)
    T, E, k = 37, 16, 4
    for mode, normalize in (("sigmoid", True), ("softmax", True), ("softmax", False)):
        lg = torch.randn(T, E, dtype=torch.float64).float().requires_grad_()
        bias = torch.randn(E) * 0.1
        counts = torch.zeros(E)
        idx, w = moe.route_topk(lg, k, bias=bias, mode=mode, scale=1.7, normalize=normalize, counts=counts)
        g = torch.randn(T, k)
        (w * g).sum().backward()
        lg2 = lg.detach().clone().requires_grad_()
        s = torch.sigmoid(lg2) if mode == "sigmoid" else torch.softmax(lg2, -1)
        _, idx2 = (s + bias).topk(k, dim=-1)
        sel = s.gather(1, idx2)
        w2 = sel / (sel.sum(-1, keepdim=True) + 1e-20) * 1.7 if normalize else sel * 1.7
        (w2 * g).sum().backward()
        assert torch.equal(idx, idx2)
        torch.testing.assert_close(w, w2)
        torch.testing.assert_close(lg.grad, lg2.grad, rtol=1e-5, atol=1e-7)
        assert counts.sum().item() == T * k


def test_yarn_table_and_fp32_output_linear():
    import torch

    from flex_shard_b200.ops.elementwise import rope_table, yarn_attention_scale
    from flex_shard_b200.ops.gemm import fp32_output_linear, split_into_bf16_pieces

    # no stretch -> the plain table; stretch -> low-frequency pairs slowed by `factor`, fast pairs untouched
    plain = rope_table(64, 64, 10000.0, "cpu")
    assert torch.equal(plain, rope_table(64, 64, 10000.0, "cpu", yarn=dict(factor=1.0, original_seq_len=4096)))
    st = rope_table(64, 64, 10000.0, "cpu", yarn=dict(factor=40.0, original_seq_len=4096))
    assert torch.equal(st[:, 0], plain[:, 0])                       # fastest pair: unchanged
    slow_plain = torch.atan2(plain[1, -1, 1], plain[1, -1, 0])
    slow_st = torch.atan2(st[1, -1, 1], st[1, -1, 0])
    assert abs(slow_st.item() * 40.0 - slow_plain.item()) < 1e-6     # slowest pair: angle / factor
    assert abs(yarn_attention_scale(192, 1.0) - 192 ** -0.5) < 1e-12
    assert yarn_attention_scale(192, 40.0) > 192 ** -0.5
    # three bf16 pieces reproduce an fp32 tensor far below bf16 resolution
    t = torch.randn(1000) * 3
    hi, mid, lo = split_into_bf16_pieces(t)
    assert (hi.float() + mid.float() + lo.float() - t).abs().max() < 1e-6 * t.abs().max()
    # logits in fp32 from bf16 operands, gradients close to the fp32 product's
    x = torch.randn(40, 64).bfloat16().requires_grad_()
    w = (torch.randn(8, 64) * 0.1).bfloat16().requires_grad_()
    y = fp32_output_linear(x, w)
    assert y.dtype == torch.float32
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    (xr @ wr.t()).backward(g)
    torch.testing.assert_close(y, xr @ wr.t(), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=1e-1)


def test_bucket_debug_names():
    from flex_shard_b200.utils.profiling import bucket_debug_fqn, strip_wrapper_path

    assert bucket_debug_fqn(["layers.0.attn.wq.weight", "layers.0.mlp.w1.weight"]) == "layers.0"
    assert bucket_debug_fqn(["layers.0._checkpoint_wrapped_module.attn.w", "layers.0._checkpoint_wrapped_module.mlp.w"]) == "layers.0"
    assert bucket_debug_fqn(["norm.weight", "lm_head.weight"]) == "lm_head, norm"
    assert bucket_debug_fqn(["layers.1.a.w", "layers.2.a.w"]) == "layers"
    assert bucket_debug_fqn([]) is None
    assert strip_wrapper_path("a._orig_mod.b") == "a.b"


def test_failed_wait_record_names_region_slot_epoch_and_peer():
    """The device status record of a failed peer wait (code, flag address, epoch, peer, value seen) is turned into
    a message that names the registered symmetric region and the flag slot."""
    from flex_shard_b200.ops import _lib

    base = 0x7F0012340000
    _lib.register_flag_range(base, 65536, lambda: "gradient ring (3 entries)", 64)
    addr = base + 17 * 64 + 4 * 3          # slot 17, the word of group rank 3
    rec = [32, addr & 0xFFFFFFFF, addr >> 32, 41, 3, 40, 0, 0]
    msg = _lib._describe([v - (1 << 32) if v >= (1 << 31) else v for v in rec])     # as int32 values
    assert "gradient ring (3 entries)" in msg and "flag slot 17" in msg
    assert "epoch 41" in msg and "group rank 3" in msg and "last value seen 40" in msg
    other = _lib._describe([18, 0, 0, 0, 0, 0, 0, 0])
    assert "code 18" in other and "flag" not in other
