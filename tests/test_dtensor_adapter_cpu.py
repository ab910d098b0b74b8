"""``dtensor_to_global_layout`` on real DTensors (4 gloo ranks as tp x dp = 2 x 2): the local tensors declare where they
sit in the full parameter, an explicit gradient dtype and tied names survive, ``flex_shard`` over the dp axis composes
its own split with the declared one, and placements other than ``Shard`` / ``Replicate`` are refused.
Parity: ``layout_adapters/dtensor.py:24-64`` and ``tests/test_flex_shard_outer_layout.py:41-141`` of the reference."""
import pytest
import torch
import torch.nn as nn

from tests.common import run_ranks


def _adapter(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Partial, Replicate, Shard, distribute_tensor

    from flex_shard_b200 import BucketSpec, flex_shard, get_global_layout
    from flex_shard_b200.checkpoint import get_flex_shard_global_layouts
    from flex_shard_b200.layout_adapters import dtensor_to_global_layout

    grid = init_device_mesh("cpu", (2, 2), mesh_dim_names=("tp", "dp"))
    tp, dp = grid["tp"], grid["dp"]
    t = tp.get_local_rank()
    torch.manual_seed(0)
    full_w, full_v, full_e = torch.randn(8, 6), torch.randn(5, 4), torch.randn(1, 6)

    m = nn.Module()
    m.col = nn.Linear(6, 8, bias=False)
    m.row = nn.Linear(4, 5, bias=False)
    m.tied = nn.Linear(6, 8, bias=False)
    m.one = nn.Linear(6, 1, bias=False)
    m.plain = nn.Linear(3, 3)
    m.col.weight = nn.Parameter(distribute_tensor(full_w, tp, [Shard(0)]))
    m.col.weight.grad_dtype = torch.float64
    m.row.weight = nn.Parameter(distribute_tensor(full_v, tp, [Shard(1)]))
    m.tied.weight = m.col.weight
    m.one.weight = nn.Parameter(distribute_tensor(full_e, tp, [Shard(0)]))      # rank 1 of tp holds no row
    dtensor_to_global_layout(m)
    out = {"plain": not any(isinstance(p, DTensor) for p in m.parameters()),
           "tied": m.tied.weight is m.col.weight,
           "grad_dtype": str(getattr(m.col.weight, "grad_dtype", None)),
           "untouched": get_global_layout(m.plain.weight) is None}
    lw, lv, le = (get_global_layout(p) for p in (m.col.weight, m.row.weight, m.one.weight))
    out["col"] = (lw.global_shape, lw.global_offsets, lw.local_sizes) == ((8, 6), ((4 * t, 0),), ((4, 6),))
    out["row"] = (lv.global_shape, lv.global_offsets, lv.local_sizes) == ((5, 4), ((0, 2 * t),), ((5, 2),))
    out["empty"] = (le.global_shape == (1, 6)) and ((le.global_offsets == ()) if t == 1 else (le.local_sizes == ((1, 6),)))
    out["values"] = bool(torch.equal(m.col.weight.detach(), full_w[4 * t:4 * t + 4]))

    # flex_shard over the dp axis: the checkpoint layout is the dp split inside the tp shard
    del m.one
    flex_shard(m, [BucketSpec(["*"], mesh=dp)])
    d = dp.get_local_rank()
    lay = get_flex_shard_global_layouts(m)["col.weight"]
    out["composed"] = (lay.global_shape, lay.global_offsets, lay.local_sizes) == ((8, 6), ((4 * t + 2 * d, 0),), ((2, 6),))
    out["local"] = bool(torch.equal(m.col.weight.detach(), full_w[4 * t + 2 * d:4 * t + 2 * d + 2]))

    bad = nn.Module()
    bad.w = nn.Parameter(DTensor.from_local(torch.zeros(2, 2), tp, [Partial()]), requires_grad=False)
    try:
        dtensor_to_global_layout(bad)
        out["partial_refused"] = False
    except NotImplementedError as e:
        out["partial_refused"] = "Shard and Replicate only" in str(e)
    rep = nn.Module()
    rep.w = nn.Parameter(distribute_tensor(full_v, tp, [Replicate()]))
    dtensor_to_global_layout(rep)
    lr = get_global_layout(rep.w)
    out["replicated"] = (lr.global_offsets, lr.local_sizes) == (((0, 0),), ((5, 4),))
    return out


def test_dtensor_parameters_become_local_tensors_with_declared_layouts():
    for out in run_ranks(_adapter, 4):
        assert all(v is True for k, v in out.items() if k != "grad_dtype"), out
        assert out["grad_dtype"] == "torch.float64"
