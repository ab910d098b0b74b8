"""One-launch segment copies on the GPU against a ``copy_`` loop (fp32 / bf16, strided, casts, zero-fill,
more runs than one launch takes), and the launch count of placements that pack through them."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(dev):
    torch.manual_seed(0)
    a = torch.randn(300, 257, device=dev)
    b = torch.randn(300, 257, device=dev).bfloat16()
    big = torch.randn(70000, 3, device=dev)                 # 70 000 runs when sliced by column: two launches
    out = {"row": torch.zeros(300 * 257 * 2 + 64, device=dev), "rowb": torch.zeros(300 * 257 + 64, device=dev, dtype=torch.bfloat16),
           "cols": torch.zeros(70000, 2, device=dev), "z": torch.ones(64, 50, device=dev)}
    n = 300 * 257
    ops = [(out["row"][:n].view(300, 257), a),
           (out["row"][n + 3:n + 3 + 300 * 100].view(300, 100), b[:, 57:157]),     # misaligned destination, cast
           (out["rowb"][1:1 + 300 * 200].view(300, 200), a[:, 1:201]),              # cast down, odd offsets
           (out["cols"], big[:, 1:3]),
           (out["z"][:, 10:40], None)]
    return ops, out


def test_one_launch_equals_copy_loop():
    from flex_shard_b200 import ops as fops
    from flex_shard_b200.ops.segments import run_segment_ops

    dev = torch.device("cuda")
    ops, out = _mk(dev)
    ref_ops, ref = _mk(dev)
    for d, s in ref_ops:
        if s is None:
            d.zero_()
        else:
            d.copy_(s)
    before = fops.launch_count()
    launches = run_segment_ops(ops)
    torch.cuda.synchronize()
    fops.check_status()
    assert launches == 2 and fops.launch_count() - before == 2      # 300+300+300+70000+64 runs > 65 535
    for k in out:
        assert torch.equal(out[k], ref[k]), k
    # second call with new tensors of the same geometry reuses the cached decomposition
    ops2, out2 = _mk(dev)
    run_segment_ops(ops2)
    torch.cuda.synchronize()
    for k in out2:
        assert torch.equal(out2[k], ref[k]), k


def test_long_runs_vector_paths_and_tails():
    """Long contiguous runs (the benchmark's gradient copy-in: bf16 -> fp32 of whole weights) go through the
    16-byte paths with four vectors in flight; lengths that are not multiples of the vector width and a
    misaligned run exercise the tails and the scalar fallback."""
    from flex_shard_b200.ops.segments import run_segment_ops

    dev = torch.device("cuda")
    torch.manual_seed(1)
    n = 8 * 1024 * 1024 + 5
    f = torch.randn(n, device=dev)
    h = torch.randn(n, device=dev).bfloat16()
    outs = [torch.zeros(n, device=dev), torch.zeros(n, device=dev, dtype=torch.bfloat16),
            torch.zeros(n, device=dev), torch.zeros(n + 1, device=dev, dtype=torch.bfloat16),
            torch.zeros(n + 1, device=dev)]
    ops = [(outs[0], h), (outs[1], f), (outs[2], f), (outs[3][1:], f), (outs[4][1:], h)]
    run_segment_ops(ops)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], h.float()) and torch.equal(outs[1], f.bfloat16()) and torch.equal(outs[2], f)
    assert torch.equal(outs[3][1:], f.bfloat16()) and torch.equal(outs[4][1:], h.float())
    assert outs[3][0] == 0 and outs[4][0] == 0


def _launch_worker(rank, world, port, out):
    import os

    import torch.distributed as dist
    import torch.nn as nn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard
        from flex_shard_b200 import ops as fops
        from flex_shard_b200.parallel.comm import set_default_backend
        from flex_shard_b200.placements import (make_block_shard_placement_fn, make_bucketed_block_shard_placement_fn,
                                                make_bucketed_owned_full_param_placement_fn, shard_placement_fn)

        set_default_backend("nccl")
        dev = torch.device("cuda", rank)
        res = {}
        fns = {"shard_dim1": shard_placement_fn(1), "block_shard": make_block_shard_placement_fn(),
               "owned": make_bucketed_owned_full_param_placement_fn(),
               "bucketed_block_shard": make_bucketed_block_shard_placement_fn()}
        for n_params in (4, 12):
            for name, fn in fns.items():
                torch.manual_seed(0)
                model = nn.Sequential(*[nn.Linear(64, 64, bias=False) for _ in range(n_params)]).to(dev)
                flex_shard(model, [BucketSpec(["*"], placement_fn=fn,
                                              mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16,
                                                                             reduce_dtype=torch.float32))])
                x = torch.randn(8, 64, device=dev, dtype=torch.bfloat16)
                model(x).float().square().mean().backward()       # warm: caches, persistent buffers
                model.zero_grad()
                torch.cuda.synchronize()
                before = fops.launch_count()
                model(x).float().square().mean().backward()
                torch.cuda.synchronize()
                res[(name, n_params)] = fops.launch_count() - before
        torch.save(res, os.path.join(out, f"l{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_packing_launches_do_not_grow_with_the_number_of_parameters(tmp_path):
    """Copy-in, copy-out and gradient packing of a bucket are one segment launch each, whatever the
    placement and however many parameters the bucket holds (forward gather + backward gather + reduce)."""
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_launch_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    res = torch.load(tmp_path / "l0.pt")
    for name in ("shard_dim1", "block_shard", "owned", "bucketed_block_shard"):
        small, large = res[(name, 4)], res[(name, 12)]
        assert small == large, (name, res)          # independent of the parameter count
        assert large <= 6, (name, res)
