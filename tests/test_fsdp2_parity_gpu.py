"""``Shard`` buckets (NCCL collectives) against PyTorch FSDP2 ``fully_shard`` on 2 and 4 GPUs, bit for
bit: the 24-configuration matrix with recorded collective inputs, and the head variants (values).
Skipped with fewer GPUs.  The same comparison runs on gloo ranks in ``test_fsdp2_parity_cpu.py``."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out, variant, only):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from torch.distributed.device_mesh import init_device_mesh

        from flex_shard_b200.parallel.comm import set_default_backend
        from tests import fsdp2_parity_common as pc

        set_default_backend("nccl")   # the bitwise-FSDP2 contract is defined on the library collectives
        mesh = init_device_mesh("cuda", (world,))
        cfgs = pc.configs()
        if only is not None:
            cfgs = [cfgs[i] for i in only]
        bad = []
        for cfg in cfgs:
            bad += pc.run_pair(torch.device("cuda", rank), mesh, rank, cfg, steps=2, variant=variant,
                               record=variant == "plain")
        torch.cuda.synchronize()
        dist.barrier()
        torch.save(bad, os.path.join(out, f"p{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(world, tmp_path, variant, only):
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_worker, args=(world, free_port(), str(tmp_path), variant, only), nprocs=world, join=True)
    bad = [m for r in range(world) for m in torch.load(tmp_path / f"p{r}.pt")]
    assert not bad, "\n".join(bad[:40])


@pytest.mark.parametrize("world", [2, 4])
def test_matrix_bitwise_equal_to_fsdp2_nccl(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run(world, tmp_path, "plain", None)


@pytest.mark.parametrize("variant", ["chunked", "head_twice"])
def test_head_variants_equal_to_fsdp2_nccl(variant, tmp_path):
    world = 4 if torch.cuda.device_count() >= 4 else 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    from tests.test_fsdp2_parity_cpu import _VARIANTS

    _run(world, tmp_path, variant, _VARIANTS[variant])
