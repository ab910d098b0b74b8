"""All-gather -> GEMM fused kernel. On one GPU the "peers" are W slices of a local tensor (the
stager CTAs copy through the same bulk-copy ring, only the link differs); the 2-GPU variant pulls
real peer shards out of a symmetric region."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,N,K,M", [(1, 512, 1024, 256), (4, 2048, 1024, 384), (8, 6144, 4096, 1024)])
def test_allgather_gemm_single_gpu_emulated_peers(world, N, K, M):
    from flex_shard_b200 import ops
    from flex_shard_b200.ops.fused import AllGatherLinear

    torch.manual_seed(0)
    dev = torch.device("cuda")
    w = (0.05 * torch.randn(N, K, device=dev)).bfloat16()
    c = N // world
    shards = [w[r * c:(r + 1) * c].clone() for r in range(world)]
    lin = AllGatherLinear([s.data_ptr() for s in shards], N, K, c, dev, n_stagers=8)
    x = torch.randn(M, K, device=dev).bfloat16()
    for _ in range(2):  # second call exercises the monotonic counters
        y = lin(x)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(lin.gathered, w)
        torch.testing.assert_close(y.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-2 * K ** 0.5 * 0.05)


def _worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import ops
        from flex_shard_b200.ops.fused import AllGatherLinear
        from flex_shard_b200.parallel.symm import SymmRegion

        dev = torch.device("cuda", rank)
        N, K, M = 4096, 2048, 1024
        c = N // world
        torch.manual_seed(7)
        w = (0.05 * torch.randn(N, K, device=dev)).bfloat16()  # same on every rank
        reg = SymmRegion(dist.group.WORLD, c * K * 2, dev)
        reg.payload[: c * K * 2].view(torch.bfloat16).view(c, K).copy_(w[rank * c:(rank + 1) * c])
        reg.signal(5, 1)  # "my shard is valid from epoch 1"
        lin = AllGatherLinear([reg.peer_payload_addr(r) for r in range(world)], N, K, c, dev, n_stagers=8,
                              flag_row_addr=reg.flag_row_addr(rank, 5))
        x = torch.randn(M, K, device=dev).bfloat16()
        y = lin(x, epoch=1)
        torch.cuda.synchronize()
        ops.check_status()
        ok_gather = bool(torch.equal(lin.gathered, w))
        err = float((y.float() - x.float() @ w.float().t()).abs().max())
        dist.barrier()
        torch.save({"gather": ok_gather, "err": err}, os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_allgather_gemm_two_gpus(tmp_path):
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"r{r}.pt")
        assert res["gather"] is True
        assert res["err"] < 0.5


def test_adamw_overlapped_with_backward_on_one_rank_matches_plain_step():
    """On a 1-rank mesh ``fuse_into_backward`` runs each bucket's AdamW on a side stream as soon as the
    bucket's gradients are final; the losses must be bit-identical to stepping after backward."""
    from flex_shard_b200 import flex_shard, ops
    from flex_shard_b200.models.llama import Llama, LlamaConfig, llama_buckets
    from flex_shard_b200.optim.adamw import FusedAdamW

    dev = torch.device("cuda")
    cfg = LlamaConfig(vocab_size=2048, d_model=256, n_layers=3, n_heads=2, n_kv_heads=1, ffn_hidden=512, max_seq_len=256)
    losses = {}
    for mode in ("plain", "in_backward"):
        torch.manual_seed(0)
        model = Llama(cfg, dtype=torch.bfloat16, device=dev)
        model.init_weights(0)
        for p in model.parameters():
            p.grad_dtype = torch.float32
        flex_shard(model, llama_buckets(model, mesh=None))
        opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
        if mode == "in_backward":
            opt.fuse_into_backward(model)
        out = []
        for s in range(5):
            tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=torch.Generator().manual_seed(s)).to(dev)
            loss = model.loss(tok[:, :-1], tok[:, 1:])
            loss.backward()
            if mode == "in_backward" and s == 1:
                assert len(opt._stepped_in_backward) > 0   # buckets were updated before step() was called
            opt.step()
            opt.zero_grad(set_to_none=True)
            out.append(float(loss.detach()))
        torch.cuda.synchronize()
        ops.check_status()
        losses[mode] = out
    assert losses["plain"] == losses["in_backward"], losses
