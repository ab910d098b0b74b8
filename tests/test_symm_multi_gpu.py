"""Peer-memory collectives against NCCL on 2+ GPUs (skipped with fewer): bitwise all-gather,
deterministic rank-order reduce-scatter, and a missing peer signal that must time out cleanly."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    import torch.distributed as dist

    # guard bytes behind every symmetric payload, checked by every ops.check_status() below
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", FSB200_CANARY="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import ops
        from flex_shard_b200.parallel.comm import Comm, plan_reduction
        from flex_shard_b200.parallel.symm import SymmComm
        from flex_shard_b200.placement_contract import GradientReduction

        dev = torch.device("cuda", rank)
        g = dist.group.WORLD
        sc, nc = SymmComm(g, rank, world, dev), Comm(g, rank, world, dev)
        torch.manual_seed(rank)
        res = {}
        for n in (1024, 1 << 20, 3 * (1 << 20) + 16):
            x = torch.randn(n, device=dev).bfloat16()
            a = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
            b = torch.empty_like(a)
            sc.all_gather_into_tensor(a, x)
            nc.all_gather_into_tensor(b, x)
            res[f"ag{n}"] = bool(torch.equal(a, b))
        plan = plan_reduction(GradientReduction(), world, torch.float32)
        for n in (4096, 1 << 20):
            gsend = torch.randn(world * n, device=dev)
            o1 = torch.empty(n, device=dev)
            o2 = torch.empty(n, device=dev)
            o3 = torch.empty(n, device=dev)
            sc.reduce_scatter_tensor(o1, gsend.clone(), plan)
            sc.reduce_scatter_tensor(o3, gsend.clone(), plan)
            nc.reduce_scatter_tensor(o2, gsend.clone(), plan)
            res[f"rs{n}_close"] = float((o1 - o2).abs().max())
            res[f"rs{n}_deterministic"] = bool(torch.equal(o1, o3))
        torch.cuda.synchronize()
        ops.check_status()
        # in-switch reduction: every rank fills row d of its own region with its contribution to rank d;
        # one multimem load per 16 bytes must return the sum over ranks (compared with the rank-order
        # peer-load kernel on the same data), twice with the same bits
        import ctypes

        from flex_shard_b200.ops import _lib
        from flex_shard_b200.parallel.symm import SymmRegion

        n = 1 << 18
        mreg = SymmRegion(g, world * n * 4, dev)
        res["multicast_mapped"] = bool(mreg.mc_base)
        rows_local = mreg.payload[: world * n * 4].view(torch.float32).view(world, n)
        rows_local.copy_(torch.randn(world, n, generator=torch.Generator().manual_seed(7 + rank)).to(dev))
        mreg.signal(5, 1)
        mreg.wait(5, 1)
        ref = torch.empty(n, device=dev)
        rows = (ctypes.c_ulonglong * world)(*[mreg.peer_payload_addr(r, rank * n * 4) for r in range(world)])
        st_ptr, stream = _lib.status_word(dev).data_ptr(), _lib.stream_ptr(dev)
        _lib.check(_lib.load().fsb_comm_reduce_rows(rows, world, n, 0.5, ref.data_ptr(), None, 0, None, None,
                                                    0.0, 0.0, 0.0, 0.0, 0.0, 1, None, 0, 1000, st_ptr, stream), "reduce")
        if mreg.mc_base:
            outs = []
            for _ in range(2):
                o = torch.empty(n, device=dev)
                _lib.check(_lib.load().fsb_comm_reduce_rows_mc(mreg.mc_payload_addr(rank * n * 4), world, n, 0.5,
                                                               o.data_ptr(), None, 0, None, None, 0.0, 0.0, 0.0, 0.0, 0.0,
                                                               1, None, 0, 1000, st_ptr, stream), "reduce_mc")
                outs.append(o)
            res["mc_close"] = float((outs[0] - ref).abs().max())
            res["mc_deterministic"] = bool(torch.equal(outs[0], outs[1]))
            if world == 2:
                res["mc_bitwise_at_two_ranks"] = bool(torch.equal(outs[0], ref))   # a two-term sum has one order
        torch.cuda.synchronize()
        mreg.signal(6, 1)
        mreg.wait(6, 1)      # nobody frees its region while a peer may still read it
        torch.cuda.synchronize()
        ops.check_status()
        # a flag that nothing sets: the wait gives up after its (shortened) limit and reports it
        reg = sc._ag
        reg.max_polls = 2000
        reg.wait(900, 1)
        torch.cuda.synchronize()
        try:
            ops.check_status()
            res["timeout_reported"] = False
        except ops.NativeError as e:
            msg = str(e)
            # the record names the region, the flag slot, the epoch and the peer that never signalled
            res["timeout_reported"] = ("peer" in msg and "flag slot 900" in msg and "epoch 1" in msg
                                       and "all-gather staging region" in msg)
        # after a first failure every later wait returns at once instead of sitting out its own limit
        reg.wait(900, 1)                       # fails again (short limit) and sets the status word
        reg.max_polls = 20_000_000             # several seconds if it were waited out
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        reg.wait(901, 1)
        t1.record()
        torch.cuda.synchronize()
        res["fails_fast_after_first_failure"] = t0.elapsed_time(t1) < 500.0
        try:
            ops.check_status()
        except ops.NativeError:
            pass
        reg.max_polls = 2000
        # the context is still usable afterwards
        res["alive"] = float(torch.ones(4, device=dev).sum()) == 4.0
        # guard bytes: intact after all of the above; a write just past the payload (made here through a view of
        # this rank's own buffer) is reported by the next status check
        from flex_shard_b200.parallel.symm import FLAG_BYTES

        ops.check_status()
        res["canary_armed"] = reg.canary_bytes == 256 and reg.canary_intact()
        reg.buf[FLAG_BYTES + reg.payload_bytes + 3] = 0
        try:
            ops.check_status()
            res["canary_reported"] = False
        except RuntimeError as e:
            res["canary_reported"] = "guard bytes" in str(e) and "all-gather staging region" in str(e)
        reg.buf[FLAG_BYTES + reg.payload_bytes + 3] = 0xA5
        dist.barrier()
        torch.save(res, os.path.join(out, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symm_collectives_match_nccl(tmp_path):
    import torch.multiprocessing as mp

    from tests.common import free_port

    world = 2
    mp.spawn(_worker, args=(world, free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(tmp_path / f"r{r}.pt")
        for k, v in res.items():
            if k.startswith("ag") or k.endswith("deterministic") or k in ("timeout_reported", "alive", "fails_fast_after_first_failure", "canary_armed", "canary_reported",
                                                                         "mc_bitwise_at_two_ranks"):
                assert v is True, (k, v)
            elif k.endswith("_close"):
                assert v < 1e-5, (k, v)


def _train_worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from torch.distributed.device_mesh import init_device_mesh

        from flex_shard_b200 import flex_shard, ops
        from flex_shard_b200.models.llama import Llama, LlamaConfig, llama_buckets
        from flex_shard_b200.optim.adamw import FusedAdamW
        from flex_shard_b200.parallel.comm import set_default_backend

        dev = torch.device("cuda", rank)
        mesh = init_device_mesh("cuda", (world,))
        cfg = LlamaConfig(vocab_size=4096, d_model=512, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=1024,
                          max_seq_len=256)
        results = {}
        for mode in ("nccl", "symm", "symm_fused_adam", "symm_fused_adam_peer_loads", "symm_fused_adam_staged",
                     "symm_fused_adam_sm_gather"):
            # default: buckets resident in symmetric memory and (where mapped) the in-switch reduction;
            # the last two arms switch one of them off each
            os.environ["FSB200_MULTIMEM_REDUCE"] = "0" if mode.endswith("peer_loads") else "1"
            os.environ["FSB200_RESIDENT"] = "0" if mode.endswith("staged") else "1"
            os.environ["FSB200_GATHER"] = "sm" if mode.endswith("sm_gather") else "dma"
            set_default_backend("symm" if mode.startswith("symm") else "nccl")
            torch.manual_seed(0)
            model = Llama(cfg, dtype=torch.bfloat16, device=dev)
            model.init_weights(0)
            for p in model.parameters():
                p.grad_dtype = torch.float32
            flex_shard(model, llama_buckets(model, mesh=mesh))
            opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
            if mode.startswith("symm_fused_adam"):
                opt.fuse_into_backward(model)
            losses = []
            for step in range(4):
                g = torch.Generator().manual_seed(100 * step + rank)
                tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=g).to(dev)
                loss = model.loss(tok[:, :-1], tok[:, 1:])
                loss.backward()
                opt.step()
                opt.zero_grad()
                losses.append(float(loss.detach()))
            torch.cuda.synchronize()
            ops.check_status()
            results[mode] = losses
            if mode.startswith("symm"):
                results[mode + "_stats"] = dict(model.sharded_bucket_storages[1].comm.stats)
                results[mode + "_mc"] = bool(getattr(model.sharded_bucket_storages[1].comm._grad_ring, "region", None)
                                             and model.sharded_bucket_storages[1].comm._grad_ring.region.mc_base)
            del model, opt
        dist.barrier()
        torch.save(results, os.path.join(out, f"t{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_training_symm_paths_match_nccl(tmp_path):
    """Peer-memory collectives, with weight gradients stored straight into the owners' memory and
    (third arm) AdamW applied inside the reduce kernel, train like the NCCL path."""
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_train_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"t{r}.pt")
        for mode in ("symm", "symm_fused_adam", "symm_fused_adam_peer_loads", "symm_fused_adam_staged",
                     "symm_fused_adam_sm_gather"):
            for a, b in zip(res[mode], res["nccl"]):
                assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (mode, res)
        # at two ranks every sum has one order: the in-switch reduction, the peer-load reduction and the
        # staged gathers must train to the same bits
        assert (res["symm_fused_adam"] == res["symm_fused_adam_peer_loads"] == res["symm_fused_adam_staged"]
                == res["symm_fused_adam_sm_gather"]), res
        assert res["symm_fused_adam_stats"]["dma_gathers"] > 0 and res["symm_fused_adam_sm_gather_stats"]["dma_gathers"] == 0
        st = res["symm_fused_adam_stats"]
        assert st["resident_gathers"] > 0 and st["staged_gathers"] == 0, st
        assert res["symm_fused_adam_staged_stats"]["resident_gathers"] == 0
        assert res["symm_fused_adam_peer_loads_stats"]["multimem_reduces"] == 0
        if res["symm_fused_adam_mc"]:
            assert st["multimem_reduces"] > 0 and st["peer_reduces"] == 0, st


def _muon_worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import ops
        from flex_shard_b200.dist_muon import BlockShard, BucketConfig, ComputeLayout, DistMuon, LocalMuonComputeLayout
        from flex_shard_b200.parallel.comm import set_default_backend
        from flex_shard_b200.placements import Shard

        dev = torch.device("cuda", rank)
        sh = Shard(0)
        shapes = {"a.w1": (512, 256), "a.heads": (384, 256), "b.w2": (256, 512)}
        torch.manual_seed(0)
        full = {n: torch.randn(s) for n, s in shapes.items()}
        grads = [{n: torch.randn(s, generator=torch.Generator().manual_seed(31 * t + i)) for i, (n, s) in enumerate(shapes.items())}
                 for t in range(3)]

        def rows(n, t):
            lo, hi = sh._range(t.shape[0], rank, world)
            return t[lo:hi].to(dev)

        results = {}
        for mode in ("nccl", "symm"):
            set_default_backend(mode)
            params = {n: torch.nn.Parameter(rows(n, t).clone()) for n, t in full.items()}
            lays = {n: LocalMuonComputeLayout("row_shard", global_shape=shapes[n], row_range=sh._range(shapes[n][0], rank, world))
                    for n in shapes}
            opt = DistMuon(list(params.values()), param_names=list(params), compute_layouts=lays, lr=0.02,
                           compute_sharding_by_fqn={"a.heads": ComputeLayout({"dp": BlockShard(0, (128,))})},
                           bucket_configs=[BucketConfig(("a.*",), "a"), BucketConfig(("b.*",), "b")])
            for t in range(3):
                for n, p in params.items():
                    p.grad = rows(n, grads[t][n]).clone()
                opt.step()
            torch.cuda.synchronize()
            ops.check_status()
            results[mode] = {n: p.detach().float().cpu() for n, p in params.items()}
            results[mode + "_p2p"] = opt.p2p_exchanges
            results[mode + "_collectives"] = opt.collectives_issued
            del opt, params
        set_default_backend(None)
        dist.barrier()
        torch.save(results, os.path.join(out, f"m{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_muon_row_redistribution_by_peer_pull_matches_all_to_all(tmp_path):
    """DistMuon on Shard(0)-stored matrices with fixed gradient tensors: the pipelined redistribution moves
    the row regions as peer pulls out of the senders' memory (both directions) instead of NCCL
    all-to-alls.  Pure data movement around the same Newton-Schulz kernels: the parameters must come out
    bit for bit the same."""
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_muon_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"m{r}.pt")
        # two buckets x two directions x three steps
        assert res["symm_p2p"] == 12 and res["nccl_p2p"] == 0 and res["nccl_collectives"] == 12, res
        for n in res["nccl"]:
            assert torch.equal(res["symm"][n], res["nccl"][n]), n


def _ep_worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import ops
        from flex_shard_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config
        from flex_shard_b200.parallel.comm import set_default_backend
        from flex_shard_b200.parallel.expert_parallel import apply_expert_parallel

        dev = torch.device("cuda", rank)
        cfg = DeepSeekV3Config(vocab_size=512, d_model=256, n_layers=2, n_dense_layers=1, n_heads=2, q_lora_rank=64,
                               kv_lora_rank=32, qk_nope_dim=32, qk_rope_dim=16, v_dim=32, dense_hidden=256,
                               n_experts=4, expert_hidden=128, top_k=2, n_shared_experts=1, max_seq_len=64)
        results = {}
        for mode in ("nccl", "symm", "symm_a2a"):
            # "symm": the host-free exchange (tables and rows through symmetric memory); "symm_a2a": the
            # all-to-all dispatcher whose rows travel as peer pulls after a host read of the counts
            os.environ["FSB200_EP_DISPATCH"] = "a2a" if mode == "symm_a2a" else "symm"
            set_default_backend("nccl" if mode == "nccl" else "symm")
            torch.manual_seed(0)
            model = DeepSeekV3(cfg, dtype=torch.bfloat16, device=dev)
            model.init_weights(0)
            apply_expert_parallel(model, dist.group.WORLD)
            losses = []
            for s in range(2):
                t = torch.randint(0, cfg.vocab_size, (2, 33), generator=torch.Generator().manual_seed(17 * s + rank)).to(dev)
                loss = model.loss(t[:, :-1], t[:, 1:], loss_is_root=False)
                loss.backward()
                losses.append(float(loss.detach()))
                model.zero_grad()
            torch.cuda.synchronize()
            ops.check_status()
            results[mode] = losses
            results[mode + "_p2p"] = sum(getattr(m.dispatcher._symm, "p2p_row_exchanges", 0)
                                         for m in model.moe_layers() if m.dispatcher._symm is not None)
            results[mode + "_hostfree"] = sum(getattr(getattr(m.dispatcher, "_ex", None), "exchanges", 0)
                                              for m in model.moe_layers())
            del model
        set_default_backend(None)
        dist.barrier()
        torch.save(results, os.path.join(out, f"e{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_rows_travel_by_peer_pull(tmp_path):
    """Expert-parallel dispatch and combine (forward and backward) with the token rows pulled out of
    the senders' memory over NVLink instead of an NCCL all-to-all: same losses."""
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_ep_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"e{r}.pt")
        assert res["symm_a2a_p2p"] >= 4 and res["nccl_p2p"] == 0, res   # 2 steps x (dispatch, combine, and their backward)
        assert res["symm_hostfree"] == 2 * 4 and res["symm_p2p"] == 0, res   # one MoE layer: 4 exchanges per step
        for mode in ("symm", "symm_a2a"):
            for a, b in zip(res[mode], res["nccl"]):
                assert abs(a - b) < 1e-3 * max(1.0, abs(b)), res


def _owned_worker(rank, world, port, out):
    import torch.distributed as dist
    import torch.nn as nn

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flex_shard_b200 import BucketSpec, flex_shard, ops
        from flex_shard_b200.parallel.comm import set_default_backend
        from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn

        dev = torch.device("cuda", rank)
        results = {}
        for mode in ("nccl", "symm"):
            set_default_backend(mode)
            torch.manual_seed(0)
            model = nn.Sequential(nn.Linear(16, 16), nn.Tanh(), nn.Linear(16, 8)).to(dev)   # owner rows of 272 and 136 elements
            flex_shard(model, [BucketSpec(["*"], placement_fn=make_bucketed_owned_full_param_placement_fn())])
            opt = torch.optim.SGD(model.parameters(), lr=0.1)
            for s_ in range(3):
                x = torch.randn(4, 16, generator=torch.Generator().manual_seed(10 * s_ + rank)).to(dev)
                model(x).square().mean().backward()
                opt.step()
                opt.zero_grad()
            torch.cuda.synchronize()
            ops.check_status()
            model.unshard()
            results[mode] = {n: p.detach().cpu() for n, p in model.named_parameters()}
            model.reshard()
            results[mode + "_stats"] = dict(getattr(model.sharded_bucket_storages[0].comm, "stats", {}))
            del model, opt
        set_default_backend(None)
        dist.barrier()
        torch.save(results, os.path.join(out, f"o{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_owner_rows_travel_both_ways_through_peer_memory(tmp_path):
    """Owner storage with rows of different lengths: the gather pulls each owner's row at its own length and
    the gradient reduction sums each owner's row out of the peers' memory; same parameters as the grouped NCCL
    collectives, bit for bit at two ranks."""
    import torch.multiprocessing as mp

    from tests.common import free_port

    mp.spawn(_owned_worker, args=(2, free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(tmp_path / f"o{r}.pt")
        assert res["symm_stats"].get("owner_row_reduces", 0) == 3, res["symm_stats"]
        for n in res["nccl"]:
            assert torch.equal(res["symm"][n], res["nccl"][n]), n
