"""Headline benchmark: training throughput (tokens/s) of a Llama-3-8B-shaped decoder.

Config (BASELINE.json, config 2): bf16 parameters and compute, fp32 gradient reduction and
optimizer state, d_model 4096, 32 layers, 32 query / 8 KV heads, SwiGLU hidden 14336, vocab
128256, sequence 8192, local batch 1, ``Shard(0)`` per-layer buckets with prefetch, AdamW.
Synthetic uniform token ids, N(0, 0.02) weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line. ``value`` is the whole-job tokens/s timed on the device (CUDA
events, max over ranks) with inputs resident on the GPU; ``e2e`` repeats the measurement through
the public API with a pinned-host -> device copy of every step's tokens and a device -> host read
of every step's loss inside the timed region.

``--impl reference`` trains a stock-PyTorch Llama of the same shape (cuBLAS, SDPA, fused AdamW,
NCCL) sharded by the unmodified reference package in ``baseline/_ref`` through its public
``flex_shard(model, buckets)`` call; ``baseline/compat.py`` supplies the few torch symbols newer than
the installed release.  ``--impl fsdp2`` shards the same model with PyTorch FSDP2 ``fully_shard``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "fsdp2"])
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--local-batch", type=int, default=1)
    ap.add_argument("--placement", choices=["shard", "fp8", "mxfp8"], default="shard",
                    help="shard (default, the headline config): Shard(0) bf16 buckets; fp8 / mxfp8: the blocks' 2-D "
                         "weights are gathered quantised and feed block-scaled GEMMs (a different configuration)")
    ap.add_argument("--keep-unsharded", type=int, default=1,
                    help="1 (default): keep the gathered bf16 parameters between forward and backward (one all-gather "
                         "per step instead of two; +2 bytes/param of HBM, affordable on 180 GB); 0: reshard after forward")
    ap.add_argument("--layers", type=int, default=32, help="debug only: fewer layers is not the headline config")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--watchdog", type=int, default=900,
                    help="seconds after which a run that has not finished prints every thread's Python stack and "
                         "exits with an error (0: off)")
    ap.add_argument("--deterministic", action="store_true",
                    help="ordered dQ accumulation in the attention backward: the loss is the same bits on every run "
                         "(off by default: the unordered kernel is faster)")
    ap.add_argument("--comm", default=os.environ.get("FSB200_COMM", "symm"), choices=["symm", "nccl"],
                    help="collectives of the sharded arm: this library's NVLink peer-memory kernels or NCCL")
    return ap.parse_args()


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only queries) while the timed
    region runs; falls back to one nvidia-smi query per sample when NVML is not importable."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.sm, self.mx, self.reasons = [], [], set()
        self._stop = threading.Event()
        self._t = None
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
        self.mx.append(float(n.nvmlDeviceGetMaxClockInfo(self._h, n.NVML_CLOCK_SM)))
        r = n.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(
            n, "nvmlDeviceGetCurrentClocksEventReasons") else n.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        table = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "sw_power_cap": 0x4}
        for name, bit in table.items():
            if r & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                              "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
        parts = [p.strip() for p in out.strip().split(",")]
        if len(parts) >= 7:
            self.sm.append(float(parts[0]))
            self.mx.append(float(parts[1]))
            for n, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"],
                            parts[3:7]):
                if v.lower().startswith("active"):
                    self.reasons.add(n)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=6)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None,
                "sm_max_mhz": max(self.mx) if self.mx else None,
                "reasons": sorted(self.reasons), "samples": len(self.sm),
                "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# --------------------------------------------------------------------------- helpers
def setup_dist(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def timed_loop(step_fn, steps: int, world: int) -> float:
    """Milliseconds per step, device time, max over ranks."""
    barrier_sync(world)
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        step_fn(i)
    e.record()
    barrier_sync(world)
    return max_over_ranks(s.elapsed_time(e), world) / steps


# --------------------------------------------------------------------------- our arm
def build_ours(args, world):
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.models.llama import Llama, LlamaConfig, llama_buckets, llama_quantized_buckets
    from flex_shard_b200.optim.adamw import FusedAdamW

    cfg = LlamaConfig(n_layers=args.layers, max_seq_len=args.seq_len)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = Llama(cfg, dtype=torch.bfloat16, device=dev)
    torch.manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm"):
                p.fill_(1.0)
            else:
                p.normal_(0.0, cfg.init_std)
    for p in model.parameters():
        p.grad_dtype = torch.float32  # keep the fp32-reduced gradients (no cast back to bf16)
    mesh = None
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh

        from flex_shard_b200.parallel.comm import set_default_backend

        set_default_backend(args.comm)
        mesh = init_device_mesh("cuda", (world,))
    placement = getattr(args, "placement", "shard")
    flex_shard(model, llama_buckets(model, mesh=mesh) if placement == "shard"
               else llama_quantized_buckets(model, mesh=mesh, kind=placement))
    if args.keep_unsharded:
        model.set_reshard_after_forward(False)
    opt = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    if world == 1 or args.comm == "symm":
        # AdamW runs as soon as a bucket's gradients are final: inside the fused reduce kernel (N > 1) or
        # as one flat launch on a side stream (N = 1), overlapped with the rest of the backward pass
        opt.fuse_into_backward(model)
    return cfg, model, opt


def run_ours(args, rank, local, world):
    from flex_shard_b200 import ops
    from flex_shard_b200.ops import attention as _attention

    _attention.set_deterministic(True if args.deterministic else None)
    cfg, model, opt = build_ours(args, world)
    B, S = args.local_batch, args.seq_len
    dev = torch.device("cuda", local)
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    n_batches = 4
    host = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    resident = [h.to(dev) for h in host]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    last_loss = [None]

    def train_step(tokens):
        loss = model.loss(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step_device(i):
        last_loss[0] = train_step(resident[i % n_batches])

    def step_e2e(i):
        tok = host[i % n_batches].to(dev, non_blocking=True)
        loss = train_step(tok)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=False)  # device -> host read of the result
        last_loss[0] = loss

    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    ops.check_status()

    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ops.launch_count()
    ms = timed_loop(step_device, args.steps, world)
    launches = ops.launch_count() - launches0
    clocks = sampler.stop()
    ops.check_status()
    loss_val = float(last_loss[0].detach().float().item())

    e2e = None
    if not args.no_e2e:
        step_e2e(0)
        ms_e2e = timed_loop(step_e2e, args.steps, world)
        tok_per_step = B * S * world
        e2e = {"value": tok_per_step / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": host[0].numel() * host[0].element_size(),
               "d2h_bytes_per_step": loss_host.numel() * loss_host.element_size()}
    # exposed communication: a few extra steps (outside both timed regions) with every wait of the compute
    # stream on a gather or a reduction bracketed by timing events; per step, max over ranks
    exposed = None
    if world > 1:
        ctx = model._fsb_ctx()
        ctx.measure_exposed_comm(True)
        n_probe = 3
        for i in range(n_probe):
            step_device(i)
        exposed = max_over_ranks(ctx.exposed_comm_ms() / n_probe, world)
        ctx.measure_exposed_comm(False)
    tokens_per_step = B * S * world
    value = tokens_per_step / (ms / 1e3)
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    if rank == 0:
        flops = cfg.flops_per_token(S) * tokens_per_step / world
        out = {
            "metric": "tokens/sec, Llama-3-8B-shaped training step (fwd+bwd+AdamW)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform random token ids, N(0,0.02) random-init weights)",
            "impl": "ours",
            "config": {"model": f"llama3-8b-shaped ({cfg.n_layers} layers, d{cfg.d_model}, {cfg.n_heads}q/{cfg.n_kv_heads}kv, "
                                f"ffn {cfg.ffn_hidden}, vocab {cfg.vocab_size})",
                       "global_batch": args.local_batch * world, "seq_len": S, "parallelism": f"dp{world}",
                       "placement": ("Shard(0) per-layer buckets" if getattr(args, "placement", "shard") == "shard" else
                                     f"{args.placement} quantised gather of the blocks' 2-D weights + Shard(0) for the rest")
                                    + ", prefetch, bf16 params / fp32 reduce+AdamW state, "
                                    + ("gathered params kept until backward" if args.keep_unsharded else "reshard after forward"),
                       "collectives": (args.comm if world > 1 else "none (1 rank)"),
                       "deterministic": bool(args.deterministic),
                       "l2": "working set per step (>=16 GB of weights) is far larger than the 126 MB L2; no explicit flush"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "exposed_comm_ms": exposed,
            "loss": loss_val, "peak_mem_gib": round(peak_gb, 2),
            "tflops_per_gpu": flops / (ms / 1e3) / 1e12,
        }
        print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------- plain-PyTorch Llama for the baseline arms
def build_plain_llama(cfg, dev):
    """The same architecture as ``flex_shard_b200.models.llama`` written with stock PyTorch modules
    (``nn.Linear`` -> cuBLAS, SDPA, ``nn.RMSNorm``): the model both baseline arms train."""
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            d, f, hd = cfg.d_model, cfg.ffn_hidden, cfg.head_dim
            self.attention_norm = nn.RMSNorm(d, eps=cfg.norm_eps)
            self.wqkv = nn.Linear(d, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, bias=False)
            self.wo = nn.Linear(d, d, bias=False)
            self.ffn_norm = nn.RMSNorm(d, eps=cfg.norm_eps)
            self.w13 = nn.Linear(d, 2 * f, bias=False)
            self.w2 = nn.Linear(f, d, bias=False)

        def forward(self, x, freqs):
            B, S, _ = x.shape
            hd = cfg.head_dim
            qkv = self.wqkv(self.attention_norm(x))
            q, k, v = qkv.split([cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.n_kv_heads * hd], dim=-1)
            q = q.view(B, S, cfg.n_heads, hd)
            k = k.view(B, S, cfg.n_kv_heads, hd)
            v = v.view(B, S, cfg.n_kv_heads, hd)

            def rope(t):
                tc = torch.view_as_complex(t.float().reshape(*t.shape[:-1], -1, 2))
                return torch.view_as_real(tc * freqs[None, :S, None, :]).flatten(3).to(t.dtype)

            q, k = rope(q), rope(k)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=True)
            x = x + self.wo(o.transpose(1, 2).reshape(B, S, -1))
            g, u = self.w13(self.ffn_norm(x)).chunk(2, dim=-1)
            return x + self.w2(F.silu(g) * u)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.d_model)
            self.layers = nn.ModuleList([Block() for _ in range(cfg.n_layers)])
            self.norm = nn.RMSNorm(cfg.d_model, eps=cfg.norm_eps)
            self.output = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)

        def forward(self, tok, freqs):
            h = self.tok_embeddings(tok)
            for layer in self.layers:
                h = layer(h, freqs)
            return self.output(self.norm(h))

    torch.manual_seed(0)
    with torch.device(dev):
        model = Model().to(torch.bfloat16)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "norm" in name:
                p.fill_(1.0)
            else:
                p.normal_(0.0, cfg.init_std)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=torch.float32) / cfg.head_dim))
    ang = torch.outer(torch.arange(cfg.max_seq_len, device=dev, dtype=torch.float32), inv)
    return model, torch.polar(torch.ones_like(ang), ang)


def shard_with_fsdp2(model, args, world):
    from torch.distributed.fsdp import MixedPrecisionPolicy as MP, fully_shard

    if world > 1:
        mp = MP(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for layer in model.layers:
            fully_shard(layer, mp_policy=mp, reshard_after_forward=not args.keep_unsharded)
        fully_shard(model, mp_policy=mp, reshard_after_forward=not args.keep_unsharded)
    return {"sharding": "torch.distributed.fsdp.fully_shard per layer + root" if world > 1 else "none (1 rank)"}


def shard_with_reference(model, args, world):
    """Shards ``model`` with the unmodified reference package (``baseline/_ref``) through its public
    ``flex_shard(model, buckets)`` call: ``Shard(0)`` buckets for the embedding, each layer and
    norm + head, the layout its FSDP2-parity test drives
    (``src/flex_shard/tests/test_flex_shard_fsdp2_parity.py:170-205``)."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flex_shard")):
        raise RuntimeError("baseline/_ref holds no installed reference package")
    sys.path.insert(0, ref_dir)
    from baseline import compat

    shims = compat.install()
    import flex_shard as ref
    from flex_shard.custom_placements import per_param_placements
    from torch.distributed.device_mesh import init_device_mesh

    if not dist.is_initialized():  # a 1-rank job still needs a process group for the mesh
        import tempfile

        store = dist.FileStore(os.path.join(tempfile.mkdtemp(prefix="fsb_ref_"), "store"), 1)
        dist.init_process_group("nccl", store=store, rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    mesh = init_device_mesh("cuda", (world,))
    mp = ref.MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)

    def bucket(patterns, reshard):
        return ref.BucketSpec(patterns, placement_fn=per_param_placements, mesh=mesh, mp_policy=mp,
                              reshard_after_forward=reshard, fsdp2_compatible=True)

    reshard = not args.keep_unsharded
    ref.flex_shard(model, buckets=[bucket(["tok_embeddings"], reshard),
                                   *(bucket([f"layers.{i}"], reshard) for i in range(len(model.layers))),
                                   bucket(["norm", "output"], False)])
    return {"sharding": "reference flex_shard(model, buckets), Shard(0) per-layer buckets, fsdp2_compatible",
            "reference_version": getattr(ref, "__version__", "0.1.0.dev0"), "torch_shims": shims}


def run_plain(args, rank, local, world, impl):
    """Times a baseline arm: the stock-PyTorch Llama sharded by ``impl`` ("reference" or "fsdp2"),
    cuBLAS + SDPA + ``torch.optim.AdamW(fused=True)``, same config, steps, timing and JSON keys."""
    import torch.nn.functional as F

    from flex_shard_b200.models.llama import LlamaConfig

    cfg = LlamaConfig(n_layers=args.layers, max_seq_len=args.seq_len)
    dev = torch.device("cuda", local)
    model, freqs = build_plain_llama(cfg, dev)
    info = (shard_with_reference if impl == "reference" else shard_with_fsdp2)(model, args, world)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    B, S = args.local_batch, args.seq_len
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory() for _ in range(4)]
    resident = [h.to(dev) for h in host]
    loss_host = torch.zeros(1).pin_memory()
    last = [None]

    def train_step(tok):
        logits = model(tok[:, :-1], freqs)
        loss = F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), tok[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        last[0] = loss
        return loss

    for i in range(args.warmup):
        train_step(resident[i % 4])
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed_loop(lambda i: train_step(resident[i % 4]), args.steps, world)
    clocks = sampler.stop()
    loss_val = float(last[0].detach().float().item())

    def e2e_step(i):
        loss = train_step(host[i % 4].to(dev, non_blocking=True))
        loss_host.copy_(loss.detach().reshape(1))

    e2e = None
    if not args.no_e2e:
        e2e_step(0)
        ms_e2e = timed_loop(e2e_step, args.steps, world)
        e2e = {"value": B * S * world / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": host[0].numel() * host[0].element_size(),
               "d2h_bytes_per_step": loss_host.numel() * loss_host.element_size()}
    tokens = B * S * world
    out = {"metric": "tokens/sec, Llama-3-8B-shaped training step (fwd+bwd+AdamW)",
           "impl": impl, "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
           "data": "synthetic (uniform random token ids, N(0,0.02) random-init weights)",
           "config": {"model": f"llama3-8b-shaped ({cfg.n_layers} layers, d{cfg.d_model}, {cfg.n_heads}q/{cfg.n_kv_heads}kv, "
                               f"ffn {cfg.ffn_hidden}, vocab {cfg.vocab_size})",
                      "global_batch": B * world, "seq_len": S, "parallelism": f"dp{world}",
                      "placement": info["sharding"] + ", bf16 params, fp32 gradient reduce, torch.optim.AdamW(fused=True), "
                                   + ("gathered params kept until backward" if args.keep_unsharded else "reshard after forward"),
                      "kernels": "stock PyTorch: cuBLAS linears, SDPA attention, NCCL collectives",
                      "l2": "working set per step (>=16 GB of weights) is far larger than the 126 MB L2; no explicit flush"},
           "clocks": clocks, "e2e": e2e, "loss": loss_val,
           "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2)}
    out.update({k: v for k, v in info.items() if k != "sharding"})
    return out


def run_reference(args, rank, local, world):
    """Reference arm.  Prints the same JSON line as the other arms with ``"impl": "reference"``; when the
    reference cannot be driven on this torch, prints ``unavailable`` naming the failing symbol, with the
    FSDP2 stand-in measured in the same process under ``stand_in``."""
    try:
        out = run_plain(args, rank, local, world, "reference")
        if rank == 0:
            print(json.dumps(out), flush=True)
        return
    except Exception as exc:  # a private torch>=2.16 API the shims do not cover, or an absent install
        import traceback

        tb = traceback.extract_tb(exc.__traceback__)
        where = f"{os.path.basename(tb[-1].filename)}:{tb[-1].lineno}" if tb else "?"
        reason = (f"reference cannot run on torch {torch.__version__}: {type(exc).__name__}: "
                  f"{str(exc).splitlines()[0][:200] if str(exc) else ''} (at {where})")
    stand_in = None
    try:
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        stand_in = run_plain(args, rank, local, world, "fsdp2")
    except Exception as exc:
        stand_in = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason, "stand_in": stand_in}), flush=True)


def run_fsdp2(args, rank, local, world):
    out = run_plain(args, rank, local, world, "fsdp2")
    if rank == 0:
        print(json.dumps(out), flush=True)


def main():
    args = parse()
    if args.impl == "reference" and not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device in this process"}), flush=True)
        return
    if args.impl == "ours":
        # before CUDA initialises: kernels that wait for a peer must not meet lazy kernel loading
        os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    if args.watchdog > 0:
        import faulthandler

        faulthandler.dump_traceback_later(args.watchdog, exit=True)
    rank, local, world = setup_dist(args)
    try:
        if args.impl == "reference":
            run_reference(args, rank, local, world)
        elif args.impl == "fsdp2":
            run_fsdp2(args, rank, local, world)
        else:
            run_ours(args, rank, local, world)
    finally:
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
