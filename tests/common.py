"""Multi-process helpers for CPU (gloo) tests: spawn N ranks on 127.0.0.1 and collect results."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world_size, port, fn, args, outdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world_size,
                                init_method=f"tcp://127.0.0.1:{port}")
        res = fn(rank, world_size, *args)
        torch.save({"ok": True, "res": res}, os.path.join(outdir, f"r{rank}.pt"))
    except Exception:
        torch.save({"ok": False, "err": traceback.format_exc()}, os.path.join(outdir, f"r{rank}.pt"))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world_size: int, *args, timeout: float = 600.0):
    """Run ``fn(rank, world_size, *args)`` in ``world_size`` gloo processes; return their results."""
    port = free_port()
    with tempfile.TemporaryDirectory() as d:
        ctx = mp.get_context("spawn")
        procs = [ctx.Process(target=_entry, args=(r, world_size, port, fn, args, d)) for r in range(world_size)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout)
        out = []
        errs = []
        for r, p in enumerate(procs):
            if p.is_alive():
                p.kill()
                errs.append(f"rank {r} timed out")
                continue
            f = os.path.join(d, f"r{r}.pt")
            if not os.path.exists(f):
                errs.append(f"rank {r} exited with code {p.exitcode} and left no result")
                continue
            blob = torch.load(f, weights_only=False)
            if not blob["ok"]:
                errs.append(f"rank {r}:\n{blob['err']}")
            else:
                out.append(blob["res"])
        if errs:
            raise AssertionError("\n".join(errs))
        return out


class FakeMesh:
    """A mesh stand-in for planning tests: no process group, just (world_size, rank)."""

    def __init__(self, world_size: int, rank: int = 0, device: str = "cpu"):
        self.world_size = world_size
        self.rank = rank
        self.device = device
        self.ndim = 1

    def size(self):
        return self.world_size

    def get_local_rank(self):
        return self.rank
