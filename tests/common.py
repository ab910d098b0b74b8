"""Multi-process helpers for CPU (gloo) tests: spawn N ranks on 127.0.0.1 and collect results."""
import atexit
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


_RANK_ENV = ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE")


def _worker(rank, world_size, conn):
    """One pooled rank: takes (port, fn, args, outdir, env) tasks until it is told to stop.  Every task gets a fresh
    gloo group and the caller's current environment; a task that raises ends the process, so that its peers see a
    closed connection instead of waiting in a collective, and the pool is rebuilt."""
    torch.set_num_threads(2)
    while True:
        task = conn.recv()
        if task is None:
            return
        port, fn, args, outdir, env = task
        for k in [k for k in os.environ if k not in env and k not in _RANK_ENV]:
            del os.environ[k]
        os.environ.update(env)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size))
        try:
            dist.init_process_group("gloo", rank=rank, world_size=world_size,
                                    init_method=f"tcp://127.0.0.1:{port}")
            res = fn(rank, world_size, *args)
            dist.destroy_process_group()
            torch.save({"ok": True, "res": res}, os.path.join(outdir, f"r{rank}.pt"))
            conn.send("ok")
        except BaseException:
            torch.save({"ok": False, "err": traceback.format_exc()}, os.path.join(outdir, f"r{rank}.pt"))
            conn.send("err")
            os._exit(1)


class _Pool:
    def __init__(self, world_size: int):
        ctx = mp.get_context("spawn")
        self.world_size, self.procs, self.conns = world_size, [], []
        for r in range(world_size):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_worker, args=(r, world_size, child), daemon=True)
            p.start()
            child.close()
            self.procs.append(p)
            self.conns.append(parent)

    def close(self, kill: bool = False) -> None:
        for p, c in zip(self.procs, self.conns):
            try:
                if not kill and p.is_alive():
                    c.send(None)
            except (OSError, ValueError):
                pass
        for p in self.procs:
            p.join(0 if kill else 5)
            if p.is_alive():
                p.kill()
                p.join(5)
        for c in self.conns:
            c.close()


_pools: dict[int, _Pool] = {}


def shutdown_pools() -> None:
    """End the pooled rank processes (called after every test module, so that state cannot leak from one test
    file into another, and at exit)."""
    for pool in _pools.values():
        pool.close()
    _pools.clear()


atexit.register(shutdown_pools)


def run_ranks(fn, world_size: int, *args, timeout: float = 600.0):
    """Run ``fn(rank, world_size, *args)`` in ``world_size`` gloo processes; return their results.  The processes
    are kept for the next call of the same test module (starting an interpreter and importing torch costs more
    than most tests); any failure or timeout ends them."""
    import time

    port = free_port()
    pool = _pools.get(world_size)
    if pool is None or not all(p.is_alive() for p in pool.procs):
        if pool is not None:
            pool.close(kill=True)
        pool = _pools[world_size] = _Pool(world_size)
    env = {k: v for k, v in os.environ.items() if k not in _RANK_ENV}
    with tempfile.TemporaryDirectory() as d:
        for c in pool.conns:
            c.send((port, fn, args, d, env))
        deadline = time.monotonic() + timeout
        out, errs, healthy = [], [], True
        for r, (p, c) in enumerate(zip(pool.procs, pool.conns)):
            status = None
            try:
                if c.poll(max(0.0, deadline - time.monotonic())):
                    status = c.recv()
            except (EOFError, OSError):
                status = "gone"
            if status is None:
                errs.append(f"rank {r} timed out")
                healthy = False
                continue
            f = os.path.join(d, f"r{r}.pt")
            if not os.path.exists(f):
                errs.append(f"rank {r} exited with code {p.exitcode} and left no result")
                healthy = False
                continue
            blob = torch.load(f, weights_only=False)
            if not blob["ok"]:
                errs.append(f"rank {r}:\n{blob['err']}")
                healthy = False
            else:
                out.append(blob["res"])
        if not healthy:
            pool.close(kill=True)
            _pools.pop(world_size, None)
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
