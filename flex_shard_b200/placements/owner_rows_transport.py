"""Owner-rows transport: exchange back-to-back owner rows of different lengths as equal chunks.

Rows of a ``BucketedOwned`` bucket have different lengths per rank; NCCL then needs grouped
broadcasts. The chunk plan cuts the concatenation of all rows into W equal, 128-element-aligned
chunks: owners write the slices of their rows that fall in other ranks' chunks straight into those
ranks' symmetric buffers, then ONE equal-sized all-gather moves the chunks. On a single NVSwitch
domain every peer is one hop away, so there are no relays; with several hosts the plan also names,
per pair of hosts, the relay ranks ("rails") that forward cross-host slices.

Parity: ``custom_placements/owner_rows_transport.py:92-166`` (plan), ``:261-307`` (environment
switches ``FLEX_SHARD_OWNER_ROWS_TRANSPORT`` = auto | chunks | grouped and
``FLEX_SHARD_OWNER_ROWS_MAX_CROSSING`` = 0.7) of the reference.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Sequence

ALIGN = 128


def _up(x, a):
    return (x + a - 1) // a * a


@dataclass(frozen=True)
class Move:
    """``length`` elements of owner ``src``'s row starting at ``src_off`` go to chunk position
    ``dst_off`` of rank ``dst`` (``via``: relay rank for a cross-host move, else -1)."""

    src: int
    src_off: int
    dst: int
    dst_off: int
    length: int
    via: int = -1


@dataclass
class ChunkPlan:
    chunk: int                       # elements per rank chunk (multiple of 128)
    moves: list[Move] = field(default_factory=list)
    buffer_elems: int = 0            # chunk + largest relay share
    cross_host_elems: int = 0
    total_elems: int = 0

    @property
    def crossing_fraction(self) -> float:
        return self.cross_host_elems / max(1, self.total_elems)


def plan_chunks(row_lens: Sequence[int], hosts: Sequence[int] | None = None) -> ChunkPlan:
    """Every position of the concatenated rows lands in exactly one chunk position."""
    W = len(row_lens)
    hosts = list(hosts) if hosts is not None else [0] * W
    total = sum(row_lens)
    chunk = _up(-(-total // W), ALIGN) if total else ALIGN
    plan = ChunkPlan(chunk=chunk, total_elems=total)
    starts = [sum(row_lens[:r]) for r in range(W)]
    relay_share: dict[tuple[int, int], int] = {}
    for src in range(W):
        a, b = starts[src], starts[src] + row_lens[src]
        pos = a
        while pos < b:
            dst = pos // chunk
            end = min(b, (dst + 1) * chunk)
            length = end - pos
            via = -1
            if hosts[src] != hosts[dst]:
                plan.cross_host_elems += length
                pair = (hosts[src], hosts[dst])
                src_side = [r for r in range(W) if hosts[r] == pair[0]]
                dst_side = [r for r in range(W) if hosts[r] == pair[1]]
                rails = min(len(src_side), len(dst_side))
                via = dst_side[(src + dst) % rails]
                relay_share[pair] = relay_share.get(pair, 0) + length
            plan.moves.append(Move(src, pos - a, dst, pos - dst * chunk, length, via))
            pos = end
    max_relay = 0
    for (ha, hb), elems in relay_share.items():
        rails = min(sum(1 for h in hosts if h == ha), sum(1 for h in hosts if h == hb))
        max_relay = max(max_relay, _up(-(-elems // rails), ALIGN))
    plan.buffer_elems = chunk + max_relay
    return plan


def choose_transport(plan: ChunkPlan) -> str:
    """``chunks`` (symmetric-memory writes + one equal all-gather) or ``grouped`` (list-form
    collectives). ``auto`` picks chunks while at most ``FLEX_SHARD_OWNER_ROWS_MAX_CROSSING`` of the
    bucket crosses hosts (the reference measured chunks ahead at 17-57 % crossing, behind at 83 %)."""
    mode = os.environ.get("FLEX_SHARD_OWNER_ROWS_TRANSPORT", "auto")
    if mode in ("chunks", "grouped"):
        return mode
    if mode != "auto":
        raise ValueError(f"FLEX_SHARD_OWNER_ROWS_TRANSPORT must be auto, chunks or grouped, got {mode!r}")
    limit = float(os.environ.get("FLEX_SHARD_OWNER_ROWS_MAX_CROSSING", "0.7"))
    return "chunks" if plan.crossing_fraction <= limit else "grouped"


def replay(plan: ChunkPlan, row_lens: Sequence[int]) -> list[list[tuple[int, int]]]:
    """Simulate the moves: for every rank the (owner, owner offset) that lands in each chunk position
    run; used to check that every position is written exactly once."""
    W = len(row_lens)
    out = [[] for _ in range(W)]
    for m in plan.moves:
        out[m.dst].append((m.dst_off, m.dst_off + m.length, m.src, m.src_off))
    return out


def gather_owner_rows(comm, row_local, row_lens_bytes, out_rows) -> None:
    """All-gather owner rows of different lengths. On a peer-memory communicator every rank pulls
    each owner's row at its own length straight from that owner's memory (one kernel, no padding, no
    chunking: inside one NVSwitch domain the chunk/relay plan above reduces to direct access);
    otherwise the list-form collective is used."""
    if hasattr(comm, "all_gather_segments") and comm.world_size > 1:
        segs = [(r, 0, out_rows[r].data_ptr(), n) for r, n in enumerate(row_lens_bytes) if n > 0]
        comm.all_gather_segments(row_local, segs, alloc_bytes=max(row_lens_bytes))
    else:
        comm.all_gather_list(out_rows, row_local)
