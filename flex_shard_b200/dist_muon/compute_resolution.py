"""From (how a parameter is stored, what the user asks Muon to compute on) to concrete matrices and owners.

``resolve_compute`` takes a parameter's storage description (``LocalMuonComputeLayout`` from the storage
bridge) and an optional public ``ComputeLayout`` and returns a ``ResolvedCompute``: the Newton-Schulz
matrices as dim-0 row blocks of the logical tensor, whether they already sit whole on one rank
(``local``) or have to travel (``redistributed``), and, for travelling ones, the owner of each matrix.
``validate_compute_layout`` rejects layouts that cannot be realised, with messages that name the
parameter, before any plan is built.

Rules (parity: the resolution and validator of the reference, ``dist_muon/optimizer.py:1468-1500`` and
``:1588-1963``, restated for plain local tensors):

* at most one mesh axis of a ``ComputeLayout`` may shard or own; the others must be absent
  (a parameter is redistributed, or gathered to its owner, along one axis only);
* ``BlockShard`` needs a 2-D parameter, ``dim == 0`` and rows in whole repetitions of ``block_sizes``; every
  block is its own matrix and the blocks are spread over the ranks in contiguous runs;
* ``Owned()`` computes the whole tensor on one rank; ``Owned(block_sizes)`` (2-D, whole repetitions) makes
  every block its own matrix with its own owner; owners come from ``owner_by_fqn`` or from the balancer;
* a native ``[n, R, C]`` batch is computed slice by slice: no ``block_sizes``; its slices are spread like
  ``Shard(0)`` over the leading dimension or owned one by one;
* storage that already holds whole matrices (owner storage, head-block storage, expert slabs) fixes the
  compute layout: a ``ComputeLayout`` is accepted only if it describes the same blocks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Mapping, Sequence

from .optimizer_reshard import BlockShard, ComputeLayout, Owned


@dataclass(frozen=True)
class ResolvedCompute:
    fqn: str
    mode: str                               # "local" | "redistributed"
    logical_shape: tuple[int, ...]
    blocks: tuple[tuple[int, int], ...]     # [lo, hi) dim-0 rows of every Newton-Schulz matrix, logical coordinates
    batch: bool = False                     # True: every block is one slice of a native [n, R, C] batch
    spread: str = "owned"                   # redistributed only: "owned" (balanced / fixed owners) | "contiguous"
    local_kind: str | None = None           # local only: owned | row_blocks | matrix_batch

    @property
    def matrix_shape(self) -> tuple[int, int]:
        if self.batch:
            return (self.logical_shape[1], math.prod(self.logical_shape[2:]))
        return (self.blocks[0][1] - self.blocks[0][0], math.prod(self.logical_shape[1:]))

    def matrix_shapes(self) -> list[tuple[int, int]]:
        if self.batch:
            return [self.matrix_shape] * len(self.blocks)
        cols = math.prod(self.logical_shape[1:])
        return [(hi - lo, cols) for lo, hi in self.blocks]


def _tile(fqn: str, rows: int, sizes: Sequence[int]) -> tuple[tuple[int, int], ...]:
    sizes = tuple(int(s) for s in sizes)
    if not sizes or any(s <= 0 for s in sizes):
        raise ValueError(f"{fqn!r}: block_sizes must be positive integers, got {sizes}")
    period = sum(sizes)
    if rows % period != 0:
        raise ValueError(f"{fqn!r}: {rows} rows are not whole repetitions of block_sizes {sizes} (period {period})")
    out, pos = [], 0
    while pos < rows:
        for s in sizes:
            out.append((pos, pos + s))
            pos += s
    return tuple(out)


def _single_sharding(fqn: str, layout: ComputeLayout):
    live = {axis: sh for axis, sh in (layout.shardings_by_mesh_axis or {}).items() if sh is not None}
    if len(live) > 1:
        raise ValueError(f"{fqn!r}: DistMuon redistributes a parameter along at most one mesh axis, "
                         f"but its ComputeLayout shards on {sorted(live)}")
    order = layout.shard_order_by_tensor_dim or {}
    for dim, axes in order.items():
        if dim != 0:
            raise ValueError(f"{fqn!r}: shard_order_by_tensor_dim may only order tensor dim 0, got dim {dim}")
        unknown = [a for a in axes if a not in (layout.shardings_by_mesh_axis or {})]
        if unknown:
            raise ValueError(f"{fqn!r}: shard_order_by_tensor_dim names mesh axes {unknown} without a sharding")
    return next(iter(live.values())) if live else None


def validate_compute_layout(fqn: str, logical_shape: Sequence[int], layout: ComputeLayout | None) -> None:
    """Raise ``ValueError`` if ``layout`` cannot describe Muon matrices of a tensor of ``logical_shape``."""
    shape = tuple(logical_shape)
    if len(shape) not in (2, 3):
        raise ValueError(f"{fqn!r}: Muon parameters are matrices or [n, R, C] matrix batches, got shape {shape}")
    if layout is None:
        return
    sh = _single_sharding(fqn, layout)
    if sh is None:
        return
    if isinstance(sh, BlockShard):
        if len(shape) != 2:
            raise ValueError(f"{fqn!r}: BlockShard needs a 2-D parameter, got shape {shape}")
        if sh.dim != 0:
            raise ValueError(f"{fqn!r}: BlockShard must cut dim 0 (rows), got dim {sh.dim}")
        _tile(fqn, shape[0], sh.block_sizes)
    elif isinstance(sh, Owned):
        if sh.block_sizes is not None:
            if len(shape) != 2:
                raise ValueError(f"{fqn!r}: Owned(block_sizes) needs a 2-D parameter, got shape {shape}")
            _tile(fqn, shape[0], sh.block_sizes)
    elif type(sh).__name__ == "Shard" and getattr(sh, "dim", None) == 0:
        if len(shape) != 3:
            raise ValueError(f"{fqn!r}: Shard(0) compute spreads a native [n, R, C] batch; got shape {shape}")
    elif type(sh).__name__ == "Replicate":
        raise ValueError(f"{fqn!r}: a replicated compute layout is not supported (every rank would redo the work)")
    else:
        raise ValueError(f"{fqn!r}: unsupported compute sharding {sh!r}")


def resolve_compute(fqn: str, storage, layout: ComputeLayout | None) -> ResolvedCompute:
    """``storage``: the parameter's ``LocalMuonComputeLayout`` (kind, global_shape, block_rows, row_range)."""
    shape = tuple(storage.global_shape) if storage.global_shape is not None else None
    if shape is None:
        raise ValueError(f"{fqn!r}: the storage layout carries no global shape")
    validate_compute_layout(fqn, shape, layout)
    sh = _single_sharding(fqn, layout) if layout is not None else None
    batch = len(shape) == 3
    if storage.kind != "row_shard":
        # the storage already holds whole matrices: nothing travels, the layout can only confirm it
        if storage.kind == "owned":
            blocks = tuple((i, i + 1) for i in range(shape[0])) if batch else ((0, shape[0]),)
            if isinstance(sh, Owned) and sh.block_sizes is not None or isinstance(sh, BlockShard):
                raise ValueError(f"{fqn!r}: stored whole on its owner; a block compute layout needs block storage")
        elif storage.kind == "matrix_batch":
            blocks = tuple((i, i + 1) for i in range(shape[0]))
        elif storage.kind == "row_blocks":
            rows = tuple(storage.block_rows or ())
            want = _tile(fqn, shape[0], sh.block_sizes) if isinstance(sh, (BlockShard, Owned)) and getattr(
                sh, "block_sizes", None) else None
            if want is not None and rows and {hi - lo for lo, hi in want} != set(rows):
                raise ValueError(f"{fqn!r}: stored in blocks of {sorted(set(rows))} rows, compute layout asks for "
                                 f"{sorted({hi - lo for lo, hi in want})}")
            blocks = want or ((0, shape[0]),)
        else:
            raise ValueError(f"{fqn!r}: unknown storage kind {storage.kind!r}")
        return ResolvedCompute(fqn, "local", shape, blocks, batch=batch and storage.kind != "row_blocks",
                               local_kind=storage.kind)
    # Shard(0) rows on several ranks: everything travels
    if batch:
        if isinstance(sh, (BlockShard,)) or (isinstance(sh, Owned) and sh.block_sizes is not None):
            raise ValueError(f"{fqn!r}: a native matrix batch takes no block_sizes")
        blocks = tuple((i, i + 1) for i in range(shape[0]))
        spread = "contiguous" if (sh is not None and type(sh).__name__ == "Shard") else "owned"
        return ResolvedCompute(fqn, "redistributed", shape, blocks, batch=True, spread=spread)
    if isinstance(sh, BlockShard):
        return ResolvedCompute(fqn, "redistributed", shape, _tile(fqn, shape[0], sh.block_sizes), spread="contiguous")
    if isinstance(sh, Owned) and sh.block_sizes is not None:
        return ResolvedCompute(fqn, "redistributed", shape, _tile(fqn, shape[0], sh.block_sizes), spread="owned")
    return ResolvedCompute(fqn, "redistributed", shape, ((0, shape[0]),), spread="owned")


def contiguous_owners(num_blocks: int, world: int) -> list[int]:
    """Blocks spread over ranks in contiguous runs of ``ceil(num_blocks / world)`` (``Shard(0)`` geometry)."""
    chunk = -(-num_blocks // world)
    return [min(b // chunk, world - 1) for b in range(num_blocks)]


def resolve_all(names: Sequence[str], storages: Mapping[str, object],
                layouts: Mapping[str, ComputeLayout] | None) -> dict[str, ResolvedCompute]:
    unknown = sorted(set(layouts or {}) - set(names))
    if unknown:
        raise ValueError(f"compute_sharding_by_fqn names parameters the optimizer does not hold: {unknown}")
    return {n: resolve_compute(n, storages[n], (layouts or {}).get(n)) for n in names}
