"""Owner assignment for Muon matrices and the bucket recipe built on it.

``assign_matrices`` balances Newton-Schulz cost over ranks with longest-processing-time first,
hosts before ranks, group by group; ``materialize_dist_muon_buckets`` turns a model description
(initial / per-block / final parameter groups) into the ``BucketSpec`` list.

Parity: ``dist_muon/bucket_planner.py:147-517`` of the reference. Note the reference's own
remark (``:159-171``): balancing each group separately leaves the most loaded rank at about
1.39x the mean on a 4-layer/8-rank example where a global LPT reaches 1.06x; ``carry_loads``
carries the loads from group to group to approach the latter.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Any, Mapping, Protocol, Sequence

import torch.distributed as dist

from ..bucket_storage import BucketSpec, MixedPrecisionPolicy
from ..placements.block_shard import BlockShard
from ..placements.mixed_bucket import MixedBucketPlacement
from ..placements.owned import BucketedOwned, newton_schulz_cost
from ..placements.shard import Shard, shard_placement_fn
from ..utils.validation import assign_to_hosts_then_ranks, mesh_rank_hosts
from .placement import get_dim0_block_partitions, get_mesh_rank_groups


@dataclass(frozen=True)
class MatrixSpec:
    fqn: str
    shape: tuple[int, ...]
    num_blocks: int = 1   # > 1: a block group (e.g. heads) spread over ranks block by block
    eligible_ranks: tuple[int, ...] | None = None   # block groups only: the ranks that may hold blocks (default: all)
    cost: float | None = None   # load of the matrix (of one block, for a block group); default: its Newton-Schulz cost

    def load(self, ns_steps: int = 5) -> float:
        if self.cost is not None:
            return float(self.cost)
        if self.num_blocks <= 1:
            return newton_schulz_cost(self.shape, ns_steps)
        return newton_schulz_cost((self.shape[0] // self.num_blocks, *self.shape[1:]), ns_steps)


# ---- the planner's inputs and answer in the shape the reference's recipes use (``dist_muon/bucket_planner.py:33-82``
# of the reference): loads are element counts, block counts follow each group's ``eligible_ranks`` order
@dataclass(frozen=True)
class WholeMatrixSpec:
    """One complete matrix stored on one rank."""
    name: str
    numel: int


@dataclass(frozen=True)
class MatrixBlockGroupSpec:
    """Equal blocks (possibly of several matrices) spread over the eligible ranks."""
    name: str
    num_blocks: int
    block_numel: int
    eligible_ranks: tuple[int, ...]


@dataclass(frozen=True)
class AssignmentGroup:
    """Whole matrices and block groups that are balanced in one step (one transformer block, say)."""
    matrices: tuple[WholeMatrixSpec, ...] = ()
    block_groups: tuple[MatrixBlockGroupSpec, ...] = ()


@dataclass(frozen=True)
class MatrixAssignment:
    """Owners of whole matrices and, per block group, blocks per rank in its ``eligible_ranks`` order."""
    rank_by_matrix: dict
    blocks_per_rank_by_group: dict


class MatrixAssignmentFn(Protocol):
    """A custom balancer: runs on every rank and must give the same answer everywhere."""

    def __call__(self, groups: Sequence[AssignmentGroup], *, num_ranks: int) -> MatrixAssignment: ...


@dataclass(frozen=True)
class PackedParameterPlan:
    """A 2-D parameter that packs ``block_plan.num_matrices`` equal matrices along dim 0 (attention heads); every
    matrix gets its own owner and the parameter is stored in whole matrices (``BlockShard``)."""
    fqn: str
    parameter: Any
    block_plan: Any      # BlockShardPlan


@dataclass(frozen=True)
class ParameterBucketPlan:
    """One step of a recipe (a transformer block): ``mixed_fqns`` go into one mixed bucket on the assignment mesh, in
    which ``owned_parameters`` are whole on an owner, ``packed_parameters`` are stored matrix by matrix and the rest is
    ``Shard(0)``; ``partitioned_parameters`` (stacked ``[blocks, ...]`` weights that an outer mesh axis already
    partitions, e.g. experts under expert parallelism) go into a flat block bucket on the partition's own ranks."""
    mixed_fqns: tuple = ()
    owned_parameters: tuple = ()
    packed_parameters: tuple = ()
    partitioned_parameters: tuple = ()
    partition_group_name_prefix: str = "partition#"


def _assign_groups(groups: Sequence[AssignmentGroup], num_ranks: int, hosts: Sequence[int] | None) -> MatrixAssignment:
    """Groups are balanced one after the other on top of the loads the earlier ones left.  Whole matrices of a group:
    without ``hosts``, packed into one pile per rank (largest first onto the lightest pile), then the heaviest pile
    goes to the rank that carries least so far; with ``hosts``, the piles go to hosts first and then to their ranks, one
    pile per rank (``assign_to_hosts_then_ranks`` with earlier loads as tie-break).
    Blocks of a block group go one by one to the least loaded eligible rank (ties: the earlier eligible rank)."""
    if num_ranks <= 0:
        raise ValueError("num_ranks must be positive")
    if hosts is not None and len(hosts) != num_ranks:
        raise ValueError(f"hosts must give each of the {num_ranks} ranks a host, got {len(hosts)} entries")
    seen: set[str] = set()
    for g in groups:
        for m in g.matrices:
            if m.numel <= 0:
                raise ValueError(f"whole matrix {m.name!r} must have a positive numel")
        for b in g.block_groups:
            if b.num_blocks <= 0 or b.block_numel <= 0:
                raise ValueError(f"block group {b.name!r} needs positive num_blocks and block_numel")
            ranks = tuple(b.eligible_ranks)
            if (not ranks or len(set(ranks)) != len(ranks) or any(not isinstance(r, int) for r in ranks)
                    or min(ranks) < 0 or max(ranks) >= num_ranks):
                raise ValueError(f"eligible_ranks of block group {b.name!r} must be distinct ranks of the "
                                 f"{num_ranks}-rank mesh, got {b.eligible_ranks!r}")
        for item in (*g.matrices, *g.block_groups):
            if item.name in seen:
                raise ValueError(f"Duplicate assignment name {item.name!r}: every matrix and block group gets one entry")
            seen.add(item.name)
    loads = [0.0] * num_ranks
    whole: dict[str, int] = {}
    blocks: dict[str, tuple[int, ...]] = {}
    for g in groups:
        if g.matrices:
            piles = [[0.0, []] for _ in range(num_ranks)]
            for m in sorted(g.matrices, key=lambda m: -m.numel):
                pile = min(piles, key=lambda p: p[0])          # min keeps the first of equals: the lowest pile index
                pile[0] += m.numel
                pile[1].append(m.name)
            if hosts is None:
                # the heaviest pile to the rank that carries least so far
                lightest_first = sorted(range(num_ranks), key=lambda r: loads[r])
                pairs = zip(sorted(piles, key=lambda p: -p[0]), lightest_first)
            else:
                # one pile per rank, hosts first: heavy and light hosts alternate in rank order
                ranks = assign_to_hosts_then_ranks([p[0] for p in piles], list(hosts), carried_loads=loads,
                                                   one_per_rank=True)
                pairs = zip(piles, ranks)
            for pile, r in list(pairs):
                for name in pile[1]:
                    whole[name] = r
                loads[r] += pile[0]
        for b in g.block_groups:
            counts = [0] * len(b.eligible_ranks)
            for _ in range(b.num_blocks):
                pos = min(range(len(counts)), key=lambda i: loads[b.eligible_ranks[i]])
                counts[pos] += 1
                loads[b.eligible_ranks[pos]] += b.block_numel
            blocks[b.name] = tuple(counts)
    return MatrixAssignment(whole, blocks)


def validate_assignment(groups: Sequence[Sequence[MatrixSpec]], num_ranks: int,
                        owners: Mapping[str, int | tuple[int, ...]]) -> None:
    """Check an assignment (from ``assign_matrices`` or a custom function): every matrix has exactly one entry, whole
    matrices name a rank of the mesh, block groups give one non-negative count per rank that sum to the number of
    blocks and are zero outside the eligible ranks.  Parity: the checks the reference applies to a custom
    ``MatrixAssignmentFn`` (``dist_muon/bucket_planner.py:260-330``)."""
    expected = {m.fqn: m for g in groups for m in g}
    missing = sorted(set(expected) - set(owners))
    unexpected = sorted(set(owners) - set(expected))
    if missing or unexpected:
        raise ValueError(f"matrix assignment does not match the recipe: missing {missing}, unexpected {unexpected}")
    for fqn, m in expected.items():
        o = owners[fqn]
        if m.num_blocks <= 1:
            if isinstance(o, bool) or not isinstance(o, int) or not 0 <= o < num_ranks:
                raise ValueError(f"owner of {fqn!r} must be a rank in [0, {num_ranks}), got {o!r}")
            continue
        if (not isinstance(o, (tuple, list)) or len(o) != num_ranks
                or any((not isinstance(c, int)) or c < 0 for c in o) or sum(o) != m.num_blocks):
            raise ValueError(f"block group {fqn!r} needs {num_ranks} non-negative block counts that sum to "
                             f"{m.num_blocks}, got {o!r}")
        if m.eligible_ranks is not None and any(c and r not in m.eligible_ranks for r, c in enumerate(o)):
            raise ValueError(f"block group {fqn!r} places blocks outside its eligible ranks {m.eligible_ranks}: {o!r}")


def assign_matrices(groups, num_ranks: int, *, ranks_per_host: int | None = None,
                    ns_steps: int = 5, carry_loads: bool = False,
                    fixed_owners: Mapping[str, int] | None = None, hosts: Sequence[int] | None = None):
    """Owner rank per matrix (or per block, as a tuple of blocks-per-rank, for block groups).

    ``groups`` of ``MatrixSpec`` lists return ``{fqn: rank | blocks per rank}``.  ``groups`` of ``AssignmentGroup``
    (the reference's recipe types: loads are element counts, carried from group to group; ``hosts`` as
    ``mesh_rank_hosts`` gives them) return a ``MatrixAssignment``."""
    groups = list(groups)
    if groups and all(isinstance(g, AssignmentGroup) for g in groups):
        if fixed_owners:
            raise ValueError("fixed_owners goes with MatrixSpec groups")
        return _assign_groups(groups, num_ranks, hosts)
    hosts = mesh_rank_hosts(num_ranks, ranks_per_host)
    loads = [0.0] * num_ranks
    out: dict[str, int | tuple[int, ...]] = {}
    seen: set[str] = set()
    for group in groups:
        for m in group:
            if m.fqn in seen:
                raise ValueError(f"matrix {m.fqn!r} is listed more than once: every matrix gets exactly one owner")
            seen.add(m.fqn)
    for fqn, r in (fixed_owners or {}).items():
        if not 0 <= int(r) < num_ranks:
            raise ValueError(f"fixed owner {r} of {fqn!r} is not a rank of the {num_ranks}-rank mesh")
    for group in groups:
        if not carry_loads:
            loads = [0.0] * num_ranks
        whole = [m for m in group if m.num_blocks <= 1]
        for m in whole:
            if fixed_owners and m.fqn in fixed_owners:
                out[m.fqn] = fixed_owners[m.fqn]
                loads[out[m.fqn]] += m.load(ns_steps)
        free = [m for m in whole if m.fqn not in out]
        owners = assign_to_hosts_then_ranks([m.load(ns_steps) for m in free], hosts, loads)
        for m, r in zip(free, owners):
            out[m.fqn] = r
        for m in group:
            if m.num_blocks <= 1:
                continue
            cost = m.load(ns_steps)
            if m.eligible_ranks is None:
                per_block = assign_to_hosts_then_ranks([cost] * m.num_blocks, hosts, loads)
            else:
                ranks = sorted(set(int(r) for r in m.eligible_ranks))
                if not ranks or ranks[0] < 0 or ranks[-1] >= num_ranks:
                    raise ValueError(f"eligible_ranks of {m.fqn!r} must name ranks of the {num_ranks}-rank mesh")
                sub = [loads[r] for r in ranks]
                local = assign_to_hosts_then_ranks([cost] * m.num_blocks, [hosts[r] for r in ranks], sub)
                per_block = [ranks[i] for i in local]
                for i, r in enumerate(ranks):
                    loads[r] = sub[i]
            counts = [0] * num_ranks
            for r in per_block:
                counts[r] += 1
            out[m.fqn] = tuple(counts)
    validate_assignment(groups, num_ranks, out)
    return out


def _check_plan_assignment(groups: Sequence[AssignmentGroup], answer, num_ranks: int) -> None:
    if not isinstance(answer, MatrixAssignment):
        raise TypeError(f"the assignment function must return a MatrixAssignment, got {type(answer).__name__}")
    want_m = {m.name for g in groups for m in g.matrices}
    want_b = {b.name: b for g in groups for b in g.block_groups}
    if set(answer.rank_by_matrix) != want_m:
        raise ValueError(f"Matrix assignment names do not match the recipe: missing "
                         f"{sorted(want_m - set(answer.rank_by_matrix))}, unexpected "
                         f"{sorted(set(answer.rank_by_matrix) - want_m)}")
    if set(answer.blocks_per_rank_by_group) != set(want_b):
        raise ValueError(f"Block group names do not match the recipe: missing "
                         f"{sorted(set(want_b) - set(answer.blocks_per_rank_by_group))}, unexpected "
                         f"{sorted(set(answer.blocks_per_rank_by_group) - set(want_b))}")
    for name, r in answer.rank_by_matrix.items():
        if isinstance(r, bool) or not isinstance(r, int) or not 0 <= r < num_ranks:
            raise ValueError(f"owner of {name!r} must be a rank in [0, {num_ranks}), got {r!r}")
    for name, counts in answer.blocks_per_rank_by_group.items():
        b = want_b[name]
        if (len(counts) != len(b.eligible_ranks) or any(isinstance(c, bool) or not isinstance(c, int) or c < 0
                                                        for c in counts) or sum(counts) != b.num_blocks):
            raise ValueError(f"block group {name!r} needs {len(b.eligible_ranks)} non-negative block counts that sum "
                             f"to {b.num_blocks}, got {tuple(counts)!r}")


def _materialize_from_plans(*, bucket_plans, assignment_name_by_fqn, initial_sharded_fqns, final_sharded_fqn_groups,
                            assignment_mesh, partition_mesh, partition_rank_axis_name, partition_axis_name, mp_policy,
                            assignment_fn) -> list[BucketSpec]:
    """The recipe form of ``materialize_dist_muon_buckets`` (parity: ``dist_muon/bucket_planner.py:328-517`` of the
    reference): initial ``Shard(0)`` bucket, per plan a mixed bucket (owned + packed + ``Shard(0)``) and a flat block
    bucket of its partitioned weights on the partition's ranks, final ``Shard(0)`` buckets that stay gathered; all
    buckets sum their gradients."""
    from ..placements.bucketed_block_shard import make_bucketed_block_shard_placement_fn
    from ..placements.mixed_bucket import make_mixed_placement_fn

    W = int(assignment_mesh.size())
    if partition_mesh is None:
        storage_mesh, rank_groups, mine = assignment_mesh, (tuple(range(W)),), 0
    else:
        storage_mesh = partition_mesh[partition_rank_axis_name]
        rank_groups = get_mesh_rank_groups(assignment_mesh, partition_mesh, rank_axis_name=partition_rank_axis_name,
                                           partition_axis_name=partition_axis_name)
        mine = int(partition_mesh.get_local_rank(partition_axis_name))
    groups, group_names, matrix_to_packed, owned_fqns = [], [], {}, []
    for plan in bucket_plans:
        matrices = []
        for fqn, p in plan.owned_parameters:
            matrices.append(WholeMatrixSpec(assignment_name_by_fqn[fqn], p.numel()))
            owned_fqns.append(fqn)
        for packed in sorted(plan.packed_parameters, key=lambda sp: assignment_name_by_fqn[sp.fqn]):
            packed.block_plan.validate_parameter(packed.fqn, packed.parameter)
            k = packed.block_plan.num_matrices
            for i in range(k):
                name = f"{assignment_name_by_fqn[packed.fqn]}#matrix{i}"
                matrices.append(WholeMatrixSpec(name, packed.parameter.numel() // k))
                matrix_to_packed[name] = packed.fqn
        block_groups = ()
        if plan.partitioned_parameters:
            (n, numel), *_ = get_dim0_block_partitions(plan.partitioned_parameters, num_partitions=len(rank_groups),
                                                       partition_index=mine)
            block_groups = tuple(MatrixBlockGroupSpec(f"{plan.partition_group_name_prefix}{i}", n, numel, ranks)
                                 for i, ranks in enumerate(rank_groups))
        groups.append(AssignmentGroup(tuple(matrices), block_groups))
        group_names.append(tuple(b.name for b in block_groups))
    if assignment_fn is None:
        # hosts from the mesh's global ranks (a sub-mesh, e.g. one pipeline stage, does not start at rank 0)
        answer = _assign_groups(groups, W, mesh_rank_hosts([int(r) for r in assignment_mesh.mesh.flatten().tolist()]))
    else:
        _assign_groups(groups, W, None)            # the same input checks a built-in run would make
        answer = assignment_fn(tuple(groups), num_ranks=W)
    _check_plan_assignment(groups, answer, W)
    owned_rank = {f: answer.rank_by_matrix[assignment_name_by_fqn[f]] for f in owned_fqns}
    counts_by_fqn: dict[str, list[int]] = {}
    for name, fqn in matrix_to_packed.items():
        counts_by_fqn.setdefault(fqn, [0] * W)[answer.rank_by_matrix[name]] += 1
    kw = dict(mp_policy=mp_policy, gradient_reduce_op=dist.ReduceOp.SUM)
    specs = []
    if initial_sharded_fqns:
        specs.append(BucketSpec(tuple(initial_sharded_fqns), placement_fn=shard_placement_fn(0), mesh=assignment_mesh,
                                reshard_after_forward=True, **kw))
    for plan, names in zip(bucket_plans, group_names):
        if plan.mixed_fqns:
            inside = set(plan.mixed_fqns)
            fn = make_mixed_placement_fn({f: r for f, r in owned_rank.items() if f in inside},
                                         {f: tuple(c) for f, c in counts_by_fqn.items() if f in inside})
            specs.append(BucketSpec(tuple(plan.mixed_fqns), placement_fn=fn, mesh=assignment_mesh,
                                    reshard_after_forward=True, **kw))
        if plan.partitioned_parameters:
            counts = answer.blocks_per_rank_by_group[names[mine]]
            specs.append(BucketSpec(tuple(f for f, _ in plan.partitioned_parameters),
                                    placement_fn=make_bucketed_block_shard_placement_fn(tuple(counts)),
                                    mesh=storage_mesh, reshard_after_forward=True, **kw))
    for fqns in final_sharded_fqn_groups:
        if fqns:
            specs.append(BucketSpec(tuple(fqns), placement_fn=shard_placement_fn(0), mesh=assignment_mesh,
                                    reshard_after_forward=False, **kw))
    return specs


def materialize_dist_muon_buckets(named_params=None, mesh=None, *, initial: Sequence[str] = (),
                                  blocks: Sequence[Sequence[str]] = (), final: Sequence[str] = (), is_matrix=None,
                                  num_blocks_of=None, mp_policy: MixedPrecisionPolicy | None = None,
                                  carry_loads: bool = True, ranks_per_host: int | None = None, assignment_fn=None,
                                  bucket_plans=None, assignment_name_by_fqn: Mapping[str, str] | None = None,
                                  initial_sharded_fqns: Sequence[str] = (),
                                  final_sharded_fqn_groups: Sequence[Sequence[str]] = (), assignment_mesh=None,
                                  partition_mesh=None, partition_rank_axis_name: str = "",
                                  partition_axis_name: str = "") -> list[BucketSpec]:
    """BucketSpecs for a Muon-trained model: ``initial`` / ``final`` pattern groups stay ``Shard(0)``
    (AdamW parameters); each entry of ``blocks`` becomes one mixed bucket whose matrices are owned
    whole (or block-sharded when ``num_blocks_of`` says so) and whose vectors are ``Shard(0)``.
    All buckets sum gradients (``ReduceOp.SUM``), as the reference's recipe does.  ``assignment_fn(groups,
    num_ranks=W) -> {fqn: rank | blocks per rank}`` replaces the built-in balancer.

    With ``bucket_plans`` (``ParameterBucketPlan``s) the call takes the reference's recipe form instead
    (``assignment_name_by_fqn``, ``initial_sharded_fqns``, ``final_sharded_fqn_groups``, ``assignment_mesh``,
    ``partition_mesh`` and its two axis names): see ``_materialize_from_plans``."""
    if bucket_plans is not None:
        if assignment_name_by_fqn is None or assignment_mesh is None:
            raise ValueError("the recipe form needs assignment_name_by_fqn and assignment_mesh")
        return _materialize_from_plans(
            bucket_plans=tuple(bucket_plans), assignment_name_by_fqn=assignment_name_by_fqn,
            initial_sharded_fqns=initial_sharded_fqns, final_sharded_fqn_groups=final_sharded_fqn_groups,
            assignment_mesh=assignment_mesh, partition_mesh=partition_mesh,
            partition_rank_axis_name=partition_rank_axis_name, partition_axis_name=partition_axis_name,
            mp_policy=mp_policy or MixedPrecisionPolicy(), assignment_fn=assignment_fn)
    if named_params is None:
        raise ValueError("materialize_dist_muon_buckets needs named_params and mesh, or bucket_plans")
    from ..parallel.comm import mesh_group

    _, _, W, _ = mesh_group(mesh)
    named = list(named_params)
    is_matrix = is_matrix or (lambda n, p: p.dim() >= 2)
    mp = mp_policy or MixedPrecisionPolicy()
    groups = []
    for pats in blocks:
        g = []
        for n, p in named:
            if any(fnmatch.fnmatchcase(n, pat) or n.startswith(pat + ".") for pat in pats) and is_matrix(n, p):
                nb = num_blocks_of(n, p) if num_blocks_of else 1
                g.append(MatrixSpec(n, tuple(p.shape), nb))
        groups.append(g)
    if assignment_fn is not None:
        # a custom balancer: called with the groups and the mesh size on every rank (it must be deterministic); its
        # answer is checked before anything is built
        answer = assignment_fn(groups, num_ranks=W)
        if isinstance(answer, MatrixAssignment):
            # block counts of a MatrixAssignment follow each group's eligible ranks (all ranks unless the spec says otherwise)
            eligible = {m.fqn: (m.eligible_ranks or tuple(range(W))) for g in groups for m in g}
            owners = dict(answer.rank_by_matrix)
            for name, counts in answer.blocks_per_rank_by_group.items():
                ranks = eligible.get(name, tuple(range(W)))
                if len(counts) != len(ranks):
                    raise ValueError(f"block group {name!r} needs one count per eligible rank ({len(ranks)}), got {counts!r}")
                full = [0] * W
                for r, c in zip(ranks, counts):
                    full[r] = c
                owners[name] = tuple(full)
        else:
            owners = dict(answer)
        validate_assignment(groups, W, owners)
    else:
        owners = assign_matrices(groups, W, ranks_per_host=ranks_per_host, carry_loads=carry_loads)

    def block_fn(named_in, mesh_in):
        res = {}
        for n, p in named_in:
            o = owners.get(n)
            if o is None:
                res[n] = MixedBucketPlacement(Shard(0))
            elif isinstance(o, tuple):
                res[n] = MixedBucketPlacement(BlockShard(o, 0))
            else:
                res[n] = MixedBucketPlacement(BucketedOwned(((o, 0, p.shape[0]),)))
        return res

    kw = dict(mesh=mesh, mp_policy=mp, gradient_reduce_op=dist.ReduceOp.SUM)
    specs = []
    if initial:
        specs.append(BucketSpec(tuple(initial), placement_fn=shard_placement_fn(0), **kw))
    for pats in blocks:
        specs.append(BucketSpec(tuple(pats), placement_fn=block_fn, **kw))
    if final:
        specs.append(BucketSpec(tuple(final), placement_fn=shard_placement_fn(0), reshard_after_forward=False, **kw))
    return specs
