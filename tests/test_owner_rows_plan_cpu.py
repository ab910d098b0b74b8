"""The chunk plan of the owner-rows transport on faked host layouts (pure planning, no process group): every
element lands once, moves inside one host need no relay, cross-host moves name a relay on the receiving host,
hosts of different sizes, rows that span several hosts, the buffer bound, the automatic fallback.
Parity: the behaviours pinned by the reference's ``tests/test_owner_rows_transport.py:134-257``."""
import pytest


def _cover(plan, lens):
    W = len(lens)
    seen = [0] * (plan.chunk * W)
    src_seen = [[0] * n for n in lens]
    for m in plan.moves:
        assert 0 <= m.dst < W and 0 <= m.dst_off and m.dst_off + m.length <= plan.chunk
        for i in range(m.length):
            seen[m.dst * plan.chunk + m.dst_off + i] += 1
            src_seen[m.src][m.src_off + i] += 1
    assert max(seen, default=0) <= 1 and sum(seen) == sum(lens)
    assert all(all(v == 1 for v in row) for row in src_seen)          # every owner element leaves exactly once
    return seen


def test_one_host_moves_inside_it():
    from flex_shard_b200.placements.owner_rows_transport import plan_chunks

    lens = [4096, 0, 1024, 512, 0, 0, 2048, 128]
    plan = plan_chunks(lens)                                          # no hosts given: one NVSwitch domain
    _cover(plan, lens)
    assert plan.cross_host_elems == 0 and plan.crossing_fraction == 0.0
    assert all(m.via == -1 for m in plan.moves)
    assert plan.buffer_elems == plan.chunk                            # no relay share on top of the chunk


def test_chunks_are_equal_and_aligned():
    from flex_shard_b200.placements.owner_rows_transport import plan_chunks

    for lens in ([1, 1, 1, 1], [1000, 0, 0, 0], [129, 127, 255, 1], [0, 0, 0, 0]):
        plan = plan_chunks(lens)
        assert plan.chunk % 128 == 0 and plan.chunk * len(lens) >= sum(lens)
        _cover(plan, lens)


def test_owner_keeps_the_part_of_its_row_that_falls_in_its_own_chunk():
    from flex_shard_b200.placements.owner_rows_transport import plan_chunks

    lens = [512, 512, 512, 512]                                       # every row is exactly its owner's chunk
    plan = plan_chunks(lens, hosts=[0, 0, 1, 1])
    assert plan.chunk == 512
    assert [(m.src, m.dst, m.src_off, m.dst_off, m.length) for m in plan.moves] == [(r, r, 0, 0, 512) for r in range(4)]
    assert plan.cross_host_elems == 0


def test_row_spanning_several_hosts_is_cut_at_chunk_borders():
    from flex_shard_b200.placements.owner_rows_transport import plan_chunks

    lens = [0, 0, 4096, 0, 0, 0]                                      # one owner (on host 1) feeds every chunk
    hosts = [0, 0, 1, 1, 2, 2]
    plan = plan_chunks(lens, hosts)
    _cover(plan, lens)
    dsts = [m.dst for m in plan.moves]
    assert dsts == sorted(dsts) and set(dsts) == {0, 1, 2, 3, 4, 5}
    off = 0
    for m in plan.moves:                                              # consecutive slices of the owner's row
        assert m.src == 2 and m.src_off == off
        off += m.length
    cross = [m for m in plan.moves if hosts[m.dst] != 1]
    assert all(m.via >= 0 and hosts[m.via] == hosts[m.dst] for m in cross)     # relays sit on the receiving host
    assert all(m.via == -1 for m in plan.moves if hosts[m.dst] == 1)
    assert plan.cross_host_elems == sum(m.length for m in cross)


def test_hosts_of_different_sizes():
    from flex_shard_b200.placements.owner_rows_transport import plan_chunks

    lens = [300, 300, 300, 300, 300]
    hosts = [0, 0, 0, 1, 1]
    plan = plan_chunks(lens, hosts)
    _cover(plan, lens)
    for m in plan.moves:
        if hosts[m.src] != hosts[m.dst]:
            assert hosts[m.via] == hosts[m.dst]
    # rails between two hosts = the smaller host's rank count: at most 2 distinct relays towards host 0
    relays_to_0 = {m.via for m in plan.moves if hosts[m.src] == 1 and hosts[m.dst] == 0}
    assert len(relays_to_0) <= 2


def test_moe_stage_on_eight_hosts_stays_within_the_buffer_bound():
    """64 ranks on 8 hosts, experts' rows on every fourth rank: the transport buffer is the chunk plus the largest
    relay share, and the crossing fraction decides the transport."""
    from flex_shard_b200.placements.owner_rows_transport import choose_transport, plan_chunks

    W = 64
    hosts = [r // 8 for r in range(W)]
    lens = [(1 << 20) if r % 4 == 0 else 0 for r in range(W)]
    plan = plan_chunks(lens, hosts)
    assert plan.total_elems == 16 << 20 and plan.chunk == (16 << 20) // W
    assert plan.chunk <= plan.buffer_elems <= 2 * plan.chunk + 128
    moved = sum(m.length for m in plan.moves)
    assert moved == plan.total_elems
    # each owner's row covers four consecutive chunks starting at its own: all inside its host
    assert plan.cross_host_elems == 0 and choose_transport(plan) == "chunks"
    # the same rows bunched on one host cross hosts for 7/8 of the bucket: grouped collectives win
    lens2 = [(2 << 20) if r < 8 else 0 for r in range(W)]
    plan2 = plan_chunks(lens2, hosts)
    assert abs(plan2.crossing_fraction - 7 / 8) < 1e-6 and choose_transport(plan2) == "grouped"


def test_transport_switch_rejects_unknown_modes(monkeypatch):
    from flex_shard_b200.placements.owner_rows_transport import ChunkPlan, choose_transport

    monkeypatch.setenv("FLEX_SHARD_OWNER_ROWS_TRANSPORT", "fastest")
    with pytest.raises(ValueError, match="auto, chunks or grouped"):
        choose_transport(ChunkPlan(chunk=128))
    monkeypatch.setenv("FLEX_SHARD_OWNER_ROWS_TRANSPORT", "grouped")
    assert choose_transport(ChunkPlan(chunk=128)) == "grouped"
