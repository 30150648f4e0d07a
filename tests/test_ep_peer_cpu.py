"""The peer-memory expert-parallel exchange, host mirror of its index arithmetic (dist.ep_positions_np, ep_plan_np):
for any number of ranks, sending every rank's pairs to the owners of their experts and laying them out as the
dispatch and plan kernels do must give, rank after rank, exactly the order of a single GPU's sort over all pairs
(the permutation contract of the sharded MoE block)."""
import numpy as np
import pytest

from oracle_lib import Oracle
from test_dist_cpu import load_dist


def offsets_of(route, experts, top_k):
    counts = np.bincount(route[:, :top_k].reshape(-1), minlength=experts)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)


@pytest.mark.parametrize("direct", [False, True], ids=["packed", "direct"])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("rows,experts,top_k,bm", [(64, 32, 4, 16), (96, 64, 8, 32), (40, 8, 2, 64)])
def test_exchange_reproduces_the_single_sort(world, rows, experts, top_k, bm, direct):
    # packed: a source's rows follow those of the sources before it (needs everybody's counts: the all-gather);
    # direct: every source has its own region of every receive buffer
    if experts % world or rows % world:
        pytest.skip("does not divide")
    d, o = load_dist(), Oracle()
    scores = o.normal((rows, experts), 11, 4, 1.0)
    route = o.route_topk(scores, top_k)
    want_list, want_tiles = o.moe_sort(route, experts, top_k, bm)
    epr, rpr = experts // world, rows // world
    # every rank sorts its own rows by global expert
    lists, offs = [], []
    for r in range(world):
        rt = np.ascontiguousarray(route[r * rpr : (r + 1) * rpr])
        lst, _ = o.moe_sort(rt, experts, top_k, bm)
        lists.append(lst)
        offs.append(offsets_of(rt, experts, top_k))
    offs_all = np.stack(offs)
    # dispatch: the global pair id of what lands in every receive-buffer row
    cap = rows * top_k
    region = cap // world if direct else 0
    recv = [np.full(cap, -1, dtype=np.int64) for _ in range(world)]
    for r in range(world):
        dest, row = d.ep_positions_np(offs_all, r, epr, region)
        assert not direct or ((row >= r * region) & (row < (r + 1) * region)).all()
        assert len(dest) == rpr * top_k
        for p in range(len(dest)):
            assert recv[dest[p]][row[p]] == -1, "two pairs in one receive row"
            recv[dest[p]][row[p]] = r * rpr * top_k + int(lists[r][p])
            assert route[(r * rpr * top_k + int(lists[r][p])) // top_k, int(lists[r][p]) % top_k] // epr == dest[p]
    # plan: the owners' lists, mapped back to global pair ids and concatenated, are the single sort
    got, tiles_rows = [], []
    for r in range(world):
        lst, tiles = d.ep_plan_np(offs_all, r, epr, bm, region)
        n_recv = int((recv[r] >= 0).sum())
        assert len(lst) == n_recv and sorted(lst.tolist()) == np.flatnonzero(recv[r] >= 0).tolist()
        got.extend(recv[r][lst].tolist())
        for t in range(int(tiles[0])):
            e, first, n = (int(v) for v in tiles[1 + 3 * t : 4 + 3 * t])
            tiles_rows.append((r * epr + e, len(got) - n_recv + first, n))
    assert np.array_equal(np.array(got, dtype=np.uint32), want_list)
    # and so are the tile tables, once the local expert ids and row offsets are made global
    want = [tuple(int(v) for v in want_tiles[1 + 3 * t : 4 + 3 * t]) for t in range(int(want_tiles[0]))]
    assert tiles_rows == want


def test_recorded_step_is_taken_down_once_and_replayed():
    """dist._Recorded: the first run of a key collects the step's kernel calls from every emitter and records them;
    later runs only tell the step to advance its own state (replay=True) and launch the recording."""
    d = load_dist()

    class FakeGraph:
        def __init__(self, ops):
            self.ops, self.launched, self.freed = list(ops), 0, False

        def launch(self):
            self.launched += 1

        def free(self):
            self.freed = True

    class FakeCtx:
        def __init__(self):
            self.recorded = []

        def record(self, ops):
            g = FakeGraph(ops)
            self.recorded.append(g)
            return g

    class Emitter:
        emit = staticmethod(d._launch_now)

    launched_directly = []
    kernel = lambda m, *ranges: launched_directly.append((m, ranges))
    a, b, ctx = Emitter(), Emitter(), FakeCtx()
    rec = d._Recorded(ctx, a, b)
    state = {"parity": 0, "replays": 0}

    def step(replay=False):
        state["parity"] ^= 1
        if replay:
            state["replays"] += 1
            return
        a.emit(kernel, 7, "x")
        b.emit(kernel, 1, "flags")
        a.emit(kernel, 7, "y")

    for call in range(4):
        rec.run(("key", state["parity"] ^ 1), step)
    assert launched_directly == []                       # nothing was launched kernel by kernel
    assert len(ctx.recorded) == 2                        # one recording per parity
    assert [op[1:] for op in ctx.recorded[0].ops] == [(7, "x"), (1, "flags"), (7, "y")]
    assert [g.launched for g in ctx.recorded] == [2, 2] and state["replays"] == 2
    assert a.emit is d._launch_now and b.emit is d._launch_now  # the emitters launch again once the step is recorded
    a.emit(kernel, 3, "z")
    assert launched_directly == [(3, ("z",))]
    rec.close()
    assert all(g.freed for g in ctx.recorded) and rec.graphs == {}
