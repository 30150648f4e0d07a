"""The peer-memory expert-parallel MoE block (dist.EpPeer, ep_dispatch / ep_plan / ep_return kernels).

On one GPU the ranks are emulated in one process: every rank has its own buffers, the "peer" tables point at the
other ranks' buffers on the same GPU, and the phases run rank after rank where the multi-GPU job has its
collectives. No kernel of the path waits for another rank, so this runs the very kernels of the multi-GPU job.
The result must equal, bit for bit, the single-GPU block over all rows (the per-row arithmetic does not depend on
which rows share a run). With two or more GPUs the same block also runs as one process per GPU over NVLink.
"""
import os
import sys

import numpy as np
import pytest
import torch

from gpu_util import within_contract
from test_dist_cpu import load_dist, n16, t16

pytestmark = pytest.mark.gpu

SHAPE = dict(m=256, h=256, mi=128, E=32, top_k=4, bm=16)


def inputs(oracle, m, h, mi, E, **_):
    x, scores = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((m, E), 4, 4, 1.0)
    wgu, wd = oracle.normal((E * 2 * mi, h), 2, 2, h**-0.5), oracle.normal((E * h, mi), 3, 3, mi**-0.5)
    return x, scores, wgu, wd


def single_gpu_block(hb200, ctx, d, x, scores, wgu, wd, m, h, mi, E, top_k, bm):
    st = d.EpPeer(hb200, ctx, 0, 1, m, h, mi, E, top_k, bm)
    st.connect([st])
    out = d.ep_moe_peer(st, x, scores, wgu, wd)
    return st, out


@pytest.fixture()
def env(hb200):
    d = load_dist()
    ctx = hb200.Context(0)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        yield d, ctx
    stream.synchronize()
    ctx.close()


@pytest.mark.parametrize("fused", [True, False])
def test_one_rank_matches_the_plain_block(env, hb200, oracle, fused):
    # the exchange kernels with a single rank (dispatch into its own receive buffer, plan, return or the fused combine)
    d, ctx = env
    s = SHAPE
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    st = d.EpPeer(hb200, ctx, 0, 1, s["m"], s["h"], s["mi"], s["E"], s["top_k"], s["bm"], fused=fused, plain_when_alone=False)
    st.connect([st])
    out = d.ep_moe_peer(st, xt, st_, wgut, wdt)
    torch.cuda.synchronize()
    plain, out_plain = single_gpu_block(hb200, ctx, d, xt, st_, wgut, wdt, **s)  # one rank as the library runs it: no exchange
    torch.cuda.synchronize()
    assert plain.plain and torch.equal(out_plain, out)
    route = oracle.route_topk(scores, s["top_k"])
    lst, tiles = oracle.moe_sort(route, s["E"], s["top_k"], s["bm"])
    assert np.array_equal(st.route.cpu().numpy().view(np.uint32), route)
    assert np.array_equal(st.list.cpu().numpy().view(np.uint32), lst)
    counts = np.bincount(route[:, : s["top_k"]].reshape(-1), minlength=s["E"])
    assert np.array_equal(st.offs.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
    # one rank: the receive buffer holds the pairs in sorted order, so the plan's list is the identity
    n = int(tiles[0])
    assert st.direct == fused
    assert np.array_equal(st.rlist.cpu().numpy()[: len(lst)], np.arange(len(lst)))
    assert np.array_equal(st.rtiles.cpu().numpy().view(np.uint32)[: 1 + 3 * n], tiles[: 1 + 3 * n])
    # against the plain block of kernels (route, sort, gather GEMM, scatter GEMM, combine) on the same inputs
    pairs = s["m"] * s["top_k"]
    ehb = torch.zeros(pairs, s["mi"], device="cuda", dtype=torch.bfloat16)
    ey = torch.zeros(pairs, s["h"], device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros(s["m"], s["h"], device="cuda", dtype=torch.bfloat16)
    w = st._w
    kw = dict(rows_max=s["m"], top_k=s["top_k"], experts=s["E"], bm=s["bm"], merge_runs=1)
    ctx.gemm(s["h"], 2 * s["mi"], 3, rows_mode=hb200.ROWS_GATHER, **kw)(s["m"], w(wgut), w(xt), w(ehb), w(st.list), w(st.tiles))
    ctx.gemm(s["mi"], s["h"], 0, rows_mode=hb200.ROWS_SCATTER, **kw)(s["m"], w(wdt), w(ehb), w(ey), w(st.list), w(st.tiles))
    ctx.moe_combine(s["h"], s["top_k"])(s["m"], w(ey), w(st.route), w(out2))
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    # and the oracle, stage by stage tolerance as for the plain block
    ey_o = oracle.moe_down(oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, lst, tiles, s["mi"], s["top_k"])), wd, lst, tiles, s["h"])
    c = oracle.compare(oracle.moe_combine(ey_o, route, s["top_k"]), n16(out.cpu()))
    assert c.max_abs_err <= c.max_abs_ref / 64 and c.over_1ulp <= 0.05 * c.count


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_equal_one_rank(env, hb200, oracle, world, fused):
    d, ctx = env
    s = SHAPE
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    _, want = single_gpu_block(hb200, ctx, d, xt, st_, wgut, wdt, **s)
    want = want.clone()
    rpr, epr = s["m"] // world, s["E"] // world
    ranks = [d.EpPeer(hb200, ctx, r, world, rpr, s["h"], s["mi"], s["E"], s["top_k"], s["bm"], fused=fused) for r in range(world)]
    for st in ranks:
        st.connect(ranks)
    for rep in range(3):  # twice: the buffers carry the previous call's rows
        for r, st in enumerate(ranks):
            st.phase_sort(xt[r * rpr : (r + 1) * rpr].contiguous(), st_[r * rpr : (r + 1) * rpr].contiguous())
        offs_all = torch.stack([st.offs for st in ranks])
        for st in ranks:
            st.offs_all.copy_(offs_all)  # what the all-gather step of the multi-GPU job delivers
        for st in ranks:
            st.phase_dispatch()
        for r, st in enumerate(ranks):
            st.phase_experts(wgut[r * epr * 2 * s["mi"] : (r + 1) * epr * 2 * s["mi"]], wdt[r * epr * s["h"] : (r + 1) * epr * s["h"]])
        outs = [st.phase_return() for st in ranks]
        torch.cuda.synchronize()
        ctx.sync()
        assert torch.equal(torch.cat(outs), want), f"pass {rep}"
    # the device plan equals its host mirror
    oa = offs_all.cpu().numpy()
    for r, st in enumerate(ranks):
        lst, tiles = d.ep_plan_np(oa, r, epr, s["bm"], region=st.cap // world if st.direct else 0)
        assert np.array_equal(st.rlist.cpu().numpy()[: len(lst)].astype(np.uint32), lst)
        assert np.array_equal(st.rtiles.cpu().numpy().view(np.uint32)[: len(tiles)], tiles)


def test_receive_buffer_too_small_is_reported_not_overrun(env, hb200, oracle):
    d, ctx = env
    s = dict(SHAPE)
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    pairs = s["m"] * s["top_k"]
    st = d.EpPeer(hb200, ctx, 0, 1, s["m"], s["h"], s["mi"], s["E"], s["top_k"], s["bm"], cap=pairs - 64, plain_when_alone=False)
    st.connect([st])
    guard = torch.full((4096,), 0x5A5A, device="cuda", dtype=torch.int16)  # lives right after nothing in particular: a canary of our own
    d.ep_moe_peer(st, xt, st_, wgut, wdt)
    torch.cuda.synchronize()
    with pytest.raises(hb200.HbError) as e:
        ctx.sync()
    assert e.value.status == hb200.KERNEL and "does not fit" in e.value.message
    assert int(st.rtiles[0]) == 0  # the plan published an empty table: the GEMMs did nothing
    assert bool((guard == 0x5A5A).all())
    ctx.sync()  # the status was cleared: the context is usable again


def test_barrier_gives_up_on_a_rank_that_never_arrives(hb200):
    # a two-rank barrier whose "peer" is a spare flag array on this GPU that nothing ever sets: the wait runs out
    # (100 ms here), the kernel returns, the context reports it and stays usable
    ctx = hb200.Context(0)
    try:
        ctx.set_peer_wait_ms(100)
        mine, spare = ctx.alloc(256), ctx.alloc(256)
        table = ctx.to_device(np.array([mine.ptr, spare.ptr], dtype=np.uint64))
        ctx.peer_sync(0, 2, 0)(1, table)
        with pytest.raises(hb200.HbError) as e:
            ctx.sync()
        assert e.value.status == hb200.KERNEL and "gave up waiting at point 5" in e.value.message
        assert spare.download(np.uint32, (2,))[0] == 1  # its own arrival was published
        ctx.sync()
        with pytest.raises(hb200.HbError):
            ctx.peer_sync(0, 1, 0)  # one rank has nobody to wait for
    finally:
        ctx.close()


def _two_process_worker(rank, world, port, repo, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, repo)
    sys.path.insert(0, os.path.join(repo, "tests"))
    import torch.distributed as dist
    from __graft_entry__ import load_package
    from oracle_lib import Oracle

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    hb = load_package()
    d = load_dist()
    o = Oracle()
    s = SHAPE
    x, scores, wgu, wd = inputs(o, **s)
    ctx = hb.Context(rank)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    ok = True
    with torch.cuda.stream(stream):
        xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
        one = d.EpPeer(hb, ctx, 0, 1, s["m"], s["h"], s["mi"], s["E"], s["top_k"], s["bm"])
        one.connect([one])
        want = d.ep_moe_peer(one, xt, st_, wgut, wdt).clone()
        rpr, epr = s["m"] // world, s["E"] // world
        xs, ss = xt[rank * rpr : (rank + 1) * rpr].contiguous(), st_[rank * rpr : (rank + 1) * rpr].contiguous()
        wl, dl = wgut[rank * epr * 2 * s["mi"] : (rank + 1) * epr * 2 * s["mi"]], wdt[rank * epr * s["h"] : (rank + 1) * epr * s["h"]]
        for fused in (True, False):  # the dispatch's flag and the combine that reads the owners' rows; barrier kernels and a return into EY
            st = d.EpPeer(hb, ctx, rank, world, rpr, s["h"], s["mi"], s["E"], s["top_k"], s["bm"], fused=fused)
            d.ep_peer_connect(st)
            # the library's barrier kernel launched step by step (0, 1), the step recorded and replayed (2..6: both
            # parities recorded, then replayed), then the NCCL form of the same steps
            for it in range(9):
                out = d.ep_moe_peer(st, xs, ss, wl, dl, nccl_sync=it >= 7, recorded=2 <= it < 7)
                stream.synchronize()
                ctx.sync()
                same = bool(torch.equal(out, want[rank * rpr : (rank + 1) * rpr]))
                if not same:
                    print(f"rank {rank}: MoE block (fused={fused}), step {it}: differs from the one-rank block", file=sys.stderr, flush=True)
                ok = ok and same
            ok = ok and len(st.recorded.graphs) == 2
            dist.barrier()
            st.close()
        # the tensor-parallel FFN: both ranks end with the same Y, equal to the all-reduce form
        m, h, inter = 200, 256, 512
        x2, wgu2, wd2, y0 = o.normal((m, h), 1, 1, 1.0), o.normal((2 * inter, h), 2, 2, h**-0.5), o.normal((h, inter), 3, 3, inter**-0.5), o.normal((m, h), 4, 4, 1.0)
        a, b = d.shard_gate_up(t16(wgu2), rank, world).cuda(), d.shard_down(t16(wd2), rank, world).cuda()
        be = d.GpuBackend(hb, ctx, rows_max=512)
        y_ref = d.tp_ffn(be, t16(x2).cuda(), a, b, t16(y0).cuda())
        # pulled by the summing kernel; pushed by the GEMM (the barriers inside tp_sum, or as kernels of their own); pushed and
        # summed beside the GEMM; pushed in groups with the barriers inside the streaming sum
        for mode, kw in (("pull", {}), ("push", {}), ("push", dict(fold_barriers=False)), ("stream", {}), ("pushsync", {})):
            tp = d.TpPeer(hb, ctx, rank, world, m, h, mode=mode, **kw)
            d.tp_peer_connect(tp)
            x2d = t16(x2).cuda()
            for it in range(6):  # step by step, recorded then replayed (1..4), with NCCL barriers
                tp.set_y(t16(y0).cuda())
                dist.barrier()
                y = d.tp_ffn_peer(tp, x2d, a, b, nccl_sync=it == 5, recorded=1 <= it < 5)
                stream.synchronize()
                ctx.sync()
                same = bool(torch.equal(y, y_ref))
                if not same:
                    print(f"rank {rank}: FFN form {mode}, step {it}: differs from the all-reduce form", file=sys.stderr, flush=True)
                ok = ok and same
                dist.barrier()
            ok = ok and len(tp.recorded.graphs) == 1
            tp.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        result.put(int(flag.item()))
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_nvlink():
    import torch.multiprocessing as mp

    world = 2
    mpc = mp.get_context("spawn")
    result = mpc.Queue()
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = [mpc.Process(target=_two_process_worker, args=(r, world, 29731, repo, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=10) == 1


# ---------------------------------------------------------------- the tensor-parallel FFN through tp_reduce

@pytest.mark.parametrize("mode", ["pull", "push", "stream", "pushsync"])
@pytest.mark.parametrize("world,m", [(1, 200), (2, 200), (4, 200), (8, 200), (4, 700), (8, 1024)])
def test_tp_reduce_emulated_ranks(env, hb200, oracle, world, m, mode):
    # push: the down GEMM stores each block of rows of its partial into its owner's staging buffer (y_shards) and the
    # sum reads local memory; pull: the partial stays whole and the sum fetches the blocks from the peers; stream: the
    # rows dealt in groups of 256, every rank sums a slice of every group (here host-ordered: the ranks share a GPU).
    # Row counts that end inside a group, inside a rank's slice of it, and on a group's edge.
    d, ctx = env
    h, inter = 256, 512
    x, wgu, wd, y0 = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((2 * inter, h), 2, 2, h**-0.5), oracle.normal((h, inter), 3, 3, inter**-0.5), oracle.normal((m, h), 4, 4, 1.0)
    xt = t16(x).cuda()
    ranks = [d.TpPeer(hb200, ctx, r, world, m, h, mode=mode) for r in range(world)]
    assert all(st.mode == (mode if world > 1 else "pull") for st in ranks)
    for st in ranks:
        st.connect(ranks)
        st.set_y(t16(y0).cuda())
    shards = [(d.shard_gate_up(t16(wgu), r, world).cuda(), d.shard_down(t16(wd), r, world).cuda()) for r in range(world)]
    # what the all-reduce form gives: the same GEMM kernels, f32 sum in rank order, then the epilogue kernel
    be = d.GpuBackend(hb200, ctx, rows_max=512)
    acc = None
    for a, b in shards:
        hm = torch.empty(m, a.shape[0] // 2, device="cuda", dtype=torch.bfloat16)
        part = torch.empty(m, h, device="cuda", dtype=torch.float32)
        ctx.gemm(h, a.shape[0], 3, rows_max=m, cta_pair=1)(m, be._w(a), be._w(xt), be._w(hm))
        ctx.gemm(hm.shape[1], h, 1, rows_max=m, cta_pair=1)(m, be._w(b), be._w(hm), be._w(part))
        torch.cuda.synchronize()
        acc = part if acc is None else acc + part
    want = be.epilogue(acc, t16(y0).cuda(), 2)
    for rep in range(2):
        for st in ranks:
            st.set_y(t16(y0).cuda())
        for st, (a, b) in zip(ranks, shards):
            st.phase_gemms(xt, a, b)
        for st in ranks:
            st.phase_reduce()
        torch.cuda.synchronize()
        for st in ranks:
            assert torch.equal(st.y_view(), want), f"rank {st.rank}, pass {rep}"
    hmid = oracle.gemm_f64(x, wgu, 3)
    within_contract(oracle, oracle.gemm_f64(hmid, wd, 2, y0), n16(ranks[0].y_view().cpu()), f"FFN over {world} emulated ranks")


def _cai(ptr, shape, typestr):
    class H:
        pass
    h = H()
    h.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}
    return h
