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
    st.connect(local_peers=[st])
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


def test_one_rank_matches_the_plain_block(env, hb200, oracle):
    d, ctx = env
    s = SHAPE
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    st, out = single_gpu_block(hb200, ctx, d, xt, st_, wgut, wdt, **s)
    torch.cuda.synchronize()
    route = oracle.route_topk(scores, s["top_k"])
    lst, tiles = oracle.moe_sort(route, s["E"], s["top_k"], s["bm"])
    assert np.array_equal(st.route.cpu().numpy().view(np.uint32), route)
    assert np.array_equal(st.list.cpu().numpy().view(np.uint32), lst)
    counts = np.bincount(route[:, : s["top_k"]].reshape(-1), minlength=s["E"])
    assert np.array_equal(st.offs.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
    # one rank: the receive buffer holds the pairs in sorted order, so the plan's list is the identity
    n = int(tiles[0])
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


@pytest.mark.parametrize("world", [2, 4])
def test_emulated_ranks_equal_one_rank(env, hb200, oracle, world):
    d, ctx = env
    s = SHAPE
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    _, want = single_gpu_block(hb200, ctx, d, xt, st_, wgut, wdt, **s)
    want = want.clone()
    rpr, epr = s["m"] // world, s["E"] // world
    ranks = [d.EpPeer(hb200, ctx, r, world, rpr, s["h"], s["mi"], s["E"], s["top_k"], s["bm"]) for r in range(world)]
    for st in ranks:
        st.connect(local_peers=ranks)
    for rep in range(2):  # twice: the buffers carry the previous call's rows
        for r, st in enumerate(ranks):
            st.phase_sort(xt[r * rpr : (r + 1) * rpr].contiguous(), st_[r * rpr : (r + 1) * rpr].contiguous())
        offs_all = torch.stack([st.offs for st in ranks])
        for st in ranks:
            st.offs_all.copy_(offs_all)
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
        lst, tiles = d.ep_plan_np(oa, r, epr, s["bm"])
        assert np.array_equal(st.rlist.cpu().numpy()[: len(lst)].astype(np.uint32), lst)
        assert np.array_equal(st.rtiles.cpu().numpy().view(np.uint32)[: len(tiles)], tiles)


def test_receive_buffer_too_small_is_reported_not_overrun(env, hb200, oracle):
    d, ctx = env
    s = dict(SHAPE)
    x, scores, wgu, wd = inputs(oracle, **s)
    xt, st_, wgut, wdt = (t16(a).cuda() for a in (x, scores, wgu, wd))
    pairs = s["m"] * s["top_k"]
    st = d.EpPeer(hb200, ctx, 0, 1, s["m"], s["h"], s["mi"], s["E"], s["top_k"], s["bm"], cap=pairs - 64)
    st.connect(local_peers=[st])
    guard = torch.full((4096,), 0x5A5A, device="cuda", dtype=torch.int16)  # lives right after nothing in particular: a canary of our own
    d.ep_moe_peer(st, xt, st_, wgut, wdt)
    torch.cuda.synchronize()
    with pytest.raises(hb200.HbError) as e:
        ctx.sync()
    assert e.value.status == hb200.KERNEL and "does not fit" in e.value.message
    assert int(st.rtiles[0]) == 0  # the plan published an empty table: the GEMMs did nothing
    assert bool((guard == 0x5A5A).all())
    ctx.sync()  # the status was cleared: the context is usable again


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
        one.connect(local_peers=[one])
        want = d.ep_moe_peer(one, xt, st_, wgut, wdt).clone()
        rpr, epr = s["m"] // world, s["E"] // world
        st = d.EpPeer(hb, ctx, rank, world, rpr, s["h"], s["mi"], s["E"], s["top_k"], s["bm"])
        d.ep_peer_connect(st)
        for _ in range(3):
            out = d.ep_moe_peer(st, xt[rank * rpr : (rank + 1) * rpr].contiguous(), st_[rank * rpr : (rank + 1) * rpr].contiguous(),
                                wgut[rank * epr * 2 * s["mi"] : (rank + 1) * epr * 2 * s["mi"]], wdt[rank * epr * s["h"] : (rank + 1) * epr * s["h"]])
            stream.synchronize()
            ok = ok and bool(torch.equal(out, want[rank * rpr : (rank + 1) * rpr]))
        dist.barrier()
        st.close()
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
