"""The sharded paths' GPU backend on one GPU (world size 1: the same code as the multi-GPU job minus the
exchange), checked against the oracle; the two-rank exchange logic itself is covered on CPU (test_dist_cpu.py)."""
import numpy as np
import pytest
import torch

from gpu_util import within_contract
from test_dist_cpu import load_dist, n16, t16

pytestmark = pytest.mark.gpu


@pytest.fixture()
def backend(hb200):
    d = load_dist()
    ctx = hb200.Context(0)
    stream = torch.cuda.Stream()
    ctx.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        yield d, d.GpuBackend(hb200, ctx, rows_max=512)
    stream.synchronize()
    ctx.close()


def test_tp_ffn_one_rank_and_split_sum(backend, oracle):
    d, be = backend
    m, h, inter = 96, 256, 384
    x, wgu, wd, y0 = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((2 * inter, h), 2, 2, h**-0.5), oracle.normal((h, inter), 3, 3, inter**-0.5), oracle.normal((m, h), 4, 4, 1.0)
    y = d.tp_ffn(be, t16(x).cuda(), t16(wgu).cuda(), t16(wd).cuda(), t16(y0).cuda())
    torch.cuda.synchronize()
    hmid = oracle.gemm_f64(x, wgu, 3)
    within_contract(oracle, oracle.gemm_f64(hmid, wd, 2, y0), n16(y.cpu()), "FFN, one rank")
    # the two shards of a 2-way split, summed in f32 on the device as the all-reduce would, then the epilogue
    xs = t16(x).cuda()
    acc = None
    for r in range(2):
        h_r = be.gemm(xs, d.shard_gate_up(t16(wgu), r, 2).cuda(), 3)
        a_r = be.gemm(h_r, d.shard_down(t16(wd), r, 2).cuda(), 1)
        acc = a_r if acc is None else acc + a_r
    y2 = be.epilogue(acc, t16(y0).cuda(), 2)
    torch.cuda.synchronize()
    within_contract(oracle, oracle.gemm_f64(hmid, wd, 2, y0), n16(y2.cpu()), "FFN, two shards summed")


def test_ep_moe_one_rank(backend, oracle):
    d, be = backend
    m, h, mi, E, top_k, bm = 128, 256, 128, 32, 4, 32
    x, scores = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((m, E), 4, 4, 1.0)
    wgu, wd = oracle.normal((E * 2 * mi, h), 2, 2, h**-0.5), oracle.normal((E * h, mi), 3, 3, mi**-0.5)
    dbg = {}
    out = d.ep_moe(be, t16(x).cuda(), t16(scores).cuda(), t16(wgu).cuda(), t16(wd).cuda(), E, top_k, mi, bm, debug=dbg)
    torch.cuda.synchronize()
    route = oracle.route_topk(scores, top_k)
    assert np.array_equal(dbg["route"].cpu().numpy().view(np.uint32), route)
    lst, tiles = oracle.moe_sort(route, E, top_k, bm)
    # one rank: the send order is the identity grouping, the local list over received pairs is the block's sort
    assert np.array_equal(dbg["send_order"].cpu().numpy()[dbg["local_list"].cpu().numpy()].astype(np.uint32), lst)
    ey = oracle.moe_down(oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, lst, tiles, mi, top_k)), wd, lst, tiles, h)
    c = oracle.compare(oracle.moe_combine(ey, route, top_k), n16(out.cpu()))
    assert c.max_abs_err <= c.max_abs_ref / 64 and c.over_1ulp <= 0.05 * c.count
