"""The multi-GPU path's host logic on CPU: two gloo ranks run the same sharding and exchange code as the GPU
job (herbert-metal-bf16_b200/dist.py), with the oracle standing in for the kernels. Checks: the tensor-parallel
FFN equals the two-way split sum exactly and the unsplit product within the contract; the expert-parallel MoE
block equals the one-rank block bit for bit, and the concatenation of the ranks' sorted lists is the one-rank
sort (the permutation contract)."""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)


def load_dist():
    spec = importlib.util.spec_from_file_location("hb200_dist", os.path.join(ROOT, "herbert-metal-bf16_b200", "dist.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def t16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def n16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


class OracleBackend:
    """dist.py's backend interface on CPU tensors, computed by the oracle."""

    def __init__(self):
        from oracle_lib import Oracle

        self.o = Oracle()

    def gemm(self, x, w, out, y=None):
        r = self.o.gemm_f64(n16(x), n16(w), out)
        return torch.from_numpy(r) if out == 1 else t16(r)

    def epilogue(self, acc, y, out):
        a = acc.numpy()
        b = a.view(np.uint32)
        r16 = ((b.astype(np.uint64) + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
        if out == 2:
            s = ((n16(y).astype(np.uint32) << 16).view(np.float32) + (r16.astype(np.uint32) << 16).view(np.float32)).astype(np.float32)
            sb = s.view(np.uint32)
            r16 = ((sb.astype(np.uint64) + 0x7FFF + ((sb >> 16) & 1)) >> 16).astype(np.uint16)
        y.copy_(t16(r16))
        return y

    def route(self, scores, top_k):
        return torch.from_numpy(self.o.route_topk(n16(scores), top_k).view(np.int32))

    def sort(self, route, experts, top_k, bm):
        lst, tiles = self.o.moe_sort(np.ascontiguousarray(route.numpy()).view(np.uint32), experts, top_k, bm)
        return torch.from_numpy(lst.view(np.int32)), torch.from_numpy(tiles.view(np.int32))

    def gather(self, x, lst, top_k):
        return x[(lst.long() // top_k)].contiguous()

    def expert_ffn(self, rows, wgu, wd, lst, tiles, experts, mi, h, bm):
        l, t = lst.numpy().view(np.uint32), tiles.numpy().view(np.uint32)
        ehb = self.o.swiglu_slots(self.o.moe_gate_up(n16(rows), n16(wgu), l, t, mi, 1))
        return t16(self.o.moe_down(ehb, n16(wd), l, t, h))

    def combine(self, ey, route, top_k):
        return t16(self.o.moe_combine(n16(ey), np.ascontiguousarray(route.numpy()).view(np.uint32), top_k))


def _worker(rank, world, port, case, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = load_dist()
        be = OracleBackend()
        o = be.o
        if case == "tp":
            m, h, inter = 24, 64, 96
            x = t16(o.normal((m, h), 1, 1, 1.0))
            wgu = t16(o.normal((2 * inter, h), 2, 2, h**-0.5))
            wd = t16(o.normal((h, inter), 3, 3, inter**-0.5))
            y0 = t16(o.normal((m, h), 4, 4, 1.0))
            y = d.tp_ffn(be, x, d.shard_gate_up(wgu, rank, world), d.shard_down(wd, rank, world), y0.clone())
            q.put((rank, n16(y)))
        else:
            m, h, mi, E, top_k, bm = 32, 64, 32, 32, 4, 16
            x = o.normal((m, h), 1, 1, 1.0)
            scores = o.normal((m, E), 4, 4, 1.0)
            wgu = o.normal((E * 2 * mi, h), 2, 2, h**-0.5)
            wd = o.normal((E * h, mi), 3, 3, mi**-0.5)
            rl, epr = m // world, E // world
            dbg = {}
            out = d.ep_moe(be, t16(x[rank * rl : (rank + 1) * rl]), t16(scores[rank * rl : (rank + 1) * rl]), t16(wgu[rank * epr * 2 * mi : (rank + 1) * epr * 2 * mi]),
                           t16(wd[rank * epr * h : (rank + 1) * epr * h]), E, top_k, mi, bm, debug=dbg)
            # the global pair id of every pair this rank received, in its local sorted order
            gathered = [None] * world
            dist.all_gather_object(gathered, (dbg["send_order"].numpy().astype(np.int64) + rank * rl * top_k, dbg["send_counts"]))
            recv_ids = []
            for src, (order, counts) in enumerate(gathered):
                off = int(sum(counts[:rank]))
                recv_ids.append(order[off : off + counts[rank]])
            recv_ids = np.concatenate(recv_ids)
            q.put((rank, n16(out), recv_ids[dbg["local_list"].numpy().astype(np.int64)]))
    finally:
        dist.destroy_process_group()


def _run(case, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    return sorted(res, key=lambda r: r[0])


def test_shards_cover_the_matrices():
    d = load_dist()
    wgu = torch.arange(2 * 12 * 3, dtype=torch.float32).reshape(24, 3)
    parts = [d.shard_gate_up(wgu, r, 4) for r in range(4)]
    assert all(p.shape == (6, 3) for p in parts)
    assert torch.equal(torch.cat([p[:3] for p in parts]), wgu[:12]) and torch.equal(torch.cat([p[3:] for p in parts]), wgu[12:])
    wd = torch.arange(5 * 8, dtype=torch.float32).reshape(5, 8)
    assert torch.equal(torch.cat([d.shard_down(wd, r, 2) for r in range(2)], dim=1), wd)
    with pytest.raises(AssertionError):
        d.shard_gate_up(wgu, 0, 5)


def test_tp_ffn_two_ranks(oracle):
    res = _run("tp")
    assert np.array_equal(res[0][1], res[1][1])  # every rank ends with the same rows
    m, h, inter = 24, 64, 96
    x, wgu, wd, y0 = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((2 * inter, h), 2, 2, h**-0.5), oracle.normal((h, inter), 3, 3, inter**-0.5), oracle.normal((m, h), 4, 4, 1.0)
    hmid = oracle.gemm_f64(x, wgu, 3)
    # exact: the f32 partials of the two K halves, added, rounded once, residual added
    ip = inter // 2
    acc = sum(oracle.gemm_f64(np.ascontiguousarray(hmid[:, r * ip : (r + 1) * ip]), np.ascontiguousarray(wd[:, r * ip : (r + 1) * ip]), 1) for r in range(2))
    be = OracleBackend()
    want = n16(be.epilogue(torch.from_numpy(acc.astype(np.float32)), t16(y0).clone(), 2))
    assert np.array_equal(res[0][1], want)
    # and within the contract of the unsplit product
    c = oracle.compare(oracle.gemm_f64(hmid, wd, 2, y0), res[0][1])
    assert c.over_1ulp <= 1e-3 * c.count + 1 and c.max_abs_err <= c.max_abs_ref / 64


def test_ep_moe_two_ranks_equals_one_rank(oracle):
    res = _run("ep")
    m, h, mi, E, top_k, bm = 32, 64, 32, 32, 4, 16
    x, scores = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((m, E), 4, 4, 1.0)
    wgu, wd = oracle.normal((E * 2 * mi, h), 2, 2, h**-0.5), oracle.normal((E * h, mi), 3, 3, mi**-0.5)
    route = oracle.route_topk(scores, top_k)
    lst, tiles = oracle.moe_sort(route, E, top_k, bm)
    ey = oracle.moe_down(oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, lst, tiles, mi, top_k)), wd, lst, tiles, h)
    want = oracle.moe_combine(ey, route, top_k)
    got = np.concatenate([r[1] for r in res])
    assert np.array_equal(got, want)
    # the permutation contract: rank 0's sorted pairs followed by rank 1's are the one-rank sorted list
    assert np.array_equal(np.concatenate([r[2] for r in res]), lst.astype(np.int64))


def test_ep_moe_single_process_path(oracle):
    # world size 1 (no process group): the same function is the plain block
    d = load_dist()
    be = OracleBackend()
    m, h, mi, E, top_k = 16, 32, 16, 32, 2
    x, scores = oracle.normal((m, h), 1, 1, 1.0), oracle.normal((m, E), 4, 4, 1.0)
    wgu, wd = oracle.normal((E * 2 * mi, h), 2, 2, h**-0.5), oracle.normal((E * h, mi), 3, 3, mi**-0.5)
    out = n16(d.ep_moe(be, t16(x), t16(scores), t16(wgu), t16(wd), E, top_k, mi, 16))
    route = oracle.route_topk(scores, top_k)
    lst, tiles = oracle.moe_sort(route, E, top_k, 16)
    ey = oracle.moe_down(oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, lst, tiles, mi, top_k)), wd, lst, tiles, h)
    assert np.array_equal(out, oracle.moe_combine(ey, route, top_k))
