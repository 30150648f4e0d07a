"""MoE path through the C ABI: route, sort and combine are bit-exact against the oracle (index and
bf16-chain work); the expert GEMMs are held to the GEMM contract. The MoE block at full size (2048 tokens, 256 experts, top-8)."""
import numpy as np
import pytest

from gpu_util import within_contract
from oracle_lib import SEED_ROUTER, SEED_W, SEED_X, SEED_Y

pytestmark = pytest.mark.gpu


def sort_on_gpu(ctx, hb200, route, experts, top_k, bm, rows_max=None):
    m = route.shape[0]
    rows_max = rows_max or m
    nt = hb200.lib().hb_moe_tiles(rows_max, top_k, experts, bm)
    d_r, d_l, d_t = ctx.to_device(route), ctx.alloc(rows_max * top_k * 4), ctx.alloc((1 + 3 * nt) * 4)
    ctx.moe_sort(experts, top_k, rows_max, bm)(m, d_r, d_l, d_t)
    ctx.sync()
    return d_l, d_t, d_l.download(np.uint32, (m * top_k,)), d_t.download(np.uint32, (1 + 3 * nt,))


@pytest.mark.parametrize("rows,experts,top_k", [(1, 32, 1), (7, 64, 4), (33, 256, 8), (300, 1024, 8), (2048, 256, 8)])
def test_route_bit_exact(ctx, oracle, rows, experts, top_k):
    scores = oracle.normal((rows, experts), SEED_ROUTER, 3, 1.0)
    if rows > 1:
        scores[1, :] = scores[1, 0]  # a row of equal scores: the lowest experts win
    d_s, d_r = ctx.to_device(scores), ctx.alloc(rows * 2 * top_k * 4)
    ctx.route(experts, top_k)(rows, d_s, d_r)
    ctx.sync()
    got = d_r.download(np.uint32, (rows, 2 * top_k))
    assert np.array_equal(got, oracle.route_topk(scores, top_k))
    if rows > 1:
        assert list(got[1, :top_k]) == list(range(top_k))


@pytest.mark.parametrize("bm", [16, 32, 64])
@pytest.mark.parametrize("rows,experts,top_k", [(1, 32, 1), (5, 32, 2), (100, 64, 8), (2048, 256, 8), (4096, 256, 8)])
def test_sort_bit_exact(ctx, hb200, oracle, rows, experts, top_k, bm):
    route = oracle.route_topk(oracle.normal((rows, experts), SEED_ROUTER, 3, 1.0), top_k)
    _, _, lst, tiles = sort_on_gpu(ctx, hb200, route, experts, top_k, bm)
    want_l, want_t = oracle.moe_sort(route, experts, top_k, bm)
    n = int(want_t[0])
    assert np.array_equal(lst, want_l)
    assert np.array_equal(tiles[: 1 + 3 * n], want_t[: 1 + 3 * n])


def test_sort_skewed_and_empty_experts(ctx, hb200, oracle):
    # every pair on two experts (many tiles each), all the others empty; and a partial block of a larger kernel
    rows, experts, top_k = 513, 64, 2
    route = np.zeros((rows, 2 * top_k), dtype=np.uint32)
    route[:, 0], route[:, 1] = 5, 63
    for bm in (16, 64):
        _, _, lst, tiles = sort_on_gpu(ctx, hb200, route, experts, top_k, bm, rows_max=2048)
        want_l, want_t = oracle.moe_sort(route, experts, top_k, bm)
        n = int(want_t[0])
        assert n == 2 * -(-rows // bm)
        assert np.array_equal(lst, want_l) and np.array_equal(tiles[: 1 + 3 * n], want_t[: 1 + 3 * n])


def test_sort_expert_repeated_within_a_row(ctx, hb200, oracle):
    # not a top-k route (the destination-rank sort of the expert-parallel path looks like this): the kernel's
    # general path must give the same stable order
    rng = np.random.default_rng(3)
    rows, experts, top_k = 700, 8, 8
    route = np.zeros((rows, 2 * top_k), dtype=np.uint32)
    route[:, :top_k] = np.sort(rng.integers(0, experts, size=(rows, top_k)), axis=1)
    for bm in (16, 64):
        _, _, lst, tiles = sort_on_gpu(ctx, hb200, route, experts, top_k, bm)
        want_l, want_t = oracle.moe_sort(route, experts, top_k, bm)
        n = int(want_t[0])
        assert np.array_equal(lst, want_l) and np.array_equal(tiles[: 1 + 3 * n], want_t[: 1 + 3 * n])


def test_sort_same_list_every_run(ctx, hb200, oracle):
    route = oracle.route_topk(oracle.normal((2048, 256), 7, 3, 1.0), 8)
    first = sort_on_gpu(ctx, hb200, route, 256, 8, 16)[2]
    for _ in range(5):
        assert np.array_equal(first, sort_on_gpu(ctx, hb200, route, 256, 8, 16)[2])


@pytest.mark.parametrize("f32_sum", [0, 1])
def test_combine_bit_exact(ctx, oracle, f32_sum):
    rows, d, top_k = 61, 2048, 8
    route = oracle.route_topk(oracle.normal((rows, 256), SEED_ROUTER, 3, 1.0), top_k)
    ey = oracle.normal((rows * top_k, d), SEED_Y, 9, 1.0)
    d_y, d_r, d_o = ctx.to_device(ey), ctx.to_device(route), ctx.alloc(rows * d * 2)
    ctx.moe_combine(d, top_k, f32_sum)(rows, d_y, d_r, d_o)
    ctx.sync()
    assert np.array_equal(d_o.download(np.uint16, (rows, d)), oracle.moe_combine(ey, route, top_k, f32=bool(f32_sum)))


def test_gather_and_swiglu_slots_bit_exact(ctx, oracle):
    rows, h, top_k, experts = 77, 256, 4, 32
    x = oracle.normal((rows, h), SEED_X, 1, 1.0)
    route = oracle.route_topk(oracle.normal((rows, experts), SEED_ROUTER, 3, 1.0), top_k)
    lst, _ = oracle.moe_sort(route, experts, top_k, 16)
    d_x, d_l, d_xs = ctx.to_device(x), ctx.to_device(lst), ctx.alloc(rows * top_k * h * 2)
    ctx.moe_gather(h, top_k)(rows, d_x, d_l, d_xs)
    ctx.sync()
    assert np.array_equal(d_xs.download(np.uint16, (rows * top_k, h)), x[lst // top_k])
    egu = oracle.normal((rows * top_k, 2 * 96), SEED_Y, 4, 2.0)
    d_g, d_h = ctx.to_device(egu), ctx.alloc(rows * top_k * 96 * 2)
    ctx.swiglu_rows(96)(rows * top_k, d_g, d_h)
    ctx.sync()
    assert np.array_equal(d_h.download(np.uint16, (rows * top_k, 96)), oracle.swiglu_slots(egu))


def moe_layer(ctx, hb200, oracle, m, h, mi, experts, top_k, bm, fused=True, pre_gather=False, merge_runs=0):
    """The whole sparse block on the GPU and in the oracle; returns both sets of intermediates."""
    x = oracle.normal((m, h), SEED_X, 1, 1.0)
    wgu = oracle.normal((experts * 2 * mi, h), SEED_W, 2, h**-0.5)
    wd = oracle.normal((experts * h, mi), SEED_W, 3, mi**-0.5)
    scores = oracle.normal((m, experts), SEED_ROUTER, 3, 1.0)
    pairs = m * top_k
    # oracle
    o_route = oracle.route_topk(scores, top_k)
    o_list, o_tiles = oracle.moe_sort(o_route, experts, top_k, bm)
    o_egu = oracle.moe_gate_up(x, wgu, o_list, o_tiles, mi, top_k)
    o_ehb = oracle.swiglu_slots(o_egu)
    o_ey = oracle.moe_down(o_ehb, wd, o_list, o_tiles, h)
    o_out = oracle.moe_combine(o_ey, o_route, top_k)
    # GPU
    d_x, d_wgu, d_wd, d_s = ctx.to_device(x), ctx.to_device(wgu), ctx.to_device(wd), ctx.to_device(scores)
    nt = hb200.lib().hb_moe_tiles(m, top_k, experts, bm)
    d_route, d_list, d_tiles = ctx.alloc(m * 2 * top_k * 4), ctx.alloc(pairs * 4), ctx.alloc((1 + 3 * nt) * 4)
    d_egu, d_ehb, d_ey, d_out, d_xs = ctx.alloc(pairs * 2 * mi * 2), ctx.alloc(pairs * mi * 2), ctx.alloc(pairs * h * 2), ctx.alloc(m * h * 2), ctx.alloc(pairs * h * 2)
    ctx.route(experts, top_k)(m, d_s, d_route)
    ctx.moe_sort(experts, top_k, m, bm)(m, d_route, d_list, d_tiles)
    kw = dict(rows_max=m, top_k=top_k, experts=experts, bm=bm, merge_runs=merge_runs)
    if pre_gather:
        ctx.moe_gather(h, top_k)(m, d_x, d_list, d_xs)
        ctx.gemm(h, 2 * mi, hb200.OUT_SWIGLU, rows_mode=hb200.ROWS_SORTED, **kw)(m, d_wgu, d_xs, d_ehb, d_list, d_tiles)
    elif fused:
        ctx.gemm(h, 2 * mi, hb200.OUT_SWIGLU, rows_mode=hb200.ROWS_GATHER, **kw)(m, d_wgu, d_x, d_ehb, d_list, d_tiles)
    else:
        ctx.gemm(h, 2 * mi, hb200.OUT_BF16, rows_mode=hb200.ROWS_GATHER, **kw)(m, d_wgu, d_x, d_egu, d_list, d_tiles)
        ctx.swiglu_rows(mi)(pairs, d_egu, d_ehb)
    ctx.gemm(mi, h, hb200.OUT_BF16, rows_mode=hb200.ROWS_SCATTER, **kw)(m, d_wd, d_ehb, d_ey, d_list, d_tiles)
    ctx.moe_combine(h, top_k)(m, d_ey, d_route, d_out)
    ctx.sync()
    n = int(o_tiles[0])
    assert np.array_equal(d_route.download(np.uint32, (m, 2 * top_k)), o_route)
    assert np.array_equal(d_list.download(np.uint32, (pairs,)), o_list)
    assert np.array_equal(d_tiles.download(np.uint32, (1 + 3 * nt,))[: 1 + 3 * n], o_tiles[: 1 + 3 * n])
    g_ehb, g_ey, g_out = d_ehb.download(np.uint16, (pairs, mi)), d_ey.download(np.uint16, (pairs, h)), d_out.download(np.uint16, (m, h))
    within_contract(oracle, o_ehb, g_ehb, "expert gate/up + SwiGLU")
    # downstream stages are checked on the GPU's own inputs so that one stage's rounding differences do not compound
    within_contract(oracle, oracle.moe_down(g_ehb, wd, o_list, o_tiles, h), g_ey, "expert down")
    assert np.array_equal(oracle.moe_combine(g_ey, o_route, top_k), g_out)
    # end to end against the all-oracle chain the roundings of three stages compound (an element one bf16 ulp off
    # after gate/up moves its down-projection sums): the hard limit holds, the 1-ulp share is looser
    c = oracle.compare(o_out, g_out)
    assert c.max_abs_err <= c.max_abs_ref / 64 and c.over_1ulp <= 0.05 * c.count, f"MoE block output: {c.over_1ulp}/{c.count} over 1 ulp, max err {c.max_abs_err}"
    return g_out


@pytest.mark.parametrize("merge_runs", [0, 1])
@pytest.mark.parametrize("bm", [16, 32, 64])
@pytest.mark.parametrize("form", ["fused", "apart", "gather+fused"])
def test_moe_layer_small(ctx, hb200, oracle, bm, form, merge_runs):
    moe_layer(ctx, hb200, oracle, 100, 256, 192, 32, 8, bm, fused=form == "fused", pre_gather=form == "gather+fused", merge_runs=merge_runs)


@pytest.mark.parametrize("bm", [16, 64])
def test_moe_layer_long_runs_merged(ctx, hb200, oracle, bm):
    # 600 tokens, 32 experts, top-16: 300 rows per expert, so an expert's run spans three 128-row work items
    moe_layer(ctx, hb200, oracle, 600, 128, 160, 32, 16, bm, merge_runs=1)


def test_moe_layer_forms_agree_bitwise(ctx, hb200, oracle):
    outs = [moe_layer(ctx, hb200, oracle, 64, 128, 128, 32, 4, bm, fused=f, pre_gather=g, merge_runs=r) for bm in (16, 64) for f, g in ((True, False), (False, False), (True, True))
            for r in (0, 1)]
    for o in outs[1:]:
        assert np.array_equal(outs[0], o)


@pytest.mark.parametrize("shape", [(100, 256, 192, 32, 8, 16), (600, 128, 160, 32, 16, 64), (2048, 2048, 512, 256, 8, 64)])
def test_moe_layer_with_overlapped_launches(ctx, hb200, oracle, shape):
    """hb_set_launch_overlap: every kernel of the block is launched before the one before it has finished and waits for
    it inside; the same checks, and the same bits as with plain launches."""
    plain = moe_layer(ctx, hb200, oracle, *shape, merge_runs=1)
    ctx.set_launch_overlap(True)
    try:
        for _ in range(2):
            over = moe_layer(ctx, hb200, oracle, *shape, merge_runs=1)
            assert np.array_equal(plain, over)
        # (the form with the SwiGLU as a kernel of its own between the expert GEMMs)
        assert np.array_equal(plain, moe_layer(ctx, hb200, oracle, *shape, fused=False, merge_runs=1))
    finally:
        ctx.set_launch_overlap(False)


@pytest.mark.parametrize("merge_runs", [0, 1])
def test_config5_full_size(ctx, hb200, oracle, merge_runs):
    # hidden 2048, 256 experts, top-8, expert intermediate 512, 2048 tokens
    moe_layer(ctx, hb200, oracle, 2048, 2048, 512, 256, 8, 16, merge_runs=merge_runs)


@pytest.mark.parametrize("rows_per_warp", [1, 2, 4, 8])
def test_experts_matvec_is_the_matvec_per_slot(ctx, hb200, oracle, rows_per_warp):
    """experts_matvec (src/metal/qwen_kernels.rs:1880-1990; moe.grouped = 0 and the decode step): slot s of row r is the
    one-row matvec, in the reference's lane order, of its input against its expert's rows: bit-exact with that matvec."""
    m, h, mi, E, top_k = 5, 256, 136, 16, 4
    x = oracle.normal((m, h), SEED_X, 1, 1.0)
    wgu = oracle.normal((E * 2 * mi, h), SEED_W, 2, h**-0.5)
    wd = oracle.normal((E * h, mi), SEED_W, 3, mi**-0.5)
    route = oracle.route_topk(oracle.normal((m, E), SEED_ROUTER, 3, 1.0), top_k)
    pairs = m * top_k
    d_x, d_wgu, d_wd, d_r = ctx.to_device(x), ctx.to_device(wgu), ctx.to_device(wd), ctx.to_device(route)
    d_egu, d_ehb, d_ey = ctx.alloc(pairs * 2 * mi * 2), ctx.alloc(pairs * mi * 2), ctx.alloc(pairs * h * 2)
    k_gu = ctx.experts_matvec(h, 2 * mi, top_k, E, h, 0, rows_per_warp)          # every slot reads the row's x
    k_dn = ctx.experts_matvec(mi, h, top_k, E, top_k * mi, mi, rows_per_warp)    # slot s reads its own SwiGLU row
    assert k_gu.name.startswith("experts_matvec_")
    k_gu(m, d_wgu, d_x, d_egu, d_r)
    ctx.swiglu_rows(mi)(pairs, d_egu, d_ehb)
    k_dn(m, d_wd, d_ehb, d_ey, d_r)
    ctx.sync()
    egu, ehb, ey = d_egu.download(np.uint16, (pairs, 2 * mi)), d_ehb.download(np.uint16, (pairs, mi)), d_ey.download(np.uint16, (pairs, h))
    for g in range(pairs):
        r, s = divmod(g, top_k)
        e = int(route[r, s])
        assert np.array_equal(egu[g], oracle.matvec_ref_order(x[r], np.ascontiguousarray(wgu[e * 2 * mi : (e + 1) * 2 * mi]))), g
        assert np.array_equal(ey[g], oracle.matvec_ref_order(ehb[g], np.ascontiguousarray(wd[e * h : (e + 1) * h]))), g
    assert np.array_equal(ehb, oracle.swiglu_slots(egu))
    # against the grouped form of the same block, under the GEMM contract (the grouped GEMMs sum in another order)
    lst, tiles = oracle.moe_sort(route, E, top_k, 16)
    want = oracle.moe_down(oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, lst, tiles, mi, top_k)), wd, lst, tiles, h)
    c = oracle.compare(want, ey)
    assert c.max_abs_err <= c.max_abs_ref / 64 and c.over_1ulp <= 0.02 * c.count
    with pytest.raises(hb200.HbError):
        ctx.experts_matvec(100, 64, 4, 8, 100)  # K not a multiple of 8 (the reference's assertion)


def test_selection_moe_grouped_0_returns_the_per_slot_form(ctx, hb200, oracle):
    m, h, mi, E, top_k = 32, 256, 128, 16, 4
    pairs = m * top_k
    x = oracle.normal((m, h), SEED_X, 1, 1.0)
    wgu, wd = oracle.normal((E * 2 * mi, h), SEED_W, 2, h**-0.5), oracle.normal((E * h, mi), SEED_W, 3, mi**-0.5)
    route = oracle.route_topk(oracle.normal((m, E), SEED_ROUTER, 3, 1.0), top_k)
    d = {n_: ctx.to_device(a) for n_, a in dict(x=x, wgu=wgu, wd=wd, route=route).items()}
    nt = hb200.lib().hb_moe_tiles(m, top_k, E, 16)
    d_l, d_t, d_ehb, d_ey, d_egu, d_out = ctx.alloc(pairs * 4), ctx.alloc((1 + 3 * nt) * 4), ctx.alloc(pairs * mi * 2), ctx.alloc(pairs * h * 2), ctx.alloc(pairs * 2 * mi * 2), ctx.alloc(m * h * 2)
    outs = []
    for tune in ("moe.grouped=0,gemm.auto=0", "gemm.auto=0"):
        sel = hb200.Selector(ctx, hb200.Tune(tune))
        try:
            pick = sel.experts(E, top_k, h, mi, m, d["route"], d_l, d_t, d["x"], d["wgu"], d["wd"], d_ehb, d_ey, egu=d_egu)
            if "grouped=0" in tune:
                assert pick["bm"] == 0 and pick["sort"] is None and pick["gate_up"].name.startswith("experts_matvec_") and pick["swiglu"] is not None
                pick["gate_up"](m, d["wgu"], d["x"], d_egu, d["route"])
                pick["swiglu"](pairs, d_egu, d_ehb)
                pick["down"](m, d["wd"], d_ehb, d_ey, d["route"])
            else:
                assert pick["bm"] == 16 and pick["sort"] is not None
                pick["sort"](m, d["route"], d_l, d_t)
                pick["gate_up"](m, d["wgu"], d["x"], d_ehb, d_l, d_t)
                pick["down"](m, d["wd"], d_ehb, d_ey, d_l, d_t)
            ctx.moe_combine(h, top_k)(m, d_ey, d["route"], d_out)
            ctx.sync()
            outs.append(d_out.download(np.uint16, (m, h)))
        finally:
            sel.close()
    c = oracle.compare(outs[1], outs[0])  # the two forms of the same block: the same values up to the order of the sums
    assert c.max_abs_err <= c.max_abs_ref / 64 and c.over_1ulp <= 0.05 * c.count
