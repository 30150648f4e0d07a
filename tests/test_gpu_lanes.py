"""Copy lanes: uploads and downloads that overlap the kernels, ordered by events (include/hb200.h).

The streamed form must give, block by block, the bits of the plain upload -> kernels -> download sequence,
whatever the interleaving, and the host must be able to read block i as soon as wait(i) returns.
"""
import numpy as np
import pytest

from gpu_util import gemm_inputs, within_contract
from oracle_lib import OUT_BF16, OUT_RESIDUAL

pytestmark = pytest.mark.gpu


def test_streamed_blocks_match_serial(ctx, hb200, oracle):
    m, k, n, blocks_n = 256, 512, 768, 7
    x0, w, y0 = gemm_inputs(oracle, m, k, n)
    rng = np.random.default_rng(5)
    xs = [np.ascontiguousarray(np.roll(x0, int(rng.integers(1, m)), axis=0)) for _ in range(blocks_n)]
    d_w = ctx.to_device(w)
    kern = ctx.gemm(k, n, OUT_BF16, rows_max=m)
    # serial
    want = []
    d_x, d_y = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    for x in xs:
        d_x.upload(x)
        kern(m, d_w, d_x, d_y)
        want.append(d_y.download(np.uint16, (m, n)))
    # streamed over three buffer sets
    sets = []
    for _ in range(3):
        dx, dy = ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
        sets.append(([(kern, m, d_w, dx, dy)], dx, dy))
    sb = hb200.StreamedBlocks(ctx, sets)
    h_in = ctx.host_array((blocks_n, m, k))
    h_out = ctx.host_array((blocks_n, m, n))
    for i, x in enumerate(xs):
        h_in[i] = x
    for i in range(blocks_n):
        sb.step(i, h_in[i], h_out[i])
        if i >= 1:
            sb.wait(i - 1)
            assert np.array_equal(h_out[i - 1], want[i - 1]), f"block {i - 1}"
    sb.wait(blocks_n - 1)
    assert np.array_equal(h_out[blocks_n - 1], want[blocks_n - 1])
    within_contract(oracle, oracle.gemm_f64(xs[-1], w), h_out[blocks_n - 1], "streamed block")
    sb.close()
    ctx.sync()


def test_events_order_lanes(ctx, hb200, oracle):
    # a download enqueued before the kernels' lane has run must still see the kernels' output
    m, k, n = 128, 256, 256
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_w, d_x, d_y = ctx.to_device(w), ctx.alloc(m * k * 2), ctx.to_device(y0)
    h_x, h_y = ctx.host_array((m, k)), ctx.host_array((m, n))
    h_x[:] = x
    up, done = ctx.event(), ctx.event()
    never = ctx.event()
    never.wait(hb200.LANE_KERNELS)  # an event nobody recorded does not block
    ctx.upload_async(d_x, h_x)
    up.record(hb200.LANE_UPLOAD).wait(hb200.LANE_KERNELS)
    ctx.gemm(k, n, OUT_RESIDUAL, rows_max=m)(m, d_w, d_x, d_y)
    done.record(hb200.LANE_KERNELS).wait(hb200.LANE_DOWNLOAD)
    ctx.download_async(h_y, d_y)
    fin = ctx.event().record(hb200.LANE_DOWNLOAD)
    fin.sync()
    within_contract(oracle, oracle.gemm_f64(x, w, OUT_RESIDUAL, y0), np.array(h_y), "residual through lanes")
    for e in (up, done, never, fin):
        e.free()
    with pytest.raises(hb200.HbError):
        ctx.event().record(7)
    ctx.sync()


def test_recorded_sequence_replays(ctx, hb200, oracle):
    # three kernels recorded once: replays give the bits of the one-by-one launches
    m, k, n = 8, 1024, 512
    x, w, y0 = gemm_inputs(oracle, m, k, 2 * n)
    d_w, d_x = ctx.to_device(w), ctx.to_device(x)
    d_gu, d_h, d_y = ctx.alloc(m * 2 * n * 2), ctx.alloc(m * n * 2), ctx.alloc(m * 2 * n * 2)
    ops = [(ctx.matvec(k, 2 * n, OUT_BF16, rows_max=m, tensor_core=2), m, d_w, d_x, d_gu), (ctx.swiglu_rows(n), m, d_gu, d_h),
           (ctx.matvec(k, 2 * n, OUT_RESIDUAL, rows_max=m, tensor_core=1), m, d_w, d_x, d_y)]
    ctx.run(ops)
    ctx.sync()
    want_h, want_y = d_h.download(np.uint16, (m, n)), d_y.download(np.uint16, (m, 2 * n))
    ctx.memset(d_y, 0)
    ctx.memset(d_h, 0)
    g = ctx.record(ops)
    before = ctx.launch_count()
    g.launch()
    ctx.sync()
    assert ctx.launch_count() == before + 3
    assert np.array_equal(d_h.download(np.uint16, (m, n)), want_h) and np.array_equal(d_y.download(np.uint16, (m, 2 * n)), want_y)
    assert g.time(5) > 0
    g.free()
    # the stream-K GEMM (partial tiles through scratch and flags that their one reader clears) replays too
    m2, k2, n2 = 64, 4096, 768
    x2, w2, _ = gemm_inputs(oracle, m2, k2, n2)
    d_w2, d_x2, d_y2 = ctx.to_device(w2), ctx.to_device(x2), ctx.alloc(m2 * n2 * 2)
    sk = ctx.gemm(k2, n2, OUT_BF16, rows_max=64, tile_n=256, stream_k=1)
    sk(m2, d_w2, d_x2, d_y2)
    ctx.sync()
    want2 = d_y2.download(np.uint16, (m2, n2))
    g2 = ctx.record([(sk, m2, d_w2, d_x2, d_y2)])
    for _ in range(3):
        ctx.memset(d_y2, 0)
        g2.launch()
        ctx.sync()
        assert np.array_equal(d_y2.download(np.uint16, (m2, n2)), want2)
    g2.free()


def test_overlapped_launches_change_nothing_but_time(hb200, oracle):
    # a decode-like chain (norm -> projection -> residual projection), each kernel consuming its predecessor's output:
    # launched ahead of their predecessors' end, the kernels wait inside; the bits are those of plain launches
    ctx = hb200.Context(0)
    try:
        k, n = 2048, 4096
        for m in (1, 8):
            x = oracle.normal((m, k), 1, m, 1.0)
            w1, w2 = oracle.normal((n, k), 2, 2, k**-0.5), oracle.normal((k, n), 3, 3, n**-0.5)
            nw = oracle.normal((k,), 4, 4, 0.1)
            outs = []
            for overlap in (False, True):
                ctx.set_launch_overlap(overlap)
                d_x, d_xn, d_h = ctx.to_device(x), ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
                d_w1, d_w2, d_nw = ctx.to_device(w1), ctx.to_device(w2), ctx.to_device(nw)
                form = dict(tensor_core=1, split=2) if m > 1 else dict(rows_per_warp=2, split=2)
                ops = [(ctx.rmsnorm(k, 1e-6, True), m, d_x, d_nw, d_xn), (ctx.matvec(k, n, OUT_BF16, rows_max=m, **form), m, d_w1, d_xn, d_h),
                       (ctx.matvec(n, k, OUT_RESIDUAL, rows_max=m, **form), m, d_w2, d_h, d_x)]
                for _ in range(5):  # the residual stream feeds the next pass: five dependent passes
                    ctx.run(ops)
                ctx.sync()
                res = [d_x.download(np.uint16, (m, k))]
                g = ctx.record(ops)
                for _ in range(5):
                    g.launch()
                ctx.sync()
                res.append(d_x.download(np.uint16, (m, k)))
                g.free()
                outs.append(res)
            assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
        ctx.set_launch_overlap(False)
    finally:
        ctx.close()
