"""The load-time selection loop on the GPU: candidates are checked against the first one with the
1/64 rule (full and partial block, zeroed output), timed, the pick cached per key; a wrong candidate
is timed, starred and never picked (the reference's incident, README.md:65-73); tune keys fix the
kernel. Also the device-boundary error behaviour."""
import re

import numpy as np
import pytest

from gpu_util import gemm_inputs, within_contract
from oracle_lib import OUT_BF16, OUT_RESIDUAL, OUT_SWIGLU, SEED_ROUTER, SEED_W, SEED_X

pytestmark = pytest.mark.gpu


def bufs(ctx, oracle, m, k, n, out=OUT_BF16):
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    ncol = n // 2 if out == OUT_SWIGLU else n
    return (x, w, y0), ctx.to_device(w), ctx.to_device(x), ctx.to_device(y0[:, :ncol].copy())


def test_gemm_selection_logs_and_caches(ctx, hb200, oracle):
    m, k, n = 512, 1024, 2048
    (x, w, y0), d_w, d_x, d_y = bufs(ctx, oracle, m, k, n)
    sel = hb200.Selector(ctx, hb200.Tune("prefill.block=512"))
    assert sel.buckets() == [64, 128, 192, 256, 320, 384, 448, 512]
    kern = sel.gemm(k, n, OUT_BF16, d_w, d_x, d_y, m)
    log = sel.log()
    line = [l for l in log.splitlines() if l.startswith("[autotune] gemm 1024x2048 Bf16, 512 rows: ") and " -> " in l]
    assert len(line) == 1
    assert re.search(r"t128x256 \d+\.\d{3} ms, t128x128 \d+\.\d{3} ms, t128x64 \d+\.\d{3} ms.* -> ((t|sk)128x\d+n?|pair256x256)$", line[0]) and "sk128x256 " in line[0] and "pair256x256 " in line[0]
    assert "wrong" not in log
    # (Y is scratch during selection: the check restores it, the timing rounds that follow write it again,
    # as in the reference where the loop runs at load before any prompt)
    # cached: a second call times nothing
    launches = ctx.launch_count()
    again = sel.gemm(k, n, OUT_BF16, d_w, d_x, d_y, m)
    assert again.name == kern.name and ctx.launch_count() == launches
    # the pick computes the right thing
    kern(m, d_w, d_x, d_y)
    ctx.sync()
    within_contract(oracle, oracle.gemm_f64(x, w), d_y.download(np.uint16, (m, n)), kern.name)
    sel.close()


def test_wrong_candidate_is_rejected_and_starred(ctx, hb200, oracle):
    m, k, n = 256, 512, 1024
    for out in (OUT_BF16, OUT_RESIDUAL):
        (x, w, y0), d_w, d_x, d_y = bufs(ctx, oracle, m, k, n, out)
        sel = hb200.Selector(ctx, hb200.Tune("prefill.block=256"))
        sel.inject_wrong(True)
        kern = sel.gemm(k, n, out, d_w, d_x, d_y, m)
        log = sel.log()
        name = "Bf16" if out == OUT_BF16 else "Residual"
        wrong = [l for l in log.splitlines() if "wrong against t128x256, never picked: wrong (" in l]
        assert len(wrong) == 1 and wrong[0].startswith(f"[autotune] gemm 512x1024 {name}, 256 rows: ")
        assert re.search(r"wrong \(256 rows: max err \d\.\d{3}e-?\d+ of \d\.\d{3}e-?\d+\)", wrong[0])
        timing = [l for l in log.splitlines() if " -> " in l][0]
        assert re.search(r"wrong\* \d+\.\d{3} ms", timing) and not timing.endswith("-> wrong")
        assert not kern.name.startswith("wrong")
        sel.close()


def test_tune_keys_name_the_kernel(ctx, hb200, oracle):
    m, k, n = 128, 512, 1024
    (x, w, y0), d_w, d_x, d_y = bufs(ctx, oracle, m, k, n)
    for setting, tile in (("gemm.mma=2,gemm.tn=16", "t128x64"), ("gemm.mma=2,gemm.tn=32", "t128x128"), ("gemm.tn=64,gemm.mma=2", "t128x256"), ("gemm.auto=0", "t128x256")):
        sel = hb200.Selector(ctx, hb200.Tune(setting))
        assert sel.buckets() == [2048]  # no timing: one bucket, the block itself
        launches = ctx.launch_count()
        kern = sel.gemm(k, n, OUT_BF16, d_w, d_x, d_y, m)
        assert tile in kern.name and ctx.launch_count() == launches and sel.log() == ""
        sel.close()
    sel = hb200.Selector(ctx, hb200.Tune("gemm.auto=0,gemm.mfirst=0"))
    assert "_mf" not in sel.gemm(k, n, OUT_BF16, d_w, d_x, d_y, m).name
    sel.close()


def test_gate_up_fused_vs_apart(ctx, hb200, oracle):
    m, k, inter = 256, 512, 768
    x, w, _ = gemm_inputs(oracle, m, k, 2 * inter)
    d_w, d_x = ctx.to_device(w), ctx.to_device(x)
    d_gu, d_h = ctx.alloc(m * 2 * inter * 2), ctx.alloc(m * inter * 2)
    want = oracle.gemm_f64(x, w, OUT_SWIGLU)
    for setting, count in (("pf.fswi=0,prefill.block=256", 2), ("pf.fswi=1,prefill.block=256", 1), ("prefill.block=256", None)):
        sel = hb200.Selector(ctx, hb200.Tune(setting))
        ks = sel.gate_up(k, inter, d_w, d_x, d_gu, d_h, m)
        if count:
            assert len(ks) == count
        else:
            assert re.search(r"\[autotune\] gate_up 512x1536, 256 rows: apart \d+\.\d{3} ms, fused128x256 ", sel.log())
        d_h.zero()
        if len(ks) == 2:
            ks[0](m, d_w, d_x, d_gu)
            ks[1](m, d_gu, d_h)
        else:
            ks[0](m, d_w, d_x, d_h)
        ctx.sync()
        within_contract(oracle, want, d_h.download(np.uint16, (m, inter)), setting)
        sel.close()


def test_matvec_selection(ctx, hb200, oracle):
    k, n, rows = 1024, 2048, 4
    x, w, _ = gemm_inputs(oracle, rows, k, n)
    copies = [ctx.to_device(w) for _ in range(3)]
    d_x, d_y = ctx.to_device(x), ctx.alloc(rows * n * 2)
    sel = hb200.Selector(ctx, hb200.Tune("mv.persists=1"))
    kern = sel.matvec(k, n, OUT_BF16, rows, copies, d_x, d_y)
    log = sel.log()
    assert re.search(r"\[autotune\] matvec 1024x2048 Bf16, 4 rows p\[1\]: r1 \d+\.\d{3} ms, r2 ", log) and "r4k2p1" in log and "r8k4p1" not in log
    kern(rows, copies[0], d_x, d_y)
    ctx.sync()
    within_contract(oracle, oracle.gemm_f64(x, w), d_y.download(np.uint16, (rows, n)), kern.name)
    fixed = hb200.Selector(ctx, hb200.Tune("mv.split=2"))
    assert "_s2" in fixed.matvec(k, n, OUT_BF16, rows, copies, d_x, d_y).name and fixed.log() == ""
    sel.close()
    fixed.close()


def test_expert_selection(ctx, hb200, oracle):
    m, h, mi, experts, top_k = 256, 256, 128, 32, 4
    pairs = m * top_k
    x = oracle.normal((m, h), SEED_X, 1, 1.0)
    wgu = oracle.normal((experts * 2 * mi, h), SEED_W, 2, h**-0.5)
    wd = oracle.normal((experts * h, mi), SEED_W, 3, mi**-0.5)
    route = oracle.route_topk(oracle.normal((m, experts), SEED_ROUTER, 3, 1.0), top_k)
    nt = hb200.lib().hb_moe_tiles(2048, top_k, experts, 16)
    d = dict(route=ctx.to_device(route), lst=ctx.alloc(pairs * 4), tiles=ctx.alloc((1 + 3 * nt) * 4), x=ctx.to_device(x), wgu=ctx.to_device(wgu),
             wdown=ctx.to_device(wd), ehb=ctx.alloc(pairs * mi * 2), ey=ctx.alloc(pairs * h * 2), egu=ctx.alloc(pairs * 2 * mi * 2), xs=ctx.alloc(pairs * h * 2))
    sel = hb200.Selector(ctx, hb200.Tune(""))
    pick = sel.experts(experts, top_k, h, mi, m, **d)
    log = sel.log()
    for bm in (16, 32, 64):
        assert f"experts gate_up {experts} experts, tiles of {bm}, {m} rows: fused " in log and "apart" in log and "gather+fused" in log
    assert pick["bm"] in (16, 32, 64) and re.search(r"\[autotune\] experts 256 rows: tiles of (16|32|64) rows", log) and "wrong" not in log
    # the list and table left behind match the picked tile size, and the picked kernels compute the layer
    want_l, want_t = oracle.moe_sort(route, experts, top_k, pick["bm"])
    assert np.array_equal(d["lst"].download(np.uint32, (pairs,)), want_l)
    if pick["gather"]:
        pick["gather"](m, d["x"], d["lst"], d["xs"])
        pick["gate_up"](m, d["wgu"], d["xs"], d["ehb"], d["lst"], d["tiles"])
    elif pick["swiglu"]:
        pick["gate_up"](m, d["wgu"], d["x"], d["egu"], d["lst"], d["tiles"])
        pick["swiglu"](pairs, d["egu"], d["ehb"])
    else:
        pick["gate_up"](m, d["wgu"], d["x"], d["ehb"], d["lst"], d["tiles"])
    pick["down"](m, d["wdown"], d["ehb"], d["ey"], d["lst"], d["tiles"])
    ctx.sync()
    ehb = oracle.swiglu_slots(oracle.moe_gate_up(x, wgu, want_l, want_t, mi, top_k))
    g_ehb = d["ehb"].download(np.uint16, (pairs, mi))
    within_contract(oracle, ehb, g_ehb, "picked gate/up")
    within_contract(oracle, oracle.moe_down(g_ehb, wd, want_l, want_t, h), d["ey"].download(np.uint16, (pairs, h)), "picked down")
    only = hb200.Selector(ctx, hb200.Tune("moe.tile=32"))
    assert only.experts(experts, top_k, h, mi, m, **d)["bm"] == 32 and "tiles of 16," not in only.log()
    sel.close()
    only.close()


def test_fill_random16_matches_reference_stream(ctx, hb200, oracle):
    buf = ctx.alloc(4096 * 2)
    hb200.fill_random16(ctx, buf, 0x9E3779B9)
    assert np.array_equal(buf.download(np.uint16, (4096,)), oracle.xorshift16(4096, 0x9E3779B9))


def test_boundary_errors(ctx, hb200):
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(100, 64)  # K not a multiple of 8
    assert e.value.status == hb200.UNSUPPORTED
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(64, 64, tile_n=96)
    assert e.value.status == hb200.UNSUPPORTED and "tile_n" in e.value.message
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(64, 64, stages=50)
    assert e.value.status == hb200.UNSUPPORTED
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(64, 63, OUT_SWIGLU)
    assert e.value.status == hb200.INVALID
    with pytest.raises(hb200.HbError):
        ctx.moe_sort(256, 8, 2048, 48)
    with pytest.raises(hb200.HbError):
        ctx.route(100, 4)  # experts must be a multiple of 32 (qwen_kernels.rs:1803)
    kern = ctx.gemm(64, 64, rows_max=16)
    small = ctx.alloc(64)
    big = ctx.alloc(64 * 64 * 2)
    with pytest.raises(hb200.HbError) as e:
        kern(16, big, big, small)  # Y range too small: refused before any launch (Range bounds, gpu.rs:44)
    assert e.value.status == hb200.INVALID and "too small" in e.value.message
    with pytest.raises(hb200.HbError):
        kern(17, big, big, big)  # m beyond rows_max
    with pytest.raises(hb200.HbError):
        kern(0, big, big, big)
    with pytest.raises(hb200.HbError):
        ctx.launch(kern, 16, big, big)  # wrong binding count
    ctx.sync()  # the context is still usable after refused launches


def test_alloc_limit_reports_oom(hb200):
    c = hb200.Context(0)
    try:
        assert "B200" in c.describe() and "148 SMs" in c.describe()
        hb200.lib().hb_set_alloc_limit(c.h, 1 << 20)
        c.alloc(1 << 19)
        with pytest.raises(hb200.HbError) as e:
            c.alloc(1 << 20)
        assert e.value.status == hb200.OOM
        hb200.lib().hb_set_alloc_limit(c.h, 0)
        c.alloc(1 << 20)
        z = c.alloc(4096)
        assert not z.download(np.uint8, (4096,)).any()  # zero-initialised (gpu.rs:92)
    finally:
        c.close()


def test_small_blocks_get_the_weight_stream_candidates(ctx, hb200, oracle):
    # a block of 64 rows or fewer: the tensor-core weight stream is among the candidates, checked like the others
    m, k, n = 48, 1024, 2048
    for out in (OUT_BF16, OUT_RESIDUAL):
        (x, w, y0), d_w, d_x, d_y = bufs(ctx, oracle, m, k, n, out)
        sel = hb200.Selector(ctx, hb200.Tune("prefill.block=2048"))
        kern = sel.gemm(k, n, out, d_w, d_x, d_y, m)
        line = [l for l in sel.log().splitlines() if l.startswith("[autotune] gemm 1024x2048") and " -> " in l][0]
        assert re.search(r"stream \d+\.\d{3} ms, streamb \d+\.\d{3} ms", line) and "wrong" not in sel.log()
        d_y.upload(y0 if out == OUT_RESIDUAL else np.zeros_like(y0))
        kern(m, d_w, d_x, d_y)
        ctx.sync()
        within_contract(oracle, oracle.gemm_f64(x, w, out, y0), d_y.download(np.uint16, (m, n)), kern.name)
        sel.close()
    inter = 512
    x, wgu = oracle.normal((m, k), 1, 1, 1.0), oracle.normal((2 * inter, k), 2, 2, k**-0.5)
    d_w, d_x, d_gu, d_h = ctx.to_device(wgu), ctx.to_device(x), ctx.alloc(m * 2 * inter * 2), ctx.alloc(m * inter * 2)
    sel = hb200.Selector(ctx, hb200.Tune(""))
    ks = sel.gate_up(k, inter, d_w, d_x, d_gu, d_h, m)
    assert "fusedstream " in sel.log() and "fusedstreamb " in sel.log()
    for kk in ks[:-1]:
        kk(m, d_w, d_x, d_gu)
    (ks[-1](m, d_w, d_x, d_h) if len(ks) == 1 else ks[-1](m, d_gu, d_h))
    ctx.sync()
    within_contract(oracle, oracle.gemm_f64(x, wgu, OUT_SWIGLU), d_h.download(np.uint16, (m, inter)), "picked gate/up at 48 rows")
    sel.close()
