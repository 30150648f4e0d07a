"""The decode projections whose input is made inside the kernel (the reference's XSrc::Norm and XSrc::Swiglu,
src/metal/kernels.rs:236-252, 355-442; engine switches dec.fnorm and dec.fswi, src/metal/qwen.rs:224-228, 1603).

"Each fusion gives the same bits as the kernels it replaces" (README.md:57): the fused kernel must equal, bit for
bit, the separate norm (or SwiGLU) kernel followed by the same form of the projection. The separate kernels are held
to the oracle elsewhere (test_gpu_rows.py: bit-exact; test_gpu_matvec.py: the engine's contract); here the chain is
also checked against the oracle's norm followed by the f64 product under that contract.
"""
import struct

import numpy as np
import pytest

from gpu_util import out_buffer, within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU

pytestmark = pytest.mark.gpu

EPS = 1e-6
EPS_BITS = struct.unpack("<I", struct.pack("<f", EPS))[0]


def inputs(oracle, m, k, n):
    x = oracle.normal((m, k), 11, 1, 1.5)
    w = oracle.normal((n, k), 12, 2, k**-0.5)
    nw = oracle.normal((k,), 13, 3, 0.2)
    y0 = oracle.normal((m, n), 14, 4, 1.0)
    return x, w, nw, y0


@pytest.mark.parametrize("m", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
def test_norm_inside_the_cuda_core_matvec(ctx, oracle, hb200, m, out):
    for k, n, plus_one in ((1024, 328, True), (4096, 512, False), (256, 40, True)):
        x, w, nw, y0 = inputs(oracle, m, k, n)
        d_x, d_w, d_nw, d_xn = ctx.to_device(x), ctx.to_device(w), ctx.to_device(nw), ctx.alloc(m * k * 2)
        ctx.rmsnorm(k, EPS, plus_one)(m, d_x, d_nw, d_xn)
        xn = oracle.rmsnorm_rows(x, nw, EPS, plus_one)
        want = oracle.gemm_f64(xn, w, out, y0)
        for rpw in (2, 4):
            for split, persist in ((1, 0), (2, 0), (1, 1), (4, 1)):
                form = dict(rows_per_warp=rpw, split=split, persist=persist)
                d_y1, dtype, shape = out_buffer(ctx, out, m, n, y0)
                d_y2, _, _ = out_buffer(ctx, out, m, n, y0)
                ctx.matvec(k, n, out, rows_max=m, **form)(m, d_w, d_xn, d_y1)
                fused = ctx.matvec(k, n, out, rows_max=m, x_src=hb200.X_NORM, norm_eps_bits=EPS_BITS, norm_plus_one=int(plus_one), **form)
                assert "_nrm" in fused.name
                fused(m, d_w, d_x, d_y2, d_nw)
                ctx.sync()
                got = d_y2.download(dtype, shape)
                assert np.array_equal(d_y1.download(dtype, shape), got), f"{fused.name} m={m}: differs from rmsnorm_rows + matvec"
                within_contract(oracle, want, got, f"{fused.name} m={m}")
        assert np.array_equal(d_xn.download(np.uint16, (m, k)), xn)


@pytest.mark.parametrize("m", [1, 3, 4, 8, 16])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
def test_norm_inside_the_tensor_core_stream(ctx, oracle, hb200, m, out):
    for k, n, plus_one in ((1024, 330, True), (4096, 512, False), (256, 96, True)):
        x, w, nw, y0 = inputs(oracle, m, k, n)
        d_x, d_w, d_nw, d_xn = ctx.to_device(x), ctx.to_device(w), ctx.to_device(nw), ctx.alloc(m * k * 2)
        ctx.rmsnorm(k, EPS, plus_one)(m, d_x, d_nw, d_xn)
        want = oracle.gemm_f64(oracle.rmsnorm_rows(x, nw, EPS, plus_one), w, out, y0)
        for tc in (1, 2):
            for kps in (1, 2):
                d_y1, dtype, shape = out_buffer(ctx, out, m, n, y0)
                d_y2, _, _ = out_buffer(ctx, out, m, n, y0)
                ctx.matvec(k, n, out, rows_max=m, tensor_core=tc, split=kps)(m, d_w, d_xn, d_y1)
                fused = ctx.matvec(k, n, out, rows_max=m, tensor_core=tc, split=kps, x_src=hb200.X_NORM, norm_eps_bits=EPS_BITS, norm_plus_one=int(plus_one))
                assert fused.name.startswith("matvec_tc_") and "_nrm" in fused.name
                for _ in range(2):  # twice: the kernel object keeps the normalised rows of its last launch
                    fused(m, d_w, d_x, d_y2, d_nw)
                    ctx.sync()
                    got = d_y2.download(dtype, shape)
                    if out == OUT_RESIDUAL:
                        break  # a second launch would add the product again
                assert np.array_equal(d_y1.download(dtype, shape), got), f"{fused.name} m={m}: differs from rmsnorm_rows + the same stream"
                within_contract(oracle, want, got, f"{fused.name} m={m}")


@pytest.mark.parametrize("m", [1, 2, 4, 8])
def test_swiglu_inside_the_down_projection(ctx, oracle, hb200, m):
    # x holds rows of [gate | up]; the projection's input is bf16(g * sigmoid(g) * u), made where x is loaded
    for k, n in ((1024, 328), (3072, 256)):
        gu = oracle.normal((m, 2 * k), 21, 1, 1.0)
        w = oracle.normal((n, k), 22, 2, k**-0.5)
        y0 = oracle.normal((m, n), 23, 3, 1.0)
        h = oracle.swiglu_rows(gu)
        d_gu, d_w, d_h = ctx.to_device(gu), ctx.to_device(w), ctx.alloc(m * k * 2)
        ctx.swiglu_rows(k)(m, d_gu, d_h)
        for out in (OUT_BF16, OUT_RESIDUAL):
            want = oracle.gemm_f64(h, w, out, y0)
            for rpw in (2, 4):
                for split, persist in ((1, 0), (2, 1)):
                    form = dict(rows_per_warp=rpw, split=split, persist=persist)
                    d_y1, dtype, shape = out_buffer(ctx, out, m, n, y0)
                    d_y2, _, _ = out_buffer(ctx, out, m, n, y0)
                    ctx.matvec(k, n, out, rows_max=m, **form)(m, d_w, d_h, d_y1)
                    fused = ctx.matvec(k, n, out, rows_max=m, x_src=hb200.X_SWIGLU, **form)
                    assert fused.name.endswith("_swi")
                    fused(m, d_w, d_gu, d_y2)
                    ctx.sync()
                    got = d_y2.download(dtype, shape)
                    assert np.array_equal(d_y1.download(dtype, shape), got), f"{fused.name} m={m}: differs from swiglu_rows + matvec"
                    within_contract(oracle, want, got, f"{fused.name} m={m}")
        assert np.array_equal(d_h.download(np.uint16, (m, k)), h)


def test_what_the_fused_forms_refuse(ctx, hb200):
    for bad in (dict(k=1000, n=64, x_src=1), dict(k=16384, n=64, x_src=1), dict(k=1024, n=64, x_src=1, rows_per_warp=1), dict(k=1024, n=64, x_src=1, x_stationary=1, rows_max=4),
                dict(k=1024, n=64, x_src=2, tensor_core=1), dict(k=1024, n=64, x_src=1, tensor_core=1, rows_max=32), dict(k=1024, n=64, x_src=3),
                dict(k=8192, n=64, x_src=2, rows_max=8)):
        kw = dict(bad)
        k, n = kw.pop("k"), kw.pop("n")
        with pytest.raises(hb200.HbError) as e:
            ctx.matvec(k, n, OUT_BF16, **kw)
        assert e.value.status in (hb200.UNSUPPORTED, hb200.INVALID), bad
    kern = ctx.matvec(1024, 64, OUT_BF16, x_src=hb200.X_NORM, norm_eps_bits=EPS_BITS)
    buf = ctx.alloc(1 << 20)
    with pytest.raises(hb200.HbError) as e:
        kern(1, buf, buf, buf)  # the norm's weights are a binding of their own
    assert e.value.status == hb200.INVALID


def test_selection_times_the_fused_step(ctx, oracle, hb200):
    """hb_select_matvec_x picks a form of the fused projection; hb_select_axis times the step with the norm apart and
    inside (the reference's tune_step axis "fnorm") and logs the line; a key given with --tune is kept untimed."""
    m, k, n = 4, 2048, 1536
    x, w, nw, y0 = inputs(oracle, m, k, n)
    d_x, d_w, d_nw, d_xn, d_y = ctx.to_device(x), ctx.to_device(w), ctx.to_device(nw), ctx.alloc(m * k * 2), ctx.alloc(m * n * 2)
    sel = hb200.Selector(ctx, hb200.Tune(""))
    try:
        apart_mv = sel.matvec(k, n, OUT_BF16, m, [d_w], d_xn, d_y)
        fused_mv = sel.matvec_x(k, n, OUT_BF16, m, hb200.X_NORM, EPS_BITS, 1, [d_w], d_x, d_y, d_nw)
        assert "_nrm" in fused_mv.name and f"matvec {k}x{n} Bf16 norm, {m} rows" in sel.log()
        assert sel.matvec_x(k, n, OUT_BF16, m, hb200.X_NORM, EPS_BITS, 1, [d_w], d_x, d_y, d_nw).name == fused_mv.name  # cached
        apart = [(ctx.rmsnorm(k, EPS, True), m, d_x, d_nw, d_xn), (apart_mv, m, d_w, d_xn, d_y)]
        fused = [(fused_mv, m, d_w, d_x, d_y, d_nw)]
        best = sel.axis("fnorm", "dec.fnorm", [apart, fused], [0, 1], position=7)
        assert best in (0, 1)
        line = [l for l in sel.log().splitlines() if "decode step at position 7, fnorm:" in l]
        assert len(line) == 1 and line[0].startswith("[autotune] decode step at position 7, fnorm: 0 ") and line[0].endswith(f"-> {best}")
        ctx.run(apart)
        ctx.sync()
        a = d_y.download(np.uint16, (m, n))
        d_y.zero()
        ctx.run(fused)
        ctx.sync()
        if apart_mv.name.split("_m")[1] == fused_mv.name.split("_m")[1].split("_nrm")[0]:
            assert np.array_equal(a, d_y.download(np.uint16, (m, n)))  # the same form picked both times: the same bits
        within_contract(oracle, oracle.gemm_f64(oracle.rmsnorm_rows(x, nw, EPS, True), w), d_y.download(np.uint16, (m, n)), fused_mv.name)
    finally:
        sel.close()
    for given, want in (("dec.fnorm=1", 1), ("dec.fnorm=0", 0), ("dec.auto=0", 0)):
        sel = hb200.Selector(ctx, hb200.Tune(given))
        try:
            assert sel.axis("fnorm", "dec.fnorm", [apart, fused], [0, 1], position=7) == want
            assert "decode step" not in sel.log()
        finally:
            sel.close()
