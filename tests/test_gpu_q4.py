"""Q4_0 weights: the decode kernel and the Q4 matvec, bit-exact with the oracle (itself pinned to the independent
restatement in tests/golden and to the reference's own unit test: a block on the grid comes back exactly)."""
import numpy as np
import pytest

from gpu_util import within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL

pytestmark = pytest.mark.gpu
G = np.load(__import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "golden.npz"))


def test_dequant_golden_and_model_shapes(ctx, oracle):
    n, k = G["q4_w"].shape
    d_w, d_s, d_o = ctx.to_device(G["q4_data"]), ctx.to_device(G["q4_scales"]), ctx.alloc(n * k * 2)
    ctx.dequant_q4(k, n)(1, d_w, d_s, d_o)
    ctx.sync()
    assert np.array_equal(d_o.download(np.uint16, (n, k)), G["q4_dequant"])
    for n, k in ((300, 4096), (1000, 2560), (7, 32)):
        w = oracle.normal((n, k), 5, n, 0.03)
        data, scales = oracle.q4_quantize(w)
        d_w, d_s, d_o = ctx.to_device(data), ctx.to_device(scales), ctx.alloc(n * k * 2)
        ctx.dequant_q4(k, n)(1, d_w, d_s, d_o)
        ctx.sync()
        assert np.array_equal(d_o.download(np.uint16, (n, k)), oracle.q4_dequant(data, scales, n, k)), (n, k)


@pytest.mark.parametrize("masks", [0, 1])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL])
@pytest.mark.parametrize("rows", [1, 2, 4])
def test_matvec_q4_bits_and_contract(ctx, oracle, out, rows, masks):
    n, k = G["q4_w"].shape
    if out == OUT_BF16:
        d_w, d_s, d_x, d_y = ctx.to_device(G["q4_data"]), ctx.to_device(G["q4_scales"]), ctx.to_device(G["q4_x"]), ctx.alloc(max(n * 2, 16))
        kern = ctx.matvec_q4(k, n, out, rows, masks)
        assert kern.name.startswith("matvec_q4s_" if masks else "matvec_q4_")
        kern(1, d_w, d_x, d_y, d_s)
        ctx.sync()
        assert np.array_equal(d_y.download(np.uint16, (n,)), G["q4s_matvec" if masks else "q4_matvec"])
    for n, k in ((1001, 4096), (330, 1024), (5, 32), (64, 12288)):
        w = oracle.normal((n, k), 6, n, k**-0.5)
        x = oracle.normal((k,), 7, k, 1.0)
        y0 = oracle.normal((n,), 8, n, 1.0)
        data, scales = oracle.q4_quantize(w)
        d_w, d_s, d_x = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x)
        if out == OUT_F32:
            d_y = ctx.alloc(n * 4)
            start = None
        else:
            start = y0 if out == OUT_RESIDUAL else np.zeros(n, dtype=np.uint16)
            d_y = ctx.to_device(start) if n * 2 >= 16 else ctx.alloc(16).upload(start)
        ctx.matvec_q4(k, n, out, rows, masks)(1, d_w, d_x, d_y, d_s)
        ctx.sync()
        got = d_y.download(np.float32 if out == OUT_F32 else np.uint16, (n,))
        want = oracle.matvec_q4(data, scales, x, n, k, out, start, masks=bool(masks))
        assert np.array_equal(got.view(np.uint32 if out == OUT_F32 else np.uint16), want.view(np.uint32 if out == OUT_F32 else np.uint16)), (n, k)
        # and the contract against the f64 product of the exact weights d * q (the matvec does not round them to bf16)
        if out != OUT_RESIDUAL:
            nib = np.stack([data.reshape(-1, 16)[:, 4 * (e // 8) + (e % 8) % 4] >> (4 if e % 8 >= 4 else 0) & 15 for e in range(32)], axis=1)
            q = ((nib ^ 8).astype(np.int32) - 8).astype(np.float64)
            wq = (q * scales.view(np.float16).astype(np.float64)[:, None]).reshape(n, k)
            xf = (x.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
            ref64 = wq @ xf
            if out == OUT_F32:
                ref = ref64.astype(np.float32).reshape(1, n)
            else:
                ref = np.array([oracle.lib.hbo_f64_to_bf16(float(v)) for v in ref64], dtype=np.uint16).reshape(1, n)
            within_contract(oracle, ref, got.reshape(1, n), f"matvec_q4 {n}x{k}")


def test_q4_prefill_is_dequant_then_gemm(ctx, oracle):
    # the reference's Q4 prefill GEMM multiplies the decoded bf16 values: decode once, then the bf16 GEMM
    m, k, n = 96, 1024, 512
    w = oracle.normal((n, k), 9, 1, k**-0.5)
    x = oracle.normal((m, k), 10, 2, 1.0)
    data, scales = oracle.q4_quantize(w)
    d_q, d_s, d_w, d_x, d_y = ctx.to_device(data), ctx.to_device(scales), ctx.alloc(n * k * 2), ctx.to_device(x), ctx.alloc(m * n * 2)
    ctx.run([(ctx.dequant_q4(k, n), 1, d_q, d_s, d_w), (ctx.gemm(k, n, OUT_BF16, rows_max=m), m, d_w, d_x, d_y)])
    ctx.sync()
    within_contract(oracle, oracle.gemm_f64(x, oracle.q4_dequant(data, scales, n, k)), d_y.download(np.uint16, (m, n)), "Q4 prefill")


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 6, 7, 8])
def test_matmul_q4_rows_have_the_decode_steps_bits(ctx, oracle, m):
    """matmul_q4 (src/metal/kernels.rs:983-1071): every row of a short block comes out as matvec_q4 gives it alone."""
    if m == 3:
        n, k = G["q4_w"].shape
        ldx = G["q4_X"].shape[1]
        d_w, d_s, d_x, d_y = ctx.to_device(G["q4_data"]), ctx.to_device(G["q4_scales"]), ctx.to_device(G["q4_X"]), ctx.alloc(3 * n * 2 + 16)
        kern = ctx.matmul_q4(k, n, 3, ldx, n)
        assert kern.name == f"matmul_q4_{k}x{n}_m3_x{ldx}_y{n}"
        kern(3, d_w, d_x, d_y, d_s)
        ctx.sync()
        assert np.array_equal(d_y.download(np.uint16, (3, n)), G["q4_matmul"])
    for n, k, pad_x, pad_y in ((1001, 4096, 0, 0), (330, 1024, 8, 3), (5, 32, 24, 1), (64, 12288, 0, 8)):
        if 2 * ((m + 1) // 2) * k * 2 > 227 * 1024:
            continue  # the rows of X do not fit in shared memory: the library says so (test_q4_limits)
        ldx, ldy = k + pad_x, n + pad_y
        w = oracle.normal((n, k), 6, n, k**-0.5)
        x = oracle.normal((m, ldx), 7, k + m, 1.0)
        data, scales = oracle.q4_quantize(w)
        start = oracle.normal((m, ldy), 8, n, 1.0)  # what lies between the rows of Y must stay
        d_w, d_s, d_x, d_y = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x), ctx.to_device(start)
        ctx.matmul_q4(k, n, m, ldx, ldy)(m, d_w, d_x, d_y, d_s)
        ctx.sync()
        got = d_y.download(np.uint16, (m, ldy))
        want = oracle.matmul_q4(data, scales, x, n, k, ldy)
        assert np.array_equal(got[:, :n], want[:, :n]), (m, n, k)
        assert np.array_equal(got[:, n:], start[:, n:]), "padding of Y written"
        # row r alone through the one-row kernel: the same bits
        r = m - 1
        d_y1 = ctx.alloc(max(n * 2, 16))
        ctx.matvec_q4(k, n, OUT_BF16, 2, 0)(1, d_w, ctx.to_device(np.ascontiguousarray(x[r, :k])), d_y1, d_s)
        ctx.sync()
        assert np.array_equal(d_y1.download(np.uint16, (n,)), got[r, :n])


def test_q4_limits(ctx, hb200):
    for bad in (lambda: ctx.matmul_q4(4096, 64, 9), lambda: ctx.matmul_q4(4096, 64, 2, 4100, 64), lambda: ctx.matmul_q4(17408, 64, 8)):
        with pytest.raises(hb200.HbError) as e:
            bad()
        assert e.value.status == hb200.UNSUPPORTED
    with pytest.raises(hb200.HbError) as e:
        ctx.matmul_q4(4096, 64, 2, 4088, 64)
    assert e.value.status == hb200.INVALID
    with pytest.raises(hb200.HbError) as e:
        ctx.matmul_q4(4096, 64, 2)(3, ctx.alloc(64 * 2048), ctx.alloc(2 * 8192), ctx.alloc(256), ctx.alloc(64 * 256))
    assert e.value.status == hb200.INVALID
    for bad in (lambda: ctx.dequant_q4(40, 8), lambda: ctx.matvec_q4(4096, 64, 3, 2), lambda: ctx.matvec_q4(4096, 64, OUT_BF16, 3), lambda: ctx.matvec_q4(4096, 64, 3, 2, 1)):
        with pytest.raises(hb200.HbError) as e:
            bad()
        assert e.value.status == hb200.UNSUPPORTED


@pytest.mark.parametrize("split", [2, 4, 8])
@pytest.mark.parametrize("rows", [1, 2, 4])
def test_matvec_q4_split_and_persistent_forms(ctx, oracle, hb200, rows, split):
    """matvec_q4_split (src/metal/kernels.rs:472-500): the blocks of a row shared by `split` warps, the partial sums added
    in warp order - bit-exact with the oracle's statement of that order; a fixed grid (persist) changes no bit."""
    for n, k in ((1001, 4096), (330, 1024), (5, 32), (64, 12288)):
        w = oracle.normal((n, k), 6, n, k**-0.5)
        x = oracle.normal((k,), 7, k, 1.0)
        y0 = oracle.normal((n,), 8, n, 1.0)
        data, scales = oracle.q4_quantize(w)
        d_w, d_s, d_x = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x)
        for out in (OUT_BF16, OUT_RESIDUAL):
            start = y0 if out == OUT_RESIDUAL else np.zeros(n, dtype=np.uint16)
            want = oracle.matvec_q4(data, scales, x, n, k, out, start, split=split)
            for persist in (0, 3):
                d_y = ctx.to_device(start) if n * 2 >= 16 else ctx.alloc(16).upload(start)
                kern = ctx.matvec_q4(k, n, out, rows, 0, split=split, persist=persist)
                assert f"_s{split}" in kern.name and (("_p3" in kern.name) == bool(persist))
                kern(1, d_w, d_x, d_y, d_s)
                ctx.sync()
                assert np.array_equal(d_y.download(np.uint16, (n,)), want), (n, k, out, persist)
    # the masks order with a split: the same form, held to the plain form under the contract
    n, k = 1001, 4096
    w = oracle.normal((n, k), 6, n, k**-0.5)
    x = oracle.normal((k,), 7, k, 1.0)
    data, scales = oracle.q4_quantize(w)
    d_w, d_s, d_x, d_y = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x), ctx.alloc(n * 2)
    ctx.matvec_q4(k, n, OUT_BF16, rows, 1, split=split)(1, d_w, d_x, d_y, d_s)
    ctx.sync()
    c = oracle.compare(oracle.matvec_q4(data, scales, x, n, k, OUT_BF16, masks=True), d_y.download(np.uint16, (n,)))
    assert c.over_1ulp <= 2 and c.max_abs_err <= c.max_abs_ref / 64
    with pytest.raises(hb200.HbError):
        ctx.matvec_q4(k, n, OUT_BF16, 2, 0, split=3)
