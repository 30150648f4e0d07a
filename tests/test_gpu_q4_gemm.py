"""The prefill GEMM on Q4_0 weights that decodes while it stages (the reference's gemm_mma_q4, src/metal/prefill.rs:
427-434, 1058-1076): "the sums are those of dequant_q4 then the GEMM, bit for bit". The fused kernel must equal
dequant_q4 (bit-exact with the oracle, test_gpu_q4.py) followed by the bf16 GEMM (held to the engine's contract,
test_gpu_gemm.py) on every output bit, for every output mode, ragged extents, a K that ends inside a stage's slice,
and the 9B-class shapes; and it is checked against the f64 product of the decoded weights under the contract."""
import numpy as np
import pytest

from gpu_util import out_buffer, within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU

pytestmark = pytest.mark.gpu


def q4_inputs(oracle, m, k, n):
    w = oracle.normal((n, k), 31, n, k**-0.5)
    x = oracle.normal((m, k), 32, m, 1.0)
    y0 = oracle.normal((m, n), 33, 3, 1.0)
    data, scales = oracle.q4_quantize(w)
    return x, y0, data, scales


@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
@pytest.mark.parametrize("m,k,n", [(200, 320, 520), (1, 64, 72), (129, 96, 40), (683, 1024, 1000), (64, 4096, 768), (300, 2080, 256)])
def test_fused_equals_dequant_then_gemm(ctx, oracle, hb200, out, m, k, n):
    if out == OUT_SWIGLU and n % 2:
        pytest.skip("odd n")
    x, y0, data, scales = q4_inputs(oracle, m, k, n)
    d_q, d_s, d_x, d_w = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x), ctx.alloc(n * k * 2)
    ctx.dequant_q4(k, n)(1, d_q, d_s, d_w)
    wdq = oracle.q4_dequant(data, scales, n, k)
    want = oracle.gemm_f64(x, wdq, out, y0)
    d_ref, dtype, shape = out_buffer(ctx, out, m, n, y0)
    ctx.gemm(k, n, out, rows_max=m)(m, d_w, d_x, d_ref)
    ctx.sync()
    ref = d_ref.download(dtype, shape)
    within_contract(oracle, want, ref, "dequant + gemm")
    for tile_n in (256, 128):
        for m_first in (1, 0):
            d_y, _, _ = out_buffer(ctx, out, m, n, y0)
            kern = ctx.gemm_q4(k, n, out, tile_n=tile_n, m_first=m_first, rows_max=m)
            assert kern.name.startswith("gemm_q4_")
            kern(m, d_q, d_x, d_y, d_s)
            ctx.sync()
            got = d_y.download(dtype, shape)
            assert np.array_equal(got.view(np.uint32 if out == OUT_F32 else np.uint16), ref.view(np.uint32 if out == OUT_F32 else np.uint16)), f"{kern.name}: differs from dequant_q4 + the bf16 GEMM"
            within_contract(oracle, want, got, kern.name)


def test_rows_beyond_m_untouched_and_any_m(ctx, oracle):
    rows_max, k, n = 300, 512, 640
    x, y0, data, scales = q4_inputs(oracle, rows_max, k, n)
    d_q, d_s, d_x = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x)
    want = oracle.gemm_f64(x, oracle.q4_dequant(data, scales, n, k))
    kern = ctx.gemm_q4(k, n, OUT_BF16, rows_max=rows_max)
    for m in (rows_max, rows_max - rows_max // 3 - 3, 1):
        d_y = ctx.to_device(np.full((rows_max, n), 0x7FC1, dtype=np.uint16))
        kern(m, d_q, d_x, d_y, d_s)
        ctx.sync()
        got = d_y.download(np.uint16, (rows_max, n))
        assert np.all(got[m:] == 0x7FC1)
        within_contract(oracle, want[:m], got[:m], f"{kern.name} m={m}")


@pytest.mark.parametrize("m,k,n,out", [(2048, 4096, 6144, OUT_BF16), (512, 4096, 24576, OUT_SWIGLU), (2048, 12288, 4096, OUT_RESIDUAL)])
def test_layer_shapes_full_size(ctx, oracle, hb200, m, k, n, out):
    """The 9B-class shapes with random nibbles and scales (any bytes are valid Q4_0): every bit against dequant + GEMM."""
    rng = np.random.default_rng(k + n)
    blocks = n * k // 32
    data = rng.integers(0, 256, size=blocks * 16, dtype=np.uint8)
    scales = (rng.random(blocks, dtype=np.float32) * 0.02 + 0.001).astype(np.float16).view(np.uint16)
    x = oracle.normal((m, k), 41, m, 1.0)
    y0 = oracle.normal((m, n), 42, 3, 1.0)
    own = hb200.Context(0)  # a context of its own: a few hundred MB, released at the end
    try:
        d_q, d_s, d_x, d_w = own.to_device(data), own.to_device(scales), own.to_device(x), own.alloc(n * k * 2)
        own.dequant_q4(k, n)(1, d_q, d_s, d_w)
        d_ref, dtype, shape = out_buffer(own, out, m, n, y0)
        d_y, _, _ = out_buffer(own, out, m, n, y0)
        own.gemm(k, n, out, rows_max=m)(m, d_w, d_x, d_ref)
        kern = own.gemm_q4(k, n, out, rows_max=m)
        kern(m, d_q, d_x, d_y, d_s)
        own.sync()
        assert np.array_equal(d_y.download(dtype, shape), d_ref.download(dtype, shape)), kern.name
        rows = [0, m // 2, m - 1]
        wdq = oracle.q4_dequant(data, scales, n, k)
        want = oracle.gemm_f64_rows(x, wdq, rows, out, y0)
        within_contract(oracle, want[rows], d_y.download(dtype, shape)[rows], f"{kern.name} sampled rows")
    finally:
        own.close()


def test_selection_q4_fuse(ctx, oracle, hb200):
    m, k, n = 256, 1024, 1536
    x, y0, data, scales = q4_inputs(oracle, m, k, n)
    d_q, d_s, d_x, d_w, d_y = ctx.to_device(data), ctx.to_device(scales), ctx.to_device(x), ctx.alloc(n * k * 2), ctx.alloc(m * n * 2)
    want = oracle.gemm_f64(x, oracle.q4_dequant(data, scales, n, k))

    def run(ks):
        d_y.zero()
        if len(ks) == 1:
            ks[0](m, d_q, d_x, d_y, d_s)
        else:
            ks[0](1, d_q, d_s, d_w)
            ks[1](m, d_w, d_x, d_y)
        ctx.sync()
        return d_y.download(np.uint16, (m, n))

    outs = []
    for tune, count in (("q4.fuse=1", 1), ("q4.fuse=0", 2), ("", None)):
        sel = hb200.Selector(ctx, hb200.Tune(tune))
        try:
            ks = sel.gemm_q4(k, n, OUT_BF16, d_q, d_s, d_w, d_x, d_y, m)
            assert count is None or len(ks) == count
            if not tune:
                log = sel.log()
                assert f"gemm {k}x{n} Bf16 q4, {m} rows: dequant+gemm" in log and "fused128x256" in log
                assert [k_.name for k_ in sel.gemm_q4(k, n, OUT_BF16, d_q, d_s, d_w, d_x, d_y, m)] == [k_.name for k_ in ks]  # cached
            got = run(ks)
            within_contract(oracle, want, got, tune or "timed")
            outs.append(got)
        finally:
            sel.close()
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    for bad in (dict(k=100, n=64), dict(k=64, n=64, tile_n=64), dict(k=64, n=63, out=OUT_SWIGLU)):
        with pytest.raises(hb200.HbError):
            ctx.gemm_q4(**bad)
