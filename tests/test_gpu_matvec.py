"""Parity of the decode matvec (M = 1..8) with the f64-accumulated oracle, through the C ABI."""
import numpy as np
import pytest

from gpu_util import gemm_inputs, out_buffer, within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU

pytestmark = pytest.mark.gpu


def run(ctx, oracle, m, k, n, out, **form):
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    d_y, dtype, shape = out_buffer(ctx, out, m, n, y0)
    kern = ctx.matvec(k, n, out, rows_max=m, **form)
    kern(m, d_w, d_x, d_y)
    ctx.sync()
    return kern, oracle.gemm_f64(x, w, out, y0), d_y.download(dtype, shape)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
def test_every_form(ctx, oracle, m, out):
    k, n = 1024, 328  # n is a multiple of no row group, so the last group is ragged
    for rpw in (1, 2, 4, 8):
        for split in (1, 2, 4):
            for persist in (0, 1):
                if out == OUT_SWIGLU and rpw == 1:
                    continue
                kern, want, got = run(ctx, oracle, m, k, n, out, rows_per_warp=rpw, split=split, persist=persist)
                within_contract(oracle, want, got, f"{kern.name} m={m}")


@pytest.mark.parametrize("m", [2, 3, 4, 7, 8])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
def test_activation_stationary_forms(ctx, oracle, hb200, m, out):
    # K split across the threads of a block, activations widened once in registers
    for k, n in ((1024, 330), (4096, 512), (72, 40), (2560, 96)):
        for rpw in (2, 4):
            kern, want, got = run(ctx, oracle, m, k, n, out, rows_per_warp=rpw, x_stationary=1)
            assert f"_x{rpw}" in kern.name
            within_contract(oracle, want, got, f"{kern.name} m={m}")
    with pytest.raises(hb200.HbError) as e:
        ctx.matvec(12288, 64, rows_max=8, x_stationary=1)  # K * rows beyond what the registers hold
    assert e.value.status == hb200.UNSUPPORTED


def test_m1_equals_reference_lane_order_closely(ctx, oracle):
    # M = 1 against the reference's own order of operations (32 lanes striding K by chunks of 8,
    # butterfly sum): the same sums up to the association of the lane fold
    k, n = 4096, 512
    x, w, _ = gemm_inputs(oracle, 1, k, n)
    d_x, d_w, d_y = ctx.to_device(x), ctx.to_device(w), ctx.alloc(n * 2)
    ctx.matvec(k, n, OUT_BF16, rows_max=1, rows_per_warp=1)(1, d_w, d_x, d_y)
    ctx.sync()
    got = d_y.download(np.uint16, (n,))
    assert np.array_equal(got, oracle.matvec_ref_order(x, w))  # same lane striding, same butterfly: same bits


@pytest.mark.parametrize("m", [1, 4, 8])
def test_config2_shapes(ctx, oracle, m):
    # the decode projections of the 9B-class layer: K=4096, N=12288 (and the LM-head-like N=151936 on a row sample of W)
    k, n = 4096, 12288
    kern, want, got = run(ctx, oracle, m, k, n, OUT_BF16, rows_per_warp=4)
    within_contract(oracle, want, got, f"{kern.name} m={m}")


def test_lm_head_shape(ctx, oracle):
    k, n, m = 4096, 151936, 4
    x = oracle.normal((m, k), 1, 1, 1.0)
    w = oracle.normal((n, k), 2, 2, k**-0.5)
    d_x, d_w, d_y = ctx.to_device(x), ctx.to_device(w), ctx.alloc(m * n * 2)
    kern = ctx.matvec(k, n, OUT_BF16, rows_max=m, rows_per_warp=4)
    kern(m, d_w, d_x, d_y)
    ctx.sync()
    got = d_y.download(np.uint16, (m, n))
    cols = np.concatenate([np.arange(0, 4096), np.arange(n - 4096, n), np.random.default_rng(0).integers(0, n, 8192)])
    want = oracle.gemm_f64(x, np.ascontiguousarray(w[cols]))
    within_contract(oracle, want, np.ascontiguousarray(got[:, cols]), kern.name)


def test_k_multiple_of_8_only_and_unsupported(ctx, oracle, hb200):
    kern, want, got = run(ctx, oracle, 2, 72, 40, OUT_BF16, rows_per_warp=2, split=2)
    within_contract(oracle, want, got, kern.name)
    with pytest.raises(hb200.HbError) as e:
        ctx.matvec(100, 64)  # K = 100 is not a multiple of 8 (reference: kernels.rs:147)
    assert e.value.status == hb200.UNSUPPORTED
    with pytest.raises(hb200.HbError):
        ctx.matvec(64, 64, rows_max=9)
    with pytest.raises(hb200.HbError):
        ctx.matvec(64, 64, OUT_SWIGLU, rows_per_warp=1)


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 40, 64])
@pytest.mark.parametrize("out", [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU])
def test_tensor_core_forms(ctx, oracle, hb200, m, out):
    # the weight stream on the tensor cores: W rows are the wide MMA operand, the 1..64 activation rows the narrow one
    for k, n in ((1024, 330), (4096, 512), (72, 40), (2560, 96), (8192, 1200)):
        if out == OUT_SWIGLU and k > 4096:
            continue  # three roundings after a sum of 8192 f32 terms: outside what the one-ulp rate is stated for
        for ks in (1, 2, 3):  # whole feature blocks per CTA; evenly dealt (block, k-block) units; blocks sized to the grid
            for kps in (1, 2, 4):
                if out == OUT_SWIGLU and kps == 4:  # two weight tiles per K block: four blocks per stage leave room for one stage only
                    with pytest.raises(hb200.HbError) as e:
                        ctx.matvec(k, n, out, rows_max=m, tensor_core=ks, split=kps)
                    assert e.value.status == hb200.UNSUPPORTED
                    continue
                kern, want, got = run(ctx, oracle, m, k, n, out, tensor_core=ks, split=kps)
                assert kern.name.startswith("matvec_tc_") and ("_blk_", "_bal_", "_fit")[ks - 1] in kern.name and kern.name.endswith(f"x{kps}")
                within_contract(oracle, want, got, f"{kern.name} m={m}")


def test_tensor_core_form_twice_and_limits(ctx, oracle, hb200):
    # the split form leaves its counters at zero: a second launch of the same kernel object gives the same bits
    m, k, n = 8, 4096, 640
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    kern = ctx.matvec(k, n, OUT_BF16, rows_max=m, tensor_core=2)
    outs = []
    for _ in range(3):
        d_y = ctx.alloc(m * n * 2)
        kern(m, d_w, d_x, d_y)
        ctx.sync()
        outs.append(d_y.download(np.uint16, (m, n)))
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    within_contract(oracle, oracle.gemm_f64(x, w), outs[0], kern.name)
    for bad in (dict(rows_max=65, tensor_core=1), dict(rows_max=8, tensor_core=4)):
        with pytest.raises(hb200.HbError) as e:
            ctx.matvec(k, n, OUT_BF16, **bad)
        assert e.value.status == hb200.UNSUPPORTED


@pytest.mark.parametrize("m", [1, 4, 8])
def test_config2_shapes_tensor_core(ctx, oracle, m):
    k, n = 4096, 12288
    for ks in (1, 2, 3):
        kern, want, got = run(ctx, oracle, m, k, n, OUT_BF16, tensor_core=ks, split=2)
        within_contract(oracle, want, got, f"{kern.name} m={m}")


@pytest.mark.parametrize("m", [1, 3, 8])
def test_fused_argmax(ctx, oracle, hb200, m):
    # the projection also reports, per activation row, the first index of its largest bf16 output
    for k, n, form in ((1024, 3000, dict(rows_per_warp=2, split=2)), (4096, 12288, dict(rows_per_warp=4)), (512, 70, dict(rows_per_warp=1, persist=1)),
                       (4096, 151936, dict(rows_per_warp=2, split=2))):
        x = oracle.normal((m, k), 1, n, 1.0)
        w = oracle.normal((n, k), 2, n, k**-0.5)
        w[n // 3] = w[2 * n // 3]  # two equal rows of W: equal outputs, so ties between far-apart indices exist
        d_x, d_w, d_y, d_i = ctx.to_device(x), ctx.to_device(w), ctx.alloc(m * n * 2), ctx.alloc(m * 4)
        kern = ctx.matvec(k, n, OUT_BF16, rows_max=m, argmax=1, **form)
        assert kern.name.endswith("_p_argmax")  # always the persistent grid
        plain = ctx.matvec(k, n, OUT_BF16, rows_max=m, **form)
        d_y2 = ctx.alloc(m * n * 2)
        plain(m, d_w, d_x, d_y2)
        for _ in range(2):  # twice: the kernel clears its own scratch
            ctx.memset(d_i, 0xEE)
            kern(m, d_w, d_x, d_y, d_i)
            ctx.sync()
            logits = d_y.download(np.uint16, (m, n))
            assert np.array_equal(logits, d_y2.download(np.uint16, (m, n)))  # the same logits as without the fusion
            assert np.array_equal(d_i.download(np.uint32, (m,)), oracle.argmax_rows(logits))
        # index only: y stays untouched
        only = ctx.matvec(k, n, OUT_BF16, rows_max=m, argmax=2, **form)
        ctx.memset(d_y, 0)
        ctx.memset(d_i, 0xEE)
        only(m, d_w, d_x, d_y, d_i)
        ctx.sync()
        assert not d_y.download(np.uint16, (m, n)).any()
        assert np.array_equal(d_i.download(np.uint32, (m,)), oracle.argmax_rows(logits))
    with pytest.raises(hb200.HbError) as e:
        ctx.matvec(1024, 512, OUT_RESIDUAL, rows_max=1, argmax=1)
    assert e.value.status == hb200.UNSUPPORTED
