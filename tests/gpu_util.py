"""Helpers of the GPU parity tests: run a kernel through the C ABI on seeded inputs and compare
with the CPU oracle under the engine's contract."""
import numpy as np

from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU, SEED_W, SEED_X, SEED_Y


def gemm_inputs(oracle, m, k, n):
    x = oracle.normal((m, k), SEED_X, 1, 1.0)
    w = oracle.normal((n, k), SEED_W, 2, k**-0.5)
    y0 = oracle.normal((m, n), SEED_Y, 5, 1.0)
    return x, w, y0


def out_buffer(ctx, out, m, n, y0):
    if out == OUT_F32:
        return ctx.alloc(m * n * 4), np.float32, (m, n)
    if out == OUT_RESIDUAL:
        return ctx.to_device(y0), np.uint16, (m, n)
    if out == OUT_SWIGLU:
        return ctx.alloc(max(16, m * (n // 2) * 2)), np.uint16, (m, n // 2)
    return ctx.alloc(max(16, m * n * 2)), np.uint16, (m, n)


def within_contract(oracle, want, got, what):
    """<= 1 bf16 ulp on >= 99.9 % of the elements, and max|err| <= max|ref| / 64 as a hard limit."""
    if want.dtype == np.float32:
        scale = max(float(np.abs(want).max()), 1e-6)
        err = float(np.abs(want - got).max())
        assert err <= 2e-6 * scale * 64 + 1e-5 * scale, f"{what}: f32 output off by {err} of {scale}"
        return
    c = oracle.compare(want, got)
    # The 99.9 % is a rate. On a small sample (under 100 000 elements) the count of outliers is tested against that
    # rate with three standard deviations of a Poisson count of slack (one element at least); large samples get none.
    lam = 1e-3 * c.count
    bound = lam if c.count >= 100000 else max(lam + 3.0 * lam**0.5, 1.0)
    assert c.over_1ulp <= bound, f"{what}: {c.over_1ulp}/{c.count} elements over 1 bf16 ulp (max {c.max_ulp})"
    assert c.max_abs_err <= c.max_abs_ref / 64, f"{what}: max err {c.max_abs_err} over 1/64 of {c.max_abs_ref}"


def run_gemm(ctx, oracle, m, k, n, out, **desc):
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    d_y, dtype, shape = out_buffer(ctx, out, m, n, y0)
    kern = ctx.gemm(k, n, out, rows_max=m, **desc)
    kern(m, d_w, d_x, d_y)
    ctx.sync()
    return kern, (x, w, y0), d_y.download(dtype, shape)
