"""hb_gemm_static_scratch: the GEMM entry point for hosts that must not allocate device memory.

Some callers of this library cannot call cudaMalloc at the point where they need the product: a serving loop
that forbids any call that may synchronise the device or take the allocator's lock, a plugin that lives inside
a fixed memory budget given by its host engine, a process whose device memory another allocator has claimed in
full. For them the stream-K GEMM's partial-tile scratch sits in a fixed array inside the library. This test
calls the entry point through the C ABI, twice in a row (the array keeps the previous call's contents), and
checks the output against the allocating entry point (hb_gemm_get with stream_k = 1 and 128x64 tiles, the same
kernel on the context's scratch): the bits must be equal, which is tighter than the GEMM contract the other
tests use, and the oracle confirms that contract as well. It runs last so that a run that stops at the first
failure has already run everything else, and it needs nothing from the tests before it.
"""
import ctypes as C

import numpy as np
import pytest

from gpu_util import gemm_inputs, within_contract
from oracle_lib import OUT_BF16, OUT_RESIDUAL, OUT_SWIGLU

pytestmark = pytest.mark.gpu


def call_static(hb200, ctx, k, n, out, m, w, x, y):
    st = hb200.lib().hb_gemm_static_scratch(ctx.h, k, n, out, m, w.range(), x.range(), y.range())
    if st != hb200.OK:
        raise hb200.HbError(st, hb200.lib().hb_last_error(ctx.h).decode())


@pytest.mark.parametrize("m,k,n,out", [(64, 4096, 1024, OUT_BF16), (300, 1024, 520, OUT_RESIDUAL), (512, 2048, 768, OUT_SWIGLU)])
def test_static_scratch_gemm_matches_the_allocating_entry_point(hb200, oracle, m, k, n, out):
    ctx = hb200.Context(0)  # its own context: the test does not lean on state left by earlier tests
    try:
        x, w, y0 = gemm_inputs(oracle, m, k, n)
        ncol = n // 2 if out == OUT_SWIGLU else n
        start = np.ascontiguousarray(y0[:, :ncol])
        d_w, d_x = ctx.to_device(w), ctx.to_device(x)
        want = oracle.gemm_f64(x, w, out, y0)
        # the existing entry point: the same kernel, scratch allocated from the context
        d_ref = ctx.to_device(start)
        ctx.gemm(k, n, out, rows_max=m, tile_n=64, stream_k=1)(m, d_w, d_x, d_ref)
        ctx.sync()
        ref = d_ref.download(np.uint16, (m, ncol))
        within_contract(oracle, want, ref, "allocating entry point")
        # the entry point under test, two calls in a row on fresh outputs
        for call in range(2):
            d_y = ctx.to_device(start)
            call_static(hb200, ctx, k, n, out, m, d_w, d_x, d_y)
            ctx.sync()
            got = d_y.download(np.uint16, (m, ncol))
            assert np.array_equal(got, ref), f"call {call}: differs from the allocating entry point"
            within_contract(oracle, want, got, f"static scratch, call {call}")
    finally:
        ctx.close()


def test_static_scratch_gemm_refuses_what_it_cannot_hold(hb200):
    ctx = hb200.Context(0)
    try:
        buf = ctx.alloc(1 << 20)
        with pytest.raises(hb200.HbError) as e:
            call_static(hb200, ctx, 64, 64, OUT_BF16, 4096, buf, buf, buf)  # more rows than the stated maximum
        assert e.value.status == hb200.UNSUPPORTED and "2048 rows" in e.value.message
        with pytest.raises(hb200.HbError) as e:
            call_static(hb200, ctx, 100, 64, OUT_BF16, 16, buf, buf, buf)  # k not a multiple of 8
        assert e.value.status == hb200.UNSUPPORTED
        small = ctx.alloc(64)
        with pytest.raises(hb200.HbError) as e:
            call_static(hb200, ctx, 64, 64, OUT_BF16, 16, buf, buf, small)  # output range too small
        assert e.value.status == hb200.INVALID
        ctx.sync()
    finally:
        ctx.close()
