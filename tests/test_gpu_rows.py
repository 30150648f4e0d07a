"""The row-wise kernels around the products (RMSNorm, argmax, the MoE block's end): bit-exact with the oracle, which
is itself pinned to the independent restatement in tests/golden."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
G = np.load(__import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "golden.npz"))


@pytest.mark.parametrize("plus_one", [False, True])
def test_rmsnorm_golden_and_shapes(ctx, oracle, plus_one):
    x, w = G["norm_x"], G["norm_w"]
    d_x, d_w, d_y = ctx.to_device(x), ctx.to_device(w), ctx.alloc(x.size * 2)
    ctx.rmsnorm(x.shape[1], 1e-6, plus_one)(x.shape[0], d_x, d_w, d_y)
    ctx.sync()
    assert np.array_equal(d_y.download(np.uint16, x.shape), G["norm_out_p1" if plus_one else "norm_out"])
    # model widths, a ragged one (scalar path), many rows; in place
    for rows, d in ((5, 4096), (3, 5120), (2048, 2048), (7, 1000), (2, 256), (3, 24)):
        x = oracle.normal((rows, d), 3, d, 2.0)
        w = oracle.normal((d,), 4, d, 0.3)
        d_x, d_w = ctx.to_device(x), ctx.to_device(w)
        ctx.rmsnorm(d, 1e-5, plus_one)(rows, d_x, d_w, d_x)
        ctx.sync()
        assert np.array_equal(d_x.download(np.uint16, (rows, d)), oracle.rmsnorm_rows(x, w, 1e-5, plus_one)), (rows, d)


def test_argmax_golden_and_lm_head_width(ctx, oracle):
    lg = G["argmax_logits"]
    d_l, d_i = ctx.to_device(lg), ctx.alloc(lg.shape[0] * 4)
    kern = ctx.argmax(lg.shape[1], rows_max=8)
    for _ in range(2):  # the kernel clears its own scratch
        kern(lg.shape[0], d_l, d_i)
        ctx.sync()
        assert np.array_equal(d_i.download(np.uint32, (lg.shape[0],)), G["argmax_out"])
    rows, n = 8, 151936
    lg = oracle.normal((rows, n), 9, 1, 4.0)
    lg[2, 70000] = lg[2, 140000] = 0x4200  # a tie of the maximum across chunks
    lg[3, :] = 0xFF80
    lg[3, n - 1] = 0xC47A                  # one finite value in the last place
    d_l, d_i = ctx.to_device(lg), ctx.alloc(rows * 4)
    kern = ctx.argmax(n, rows_max=rows)
    kern(rows, d_l, d_i)
    ctx.sync()
    got = d_i.download(np.uint32, (rows,))
    assert np.array_equal(got, oracle.argmax_rows(lg)) and got[2] == 70000 and got[3] == n - 1
    kern(1, d_l, d_i)  # fewer rows than it was built for
    ctx.sync()
    assert d_i.download(np.uint32, (1,))[0] == got[0]


def test_moe_out_golden_and_shapes(ctx, oracle):
    names = ("moe_out_xn", "moe_out_gate", "moe_out_experts", "moe_out_shared", "moe_out_x")
    bufs = [ctx.to_device(G[n]) for n in names]
    rows, d = G["moe_out_x"].shape
    ctx.moe_out(d)(rows, *bufs)
    ctx.sync()
    assert np.array_equal(bufs[4].download(np.uint16, (rows, d)), G["moe_out_out"])
    for rows, d in ((2048, 2048), (3, 1000), (5, 4096)):
        xn, ex, sh, x = (oracle.normal((rows, d), 20 + i, d, s) for i, s in enumerate((1.0, 0.6, 0.6, 1.0)))
        gate = oracle.normal((d,), 30, d, d**-0.5)
        bufs = [ctx.to_device(a) for a in (xn, gate, ex, sh, x)]
        ctx.moe_out(d)(rows, *bufs)
        ctx.sync()
        assert np.array_equal(bufs[4].download(np.uint16, (rows, d)), oracle.moe_out(xn, gate, ex, sh, x)), (rows, d)
