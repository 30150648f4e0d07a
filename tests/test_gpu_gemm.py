"""Parity of the tcgen05 prefill GEMM with the f64-accumulated oracle, through the C ABI.
Tolerance (the engine's contract): <= 1 bf16 ulp on >= 99.9 % of elements, hard limit
max|err| <= max|ref|/64. Edge cases follow the reference's: a last block whose row count is a
multiple of no tile (qwen.rs:2514), columns and K that are multiples of no tile, one row."""
import numpy as np
import pytest

from gpu_util import gemm_inputs, out_buffer, run_gemm, within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU, SEED_W, SEED_X

pytestmark = pytest.mark.gpu

MODES = [OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU]


@pytest.mark.parametrize("tile_n", [64, 128, 256])
@pytest.mark.parametrize("out", MODES)
def test_small_ragged_all_modes(ctx, oracle, out, tile_n):
    m, k, n = 200, 320, 520  # no extent is a multiple of its tile
    kern, (x, w, y0), got = run_gemm(ctx, oracle, m, k, n, out, tile_n=tile_n)
    within_contract(oracle, oracle.gemm_f64(x, w, out, y0), got, kern.name)


@pytest.mark.parametrize("m", [1, 3, 17, 63, 65, 127, 129, 683])
def test_row_counts_that_fit_no_tile(ctx, oracle, m):
    k, n = 256, 384
    for out in (OUT_BF16, OUT_RESIDUAL):
        kern, (x, w, y0), got = run_gemm(ctx, oracle, m, k, n, out)
        within_contract(oracle, oracle.gemm_f64(x, w, out, y0), got, f"{kern.name} m={m}")


@pytest.mark.parametrize("k,n", [(8, 8), (72, 72), (1000, 2040), (64, 6), (4096, 100)])
def test_k_and_n_tails(ctx, oracle, k, n):
    # K a multiple of 8 only (the TMA row rule), N with a partial last tile and rows that are not 16-byte multiples
    for out in (OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU):
        if out == OUT_SWIGLU and n % 2:
            continue
        kern, (x, w, y0), got = run_gemm(ctx, oracle, 70, k, n, out, tile_n=128)
        within_contract(oracle, oracle.gemm_f64(x, w, out, y0), got, kern.name)


@pytest.mark.parametrize("out", MODES)
@pytest.mark.parametrize("m,k,n,tile_n", [(200, 320, 520, 64), (64, 4096, 768, 256), (1, 2048, 264, 128), (683, 1024, 1024, 256), (300, 8192, 256, 128), (129, 72, 40, 64)])
def test_stream_k_forms(ctx, oracle, out, m, k, n, tile_n):
    # tiles cut across CTAs and completed through the scratch partials: two-way cuts (many tiles) and
    # many-way K splits (fewer tiles than SMs), ragged extents, every output mode
    kern, (x, w, y0), got = run_gemm(ctx, oracle, m, k, n, out, tile_n=tile_n, stream_k=1)
    assert kern.name.startswith("gemm_sk_")
    within_contract(oracle, oracle.gemm_f64(x, w, out, y0), got, kern.name)


def test_stream_k_repeated_launches_and_config1(ctx, oracle):
    # launches are told apart by an epoch: the same kernel object run many times back to back stays right
    m, k, n = 512, 1024, 4096
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w, d_y = ctx.to_device(x), ctx.to_device(w), ctx.alloc(m * n * 2)
    kern = ctx.gemm(k, n, OUT_BF16, rows_max=m, stream_k=1)
    want = oracle.gemm_f64(x, w)
    for _ in range(20):
        kern(m, d_w, d_x, d_y)
    ctx.sync()
    within_contract(oracle, want, d_y.download(np.uint16, (m, n)), kern.name)
    first = d_y.download(np.uint16, (m, n))
    for _ in range(3):
        d_y.zero()
        kern(m, d_w, d_x, d_y)
        ctx.sync()
        assert np.array_equal(first, d_y.download(np.uint16, (m, n)))  # a fixed summation order: the same bits every run


@pytest.mark.parametrize("tile_n", [256, 192])
@pytest.mark.parametrize("out", MODES)
@pytest.mark.parametrize("m,k,n", [(300, 320, 520), (256, 64, 256), (1, 64, 72), (683, 1024, 1000), (2048, 4096, 1024), (257, 72, 40)])
def test_cta_pair_form(ctx, oracle, out, m, k, n, tile_n):
    # two CTAs of a cluster share a 256 x 256 (or 256 x 192) tile (tcgen05 cta_group::2): rows and columns that fill only
    # one CTA's half, ragged extents, every output mode
    if out == OUT_SWIGLU and n % 2:
        pytest.skip("odd n")
    kern, (x, w, y0), got = run_gemm(ctx, oracle, m, k, n, out, cta_pair=1, tile_n=tile_n)
    assert kern.name.startswith("gemm_pair_") and f"_t256x{tile_n}_" in kern.name
    within_contract(oracle, oracle.gemm_f64(x, w, out, y0), got, kern.name)


@pytest.mark.parametrize("out", MODES)
@pytest.mark.parametrize("m,k,n,splits", [(300, 320, 520, (2, 5)), (256, 128, 256, (2,)), (1, 1024, 72, (3, 16)), (683, 1024, 1000, (2, 7)), (512, 4096, 1024, (4, 9)), (1024, 200, 264, (3,))])
def test_cta_pair_split_k_form(ctx, oracle, hb200, out, m, k, n, splits):
    # every 256 x 256 tile as S work items over equal slices of K, the f32 partials summed in slice order by whoever
    # finishes a quarter of the tile last: the contract holds, and the bits do not depend on who that was
    if out == OUT_SWIGLU and n % 2:
        pytest.skip("odd n")
    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    want = oracle.gemm_f64(x, w, out, y0)
    for sp in splits:
        kern = ctx.gemm(k, n, out, rows_max=m, cta_pair=1, split_k=sp)
        assert kern.name.startswith("gemm_pair_") and kern.name.endswith(f"_k{sp}")
        outs = []
        for _ in range(3):  # the counters are back at zero after every launch
            d_y, dtype, shape = out_buffer(ctx, out, m, n, y0)
            kern(m, d_w, d_x, d_y)
            ctx.sync()
            outs.append(d_y.download(dtype, shape))
        within_contract(oracle, want, outs[0], kern.name)
        assert all(np.array_equal(outs[0].view(np.uint8), o.view(np.uint8)) for o in outs[1:]), f"{kern.name}: the bits change from launch to launch"


def test_cta_pair_split_k_limits(ctx, hb200):
    for bad in (dict(split_k=65), dict(split_k=2, y_shards=2, out=OUT_F32)):
        with pytest.raises(hb200.HbError) as e:
            ctx.gemm(1024, 512, **dict(dict(out=OUT_BF16, cta_pair=1, rows_max=256), **bad))
        assert e.value.status == hb200.UNSUPPORTED
    kern = ctx.gemm(128, 512, OUT_BF16, rows_max=2048, cta_pair=1, split_k=2)
    buf = ctx.alloc(2048 * 512 * 2)
    with pytest.raises(hb200.HbError) as e:
        kern(2048, buf, buf, buf)  # the partial-tile scratch is sized for short blocks
    assert e.value.status == hb200.INVALID and "1024 rows" in e.value.message
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(128, 512, OUT_BF16, rows_max=256, cta_pair=1, split_k=3)(256, buf, buf, buf)  # K = 128 is two blocks of 64
    assert e.value.status == hb200.INVALID
    # the stream-K form refuses a pipeline smaller than one f32 partial tile (it would land a partial beyond its shared memory)
    with pytest.raises(hb200.HbError) as e:
        ctx.gemm(1024, 512, OUT_BF16, rows_max=256, stream_k=1, tile_n=256, stages=2)
    assert e.value.status == hb200.UNSUPPORTED and "partial tile" in e.value.message
    ctx.gemm(1024, 512, OUT_BF16, rows_max=256, stream_k=1, tile_n=128, stages=2)  # 64 KiB of pipeline for a 64 KiB tile: fits


def test_cta_pair_matches_single_cta_bits(ctx, oracle):
    # the pair changes who stages what, not the order of the K loop: same bits as the 128 x 256 kernel
    m, k, n = 512, 2048, 768
    a = run_gemm(ctx, oracle, m, k, n, OUT_BF16, cta_pair=1)[2]
    b = run_gemm(ctx, oracle, m, k, n, OUT_BF16, tile_n=256)[2]
    c = run_gemm(ctx, oracle, m, k, n, OUT_BF16, cta_pair=1, tile_n=192)[2]
    assert np.array_equal(a, b) and np.array_equal(a, c)


@pytest.mark.parametrize("form", [dict(cta_pair=1), dict(cta_pair=1, tile_n=192), dict(tile_n=256), dict(tile_n=128), dict(tile_n=64), dict(stream_k=1, tile_n=128), dict(stream_k=1, tile_n=64)], ids=str)
def test_gemm_chain_with_overlapped_launches(ctx, oracle, form):
    """hb_set_launch_overlap: every GEMM of a chain starts under the tail of the one before (its first weight stages are
    requested before it waits for its predecessor). A chain with true dependencies (each product is the next one's
    input, the last adds into a residual twice): the same bits as with plain launches, several times over."""
    m, dims = 600, (512, 1280, 768, 512)
    x0 = oracle.normal((m, dims[0]), SEED_X, 1, 1.0)
    ws = [oracle.normal((dims[i + 1], dims[i]), SEED_W, 2 + i, dims[i] ** -0.5) for i in range(3)]
    d_ws = [ctx.to_device(w) for w in ws]
    d_x = ctx.to_device(x0)
    bufs = [d_x] + [ctx.alloc(m * dims[i + 1] * 2) for i in range(3)]
    ops = [(ctx.gemm(dims[i], dims[i + 1], OUT_BF16 if i < 2 else OUT_RESIDUAL, rows_max=m, **form), m, d_ws[i], bufs[i], bufs[i + 1]) for i in range(3)]
    ops = ops + [ops[2]]  # the residual product twice in a row: read-modify-write of the same rows by neighbours

    def once():
        bufs[3].zero()
        ctx.run(ops)
        ctx.sync()
        return bufs[3].download(np.uint16, (m, dims[3]))

    plain = once()
    ctx.set_launch_overlap(True)
    try:
        for _ in range(5):
            assert np.array_equal(plain, once())
    finally:
        ctx.set_launch_overlap(False)


def test_config1_dense_gemm(ctx, oracle):
    # the small dense GEMM: M=512, K=1024, N=4096
    for m_first in (1, 0):
        kern, (x, w, y0), got = run_gemm(ctx, oracle, 512, 1024, 4096, OUT_BF16, m_first=m_first)
        within_contract(oracle, oracle.gemm_f64(x, w), got, kern.name)


def test_rows_beyond_m_are_untouched_and_partial_block(ctx, oracle):
    # one kernel object serves every 1 <= m <= rows_max; rows past m keep their canary
    rows_max, k, n = 300, 512, 640
    x, w, y0 = gemm_inputs(oracle, rows_max, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    kern = ctx.gemm(k, n, OUT_BF16, rows_max=rows_max)
    want = oracle.gemm_f64(x, w)
    for m in (rows_max, rows_max - rows_max // 3 - 3, 1):
        canary = np.full((rows_max, n), 0x7FC1, dtype=np.uint16)
        d_y = ctx.to_device(canary)
        kern(m, d_w, d_x, d_y)
        ctx.sync()
        got = d_y.download(np.uint16, (rows_max, n))
        assert np.all(got[m:] == 0x7FC1)
        within_contract(oracle, want[:m], got[:m], f"{kern.name} m={m}")


def test_residual_rounds_twice(ctx, oracle):
    # y = bf16(f32(y_old) + f32(bf16(acc))): differs from bf16(y_old + acc) on a measurable share of elements
    m, k, n = 128, 512, 256
    kern, (x, w, y0), got = run_gemm(ctx, oracle, m, k, n, OUT_RESIDUAL)
    want = oracle.gemm_f64(x, w, OUT_RESIDUAL, y0)
    within_contract(oracle, want, got, kern.name)
    acc = oracle.gemm_f64(x, w, OUT_F32)
    from oracle_lib import bf16_to_f32

    once = (bf16_to_f32(y0) + acc).astype(np.float32)
    once16 = ((once.view(np.uint32).astype(np.uint64) + 0x7FFF + ((once.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
    assert (once16 != want).mean() > 1e-3  # the oracle really has the double rounding ...
    assert (got != want).mean() < (once16 != want).mean()  # ... and the kernel follows it


def test_swiglu_fused_equals_apart(ctx, oracle):
    # "each fusion gives the same bits as the kernels it replaces" (README.md:57): fused epilogue == GEMM + swiglu_rows
    m, k, inter = 150, 512, 384
    x, w, _ = gemm_inputs(oracle, m, k, 2 * inter)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    d_gu, d_h1, d_h2 = ctx.alloc(m * 2 * inter * 2), ctx.alloc(m * inter * 2), ctx.alloc(m * inter * 2)
    ctx.gemm(k, 2 * inter, OUT_BF16, rows_max=m)(m, d_w, d_x, d_gu)
    ctx.swiglu_rows(inter)(m, d_gu, d_h1)
    ctx.gemm(k, 2 * inter, OUT_SWIGLU, rows_max=m)(m, d_w, d_x, d_h2)
    ctx.sync()
    assert np.array_equal(d_h1.download(np.uint16, (m, inter)), d_h2.download(np.uint16, (m, inter)))


def test_tile_forms_agree_bitwise(ctx, oracle):
    # the tile width changes the schedule, not the per-element accumulation order along K
    m, k, n = 256, 2048, 768
    outs = [run_gemm(ctx, oracle, m, k, n, OUT_BF16, tile_n=t, m_first=f)[2] for t in (64, 128, 256) for f in (0, 1)]
    for o in outs[1:]:
        assert np.array_equal(outs[0], o)


def test_reference_inputs_xorshift_and_random16(ctx, oracle):
    # the reference's own input streams: autotune inputs in [-1, 1) (qwen.rs:2613) and the probe's
    # magnitudes 2^-6..2^-1 (herbert-metal-probe.rs:446)
    m, k, n = 192, 1024, 512
    for x, w in ((oracle.xorshift16((m, k), 0x9E3779B9), oracle.xorshift16((n, k), 0x2545F491)), (oracle.random16((m, k), 1), oracle.random16((n, k), 2))):
        d_x, d_w, d_y = ctx.to_device(x), ctx.to_device(w), ctx.alloc(m * n * 2)
        ctx.gemm(k, n, OUT_BF16, rows_max=m)(m, d_w, d_x, d_y)
        ctx.sync()
        within_contract(oracle, oracle.gemm_f64(x, w), d_y.download(np.uint16, (m, n)), "reference input streams")


@pytest.mark.parametrize(
    "m,k,n,out",
    [
        (2048, 4096, 6144, OUT_BF16),       # qkv
        (2048, 4096, 4096, OUT_RESIDUAL),   # o_proj
        (2048, 4096, 24576, OUT_SWIGLU),    # gate/up + SiLU*mul
        (2048, 12288, 4096, OUT_RESIDUAL),  # down
        (64, 4096, 6144, OUT_BF16),
        (512, 12288, 4096, OUT_RESIDUAL),
    ],
)
def test_config3_layer_shapes_full_size(ctx, oracle, m, k, n, out):
    """Full-size 9B-class shapes. The CPU oracle covers a sample of rows (every element of those rows);
    every element of the output is compared against an f64 matmul on the GPU whose own result is pinned
    to the oracle on the sampled rows."""
    import torch

    x, w, y0 = gemm_inputs(oracle, m, k, n)
    d_x, d_w = ctx.to_device(x), ctx.to_device(w)
    d_y, dtype, shape = out_buffer(ctx, out, m, n, y0)
    kern = ctx.gemm(k, n, out, rows_max=m)
    kern(m, d_w, d_x, d_y)
    ctx.sync()
    got = d_y.download(dtype, shape)
    rows = sorted(set([0, m - 1] + list(np.random.default_rng(m + n).integers(0, m, size=14))))
    want_rows = oracle.gemm_f64_rows(x, w, rows, out, y0)
    within_contract(oracle, want_rows[rows], got[rows], f"{kern.name} sampled rows")
    # the reference's own spot pattern: rows {0, M-1} x cols {0..3, N-4..N-1} (herbert-metal-probe.rs:788-799)
    nc = shape[1]
    cols = list(range(4)) + list(range(nc - 4, nc))
    spot_want = np.ascontiguousarray(want_rows[[0, m - 1]][:, cols])
    spot_got = np.ascontiguousarray(got[[0, m - 1]][:, cols])
    spot = oracle.compare(spot_want, spot_got)
    assert spot.max_abs_err <= max(spot.max_abs_ref, 1e-3) / 64, "the probe's 16 spot outputs"
    # all elements: f64 product on the GPU, the epilogue in torch with the same roundings
    tx = torch.from_numpy(x.view(np.int16)).cuda().view(torch.bfloat16).double()
    tw = torch.from_numpy(w.view(np.int16)).cuda().view(torch.bfloat16).double()
    acc = (tx @ tw.t()).float().bfloat16()
    if out == OUT_RESIDUAL:
        ty = torch.from_numpy(y0.view(np.int16)).cuda().view(torch.bfloat16)
        full = (ty.float() + acc.float()).bfloat16()
    elif out == OUT_SWIGLU:
        g, u = acc[:, : n // 2].float(), acc[:, n // 2 :].float()
        full = ((g * (1.0 / (1.0 + torch.exp(-g)))) * u).bfloat16()
    else:
        full = acc
    full16 = full.view(torch.int16).cpu().numpy().view(np.uint16)
    c = oracle.compare(want_rows[rows], full16[rows])  # the GPU-side f64 reference is itself pinned to the oracle
    assert c.over_1ulp <= 1e-3 * c.count
    within_contract(oracle, full16, got, f"{kern.name} all elements")
