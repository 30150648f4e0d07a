"""Full-size parity of the forms the selection loop picks at the workloads' real shapes.

Every GEMM form that the load-time loop can choose for a 9B-class layer (the one-CTA 128x256 tile, the CTA pair,
stream-K with each tile width, and for blocks of at most 64 rows the two tensor-core weight streams) runs at
2048, 512 and 64 rows on the layer's own K and N; the 27B-class FFN runs at K=5120 -> N=2x17408 and
K=17408 -> N=5120 whole and as the shards of 2, 4 and 8 tensor-parallel ranks (widths 8704, 4352 and 2176, the
last one 8.5 pair tiles wide) emulated on one GPU; the LM-head-sized weight stream runs at N=151936.

Oracle: the CPU restatement computes a sample of rows (every element of them, f64 accumulation, one rounding)
and the probe's 16 spot outputs (rows {0, M-1} x columns {0..3, N-4..N-1}, src/bin/herbert-metal-probe.rs:788-799);
every element is compared with an f64 product on the GPU whose own result is pinned to the CPU rows first.
Tolerance (the engine's contract): at most 1 bf16 ulp on at least 99.9 % of the elements, max|err| <= max|ref|/64.
"""
import numpy as np
import pytest
import torch

from gpu_util import gemm_inputs, out_buffer, within_contract
from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU, SEED_X, SEED_Y
from test_dist_cpu import load_dist, n16, t16

pytestmark = pytest.mark.gpu


def _dev16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda().view(torch.bfloat16)


def _bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def f64_reference(x, w, out, y0, chunk=8192):
    """The product in f64 on the GPU with the output mode's roundings in torch; bf16 bits [m][n or n/2]."""
    tx = _dev16(x).double()
    tw = _dev16(w)
    n = w.shape[0]
    acc = torch.empty((x.shape[0], n), device="cuda", dtype=torch.bfloat16)
    for c in range(0, n, chunk):  # f64 copies of W a slab at a time
        acc[:, c : c + chunk] = (tx @ tw[c : c + chunk].double().t()).float().bfloat16()
    if out == OUT_RESIDUAL:
        return _bits((_dev16(y0).float() + acc.float()).bfloat16())
    if out == OUT_SWIGLU:
        g, u = acc[:, : n // 2].float(), acc[:, n // 2 :].float()
        return _bits(((g * (1.0 / (1.0 + torch.exp(-g)))) * u).bfloat16())
    return _bits(acc)


_last_w = {}  # the weights of the last (k, n): they do not depend on the row count, and the big ones take seconds to make


class Shape:
    """Inputs of one (m, k, n, out) on the host and the device, with the CPU rows and the pinned f64 reference."""

    def __init__(self, ctx, oracle, m, k, n, out):
        self.m, self.k, self.n, self.out = m, k, n, out
        if (k, n) in _last_w:
            self.w = _last_w[(k, n)]
            self.x, self.y0 = oracle.normal((m, k), SEED_X, 1, 1.0), oracle.normal((m, n), SEED_Y, 5, 1.0)  # as gemm_inputs makes them
        else:
            self.x, self.w, self.y0 = gemm_inputs(oracle, m, k, n)
            _last_w.clear()
            _last_w[(k, n)] = self.w
        self.d_x, self.d_w = ctx.to_device(self.x), ctx.to_device(self.w)
        self.rows = sorted(set([0, m - 1] + list(np.random.default_rng(m + n).integers(0, m, size=14))))
        self.want_rows = oracle.gemm_f64_rows(self.x, self.w, self.rows, out, self.y0)
        self.full = f64_reference(self.x, self.w, out, self.y0)
        c = oracle.compare(self.want_rows[self.rows], self.full[self.rows])
        assert c.over_1ulp <= 1e-3 * c.count, "the f64 product on the GPU is off the CPU oracle on the sampled rows"

    def check(self, ctx, oracle, kern):
        m = self.m
        d_y, dtype, shape = out_buffer(ctx, self.out, m, self.n, self.y0)
        kern(m, self.d_w, self.d_x, d_y)
        ctx.sync()
        got = d_y.download(dtype, shape)
        within_contract(oracle, self.want_rows[self.rows], got[self.rows], f"{kern.name} sampled rows")
        nc = shape[1]
        cols = list(range(4)) + list(range(nc - 4, nc))
        spot = oracle.compare(np.ascontiguousarray(self.want_rows[[0, m - 1]][:, cols]), np.ascontiguousarray(got[[0, m - 1]][:, cols]))
        assert spot.max_abs_err <= max(spot.max_abs_ref, 1e-3) / 64, f"{kern.name}: the probe's 16 spot outputs"
        within_contract(oracle, self.full, got, f"{kern.name} all elements")
        return got


@pytest.fixture()
def ctx(hb200):
    """A context per test: the buffers of these shapes (hundreds of MB each) are released when the test ends."""
    c = hb200.Context(0)
    yield c
    c.close()


LAYER_9B = [("qkv", 4096, 6144, OUT_BF16), ("o_proj", 4096, 4096, OUT_RESIDUAL), ("gate_up", 4096, 24576, OUT_SWIGLU), ("down", 12288, 4096, OUT_RESIDUAL)]


@pytest.mark.parametrize("m", [2048, 512])  # (the upper decorator varies fastest: both row counts of a shape share its weights)
@pytest.mark.parametrize("name,k,n,out", LAYER_9B, ids=[f"{s[0]}_{s[1]}x{s[2]}" for s in LAYER_9B])
def test_layer_9b_every_gemm_form(ctx, oracle, m, name, k, n, out):
    """The candidates of hb_select_gemm / hb_select_gate_up at 2048 and 512 rows: all must hold the contract, and the
    forms that keep the K order of the one-CTA kernel must give its bits."""
    s = Shape(ctx, oracle, m, k, n, out)
    base = s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m))
    pair = s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m, cta_pair=1))
    assert np.array_equal(pair, base), "the CTA pair changes who stages what, not the order of the K loop"
    for tile_n in (256, 128, 64):
        kern = ctx.gemm(k, n, out, rows_max=m, tile_n=tile_n, stream_k=1)
        assert kern.name.startswith("gemm_sk_")
        s.check(ctx, oracle, kern)
    for tile_n in (128, 64):
        assert np.array_equal(s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m, tile_n=tile_n)), base)
    assert np.array_equal(s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m, m_first=0)), base)
    if m <= 1024:  # the split-K candidates of a short block ("pair256x256k{S}")
        for sp in (2, 4, 9):
            kern = ctx.gemm(k, n, out, rows_max=m, cta_pair=1, split_k=sp)
            assert kern.name.endswith(f"_k{sp}")
            s.check(ctx, oracle, kern)


@pytest.mark.parametrize("name,k,n,out", LAYER_9B, ids=[f"{s[0]}_{s[1]}x{s[2]}" for s in LAYER_9B])
def test_layer_9b_64_rows_gemm_and_stream_forms(ctx, oracle, hb200, name, k, n, out):
    """A block of 64 rows: the GEMM forms and the tensor-core weight streams ("stream", "streamb" and their SwiGLU
    twins) that the selection times against them."""
    m = 64
    s = Shape(ctx, oracle, m, k, n, out)
    s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m))
    s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m, cta_pair=1))
    for tile_n in (256, 128, 64):
        s.check(ctx, oracle, ctx.gemm(k, n, out, rows_max=m, tile_n=tile_n, stream_k=1))
    forms = [(1, 2), (2, 2), (3, 2)] if out == OUT_SWIGLU else [(1, 2), (2, 1), (1, 1), (3, 2)]
    for tc, kps in forms:
        kern = ctx.matvec(k, n, out, rows_max=m, tensor_core=tc, split=kps)
        assert kern.name.startswith("matvec_tc_")
        s.check(ctx, oracle, kern)


@pytest.mark.parametrize("m", [4, 8])
def test_lm_head_151936_tensor_core_streams(ctx, oracle, m):
    """The forms hb_select_matvec picks for 4 and 8 rows at the LM-head shape, all 151936 outputs of every row."""
    k, n = 4096, 151936
    s = Shape(ctx, oracle, m, k, n, OUT_BF16)
    for tc, kps in ((1, 2), (1, 4), (2, 2), (2, 4), (3, 2), (3, 4)):
        kern = ctx.matvec(k, n, OUT_BF16, rows_max=m, tensor_core=tc, split=kps)
        s.check(ctx, oracle, kern)


# ------------------------------------------------------------------ the 27B-class FFN, whole and sharded

FFN_M, FFN_H, FFN_INTER = 2048, 5120, 17408


@pytest.fixture(scope="module")
def ffn27(oracle):
    """Inputs of the 27B-class FFN and its two stages' f64 references (gate/up + SwiGLU; down + residual over the
    SwiGLU rows the first stage's reference gives)."""
    m, h, inter = FFN_M, FFN_H, FFN_INTER
    x = oracle.normal((m, h), 1, 1, 1.0)
    wgu = oracle.normal((2 * inter, h), 2, 2, h**-0.5)
    wd = oracle.normal((h, inter), 3, 3, inter**-0.5)
    y0 = oracle.normal((m, h), 4, 4, 1.0)
    rows = sorted(set([0, m - 1] + list(np.random.default_rng(27).integers(0, m, size=6))))
    hmid_full = f64_reference(x, wgu, OUT_SWIGLU, None)
    hmid_rows = oracle.gemm_f64_rows(x, wgu, rows, OUT_SWIGLU, None)
    c = oracle.compare(hmid_rows[rows], hmid_full[rows])
    assert c.over_1ulp <= 1e-3 * c.count
    return dict(x=x, wgu=wgu, wd=wd, y0=y0, rows=rows, hmid_full=hmid_full, hmid_rows=hmid_rows)


def _check_down(oracle, f, hmid_gpu, y_gpu, what):
    """Y against bf16(y0 + bf16(f64 sum of hmid_gpu . wd)): sampled rows on the CPU, every element on the GPU."""
    rows = f["rows"]
    want_rows = oracle.gemm_f64_rows(hmid_gpu, f["wd"], rows, OUT_RESIDUAL, f["y0"])
    full = f64_reference(hmid_gpu, f["wd"], OUT_RESIDUAL, f["y0"])
    c = oracle.compare(want_rows[rows], full[rows])
    assert c.over_1ulp <= 1e-3 * c.count
    within_contract(oracle, want_rows[rows], y_gpu[rows], f"{what}: sampled rows")
    cols = list(range(4)) + list(range(FFN_H - 4, FFN_H))
    spot = oracle.compare(np.ascontiguousarray(want_rows[[0, FFN_M - 1]][:, cols]), np.ascontiguousarray(y_gpu[[0, FFN_M - 1]][:, cols]))
    assert spot.max_abs_err <= max(spot.max_abs_ref, 1e-3) / 64, f"{what}: the probe's 16 spot outputs"
    within_contract(oracle, full, y_gpu, f"{what}: all elements")


def _check_swiglu_chain(oracle, f, hmid, what):
    """The SwiGLU rows against the f64 chain (f64 sums, then the three roundings). A gate or up sum that lands on the
    other side of a bf16 boundary than its f64 twin moves the product by one to three ulps, and sums that cancel to
    nearly nothing by many, so the one-ulp rate of a single rounding does not carry over: at K = 5120 about 0.1 % of
    the outputs are further than one ulp. The product itself is held to the contract by the plain-output run of the
    same kernel and the epilogue to bit equality; here the chain gets three times the rate and the same hard limit."""
    for want, got in ((f["hmid_rows"][f["rows"]], hmid[f["rows"]]), (f["hmid_full"], hmid)):
        c = oracle.compare(np.ascontiguousarray(want), np.ascontiguousarray(got))
        assert c.over_1ulp <= 3e-3 * c.count, f"{what}: {c.over_1ulp}/{c.count} SwiGLU outputs over 1 bf16 ulp"
        assert c.max_abs_err <= c.max_abs_ref / 64, f"{what}: max err {c.max_abs_err} over 1/64 of {c.max_abs_ref}"


@pytest.mark.parametrize("form", ["one", "pair"])
def test_ffn_27b_2048x5120x34816_then_2048x17408x5120_one_gpu(ctx, oracle, ffn27, form):
    f = ffn27
    m, h, inter = FFN_M, FFN_H, FFN_INTER
    kw = dict(cta_pair=1) if form == "pair" else {}
    d_x, d_wgu, d_wd = ctx.to_device(f["x"]), ctx.to_device(f["wgu"]), ctx.to_device(f["wd"])
    d_gu, d_h, d_h2, d_y = ctx.alloc(m * 2 * inter * 2), ctx.alloc(m * inter * 2), ctx.alloc(m * inter * 2), ctx.to_device(f["y0"])
    k_gu = ctx.gemm(h, 2 * inter, OUT_SWIGLU, rows_max=m, **kw)
    k_dn = ctx.gemm(inter, h, OUT_RESIDUAL, rows_max=m, **kw)
    k_gu(m, d_wgu, d_x, d_h)
    k_dn(m, d_wd, d_h, d_y)
    # the same product with the plain output, and the SwiGLU over its rows as a kernel of its own
    k_plain = ctx.gemm(h, 2 * inter, OUT_BF16, rows_max=m, **kw)
    k_plain(m, d_wgu, d_x, d_gu)
    ctx.swiglu_rows(inter)(m, d_gu, d_h2)
    ctx.sync()
    hmid = d_h.download(np.uint16, (m, inter))
    gu = d_gu.download(np.uint16, (m, 2 * inter))
    rows = f["rows"]
    # (i) the product under the contract: sampled rows on the CPU, every element against the pinned f64 product
    gu_rows = oracle.gemm_f64_rows(f["x"], f["wgu"], rows, OUT_BF16, None)
    gu_full = f64_reference(f["x"], f["wgu"], OUT_BF16, None)
    c = oracle.compare(gu_rows[rows], gu_full[rows])
    assert c.over_1ulp <= 1e-3 * c.count
    within_contract(oracle, gu_rows[rows], gu[rows], f"{k_plain.name} sampled rows")
    within_contract(oracle, gu_full, gu, f"{k_plain.name} all elements")
    # (ii) the epilogue bit for bit: fused == apart on the GPU, and == the oracle's SwiGLU over the same gate/up rows
    assert np.array_equal(hmid, d_h2.download(np.uint16, (m, inter))), "fused SwiGLU differs from GEMM + swiglu_rows"
    assert np.array_equal(hmid[rows], oracle.swiglu_rows(np.ascontiguousarray(gu[rows])))
    # (iii) the chain from x, with the rate three roundings allow
    _check_swiglu_chain(oracle, f, hmid, k_gu.name)
    _check_down(oracle, f, hmid, d_y.download(np.uint16, (m, h)), k_dn.name)


@pytest.fixture()
def env(hb200):
    d = load_dist()
    c = hb200.Context(0)
    stream = torch.cuda.Stream()
    c.set_stream(stream.cuda_stream)
    with torch.cuda.stream(stream):
        yield d, c
    stream.synchronize()
    c.close()


@pytest.mark.parametrize("mode", ["stream", "pushsync", "push", "pull"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ffn_27b_tensor_parallel_emulated_ranks_real_shapes(env, hb200, oracle, ffn27, world, mode):
    """The sharded FFN at its real shapes, the ranks emulated on one GPU (no kernel of the step waits for another
    rank): shard widths 17408 / world = 8704, 4352, 2176. Each rank's SwiGLU rows against the oracle's columns of
    that shard; every rank's Y against the oracle over those rows; and bit for bit against the plain kernels' f32
    partials summed in rank order."""
    d, ctx = env
    f = ffn27
    m, h, inter = FFN_M, FFN_H, FFN_INTER
    ip = inter // world
    xt, y0t = t16(f["x"]).cuda(), t16(f["y0"]).cuda()
    ranks = [d.TpPeer(hb200, ctx, r, world, m, h, mode=mode) for r in range(world)]
    for st in ranks:
        st.connect(ranks)
        st.set_y(y0t)
    wgu_t, wd_t = t16(f["wgu"]), t16(f["wd"])
    shards = [(d.shard_gate_up(wgu_t, r, world).cuda(), d.shard_down(wd_t, r, world).cuda()) for r in range(world)]
    for st, (a, b) in zip(ranks, shards):
        st.phase_gemms(xt, a, b)
    for st in ranks:
        st.phase_reduce()
    torch.cuda.synchronize()
    ctx.sync()
    hmid = np.concatenate([n16(st.kernels[(h, ip)][2].cpu()) for st in ranks], axis=1)
    # a shard's SwiGLU rows are the unsharded kernel's columns of that shard, bit for bit (the K loop of an output does
    # not depend on which tile holds it); the unsharded rows are held to the oracle here and, stage by stage, in the
    # one-GPU test above
    be = d.GpuBackend(hb200, ctx, rows_max=m)
    whole = torch.empty(m, inter, device="cuda", dtype=torch.bfloat16)
    wgu_dev = wgu_t.cuda()
    ctx.gemm(h, 2 * inter, OUT_SWIGLU, rows_max=m, cta_pair=1)(m, be._w(wgu_dev), be._w(xt), be._w(whole))
    torch.cuda.synchronize()
    whole = n16(whole.cpu())
    for r in range(world):
        cols = slice(r * ip, (r + 1) * ip)
        assert np.array_equal(hmid[:, cols], whole[:, cols]), f"rank {r} of {world}: SwiGLU rows of width {ip} differ from the unsharded kernel's"
    _check_swiglu_chain(oracle, f, hmid, f"SwiGLU rows over {world} ranks")
    y = n16(ranks[0].y_view().cpu())
    for st in ranks[1:]:
        assert torch.equal(st.y_view(), ranks[0].y_view()), f"rank {st.rank} holds another Y than rank 0"
    _check_down(oracle, f, hmid, y, f"FFN over {world} ranks ({mode})")
    # the same sum from the plain kernels: f32 partials of every shard added in rank order, then the output mode
    acc = None
    for st, (a, b) in zip(ranks, shards):
        part = torch.empty(m, h, device="cuda", dtype=torch.float32)
        ctx.gemm(ip, h, OUT_F32, rows_max=m, cta_pair=1)(m, be._w(b), be._w(st.kernels[(h, ip)][2]), be._w(part))
        torch.cuda.synchronize()
        acc = part if acc is None else acc + part
    want = be.epilogue(acc, y0t.clone(), OUT_RESIDUAL)
    torch.cuda.synchronize()
    assert torch.equal(ranks[0].y_view(), want), "the sharded step is not the rank-order sum of the plain partials"
    for st in ranks:
        st.close()
