"""The C oracle against the golden vectors (tests/golden/golden.npz, made by an independent numpy /
pure-Python restatement of the reference's rules in tests/golden/make_golden.py) and against
hand-derived known answers. CPU only."""
import os

import numpy as np
import pytest

from oracle_lib import OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU, bf16_to_f32

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))


def test_rne_known_answers(oracle):
    # ties to even at ...8000, sticky bits, carry into the exponent and into infinity, zeros, subnormals
    for bits, want in zip(G["rne_in"], G["rne_out"]):
        got = oracle.lib.hbo_f32_to_bf16(np.array([bits], dtype=np.uint32).view(np.float32)[0])
        assert got == want, hex(int(bits))
    hand = {0x3F808000: 0x3F80, 0x3F818000: 0x3F82, 0x3F808001: 0x3F81, 0x7F7F8000: 0x7F80, 0x80000000: 0x8000, 0x00018000: 0x0002}
    for bits, want in hand.items():
        assert oracle.lib.hbo_f32_to_bf16(np.array([bits], dtype=np.uint32).view(np.float32)[0]) == want


def test_rne_matches_integer_form_everywhere(oracle):
    # (bits + 0x7fff + lsb) >> 16, the GPU form (msl/mod.rs:1343), equals the CPU form (bf16.rs:13-23)
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 2**32, size=200000, dtype=np.uint64).astype(np.uint32)
    bits = bits[(bits & 0x7F800000) != 0x7F800000]  # NaN/Inf payloads excluded from the contract
    want = ((bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    got = np.array([oracle.lib.hbo_f32_to_bf16(v) for v in bits.view(np.float32)[:20000]], dtype=np.uint16)
    assert np.array_equal(got, want[:20000])


def test_widening_is_exact(oracle):
    for h in (0x0000, 0x3F80, 0xBF80, 0x4049, 0x0001, 0x7F7F):
        assert oracle.lib.hbo_bf16_to_f32(h) == np.array([h << 16], dtype=np.uint32).view(np.float32)[0]


def test_f64_to_bf16_rounds_once(oracle):
    # 1 + 2^-8 + 2^-40: above the tie, must round up; via f32 (RNE) first it would land on the tie and round to even
    v = 1.0 + 2.0**-8 + 2.0**-40
    assert oracle.lib.hbo_f64_to_bf16(v) == 0x3F81
    assert oracle.lib.hbo_f64_to_bf16(1.0 + 2.0**-8) == 0x3F80  # exact tie -> even
    assert oracle.lib.hbo_f64_to_bf16(1.0 + 3 * 2.0**-8) == 0x3F82
    assert oracle.lib.hbo_f64_to_bf16(-0.0) == 0x8000


def test_exp_bits_and_accuracy(oracle):
    got = np.array([oracle.lib.hbo_expf(float(v)) for v in G["exp_in"]], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), G["exp_out"].view(np.uint32))
    xs = np.linspace(-87.0, 88.0, 20001).astype(np.float32)
    got = np.array([oracle.lib.hbo_expf(float(v)) for v in xs], dtype=np.float32)
    ref = np.exp(xs.astype(np.float64))
    ulp = np.abs(got.astype(np.float64) - ref) / np.spacing(ref.astype(np.float32)).astype(np.float64)
    assert ulp.max() < 1.0
    assert oracle.lib.hbo_expf(0.0) == 1.0 and oracle.lib.hbo_expf(-200.0) == 0.0 and np.isinf(oracle.lib.hbo_expf(89.0))


def test_swiglu_known_answers(oracle):
    got = np.array([oracle.lib.hbo_swiglu_one(int(g), int(u)) for g, u in zip(G["swiglu_g"], G["swiglu_u"])], dtype=np.uint16)
    assert np.array_equal(got, G["swiglu_out"])
    gu = np.concatenate([G["swiglu_g"].reshape(2, 32), G["swiglu_u"].reshape(2, 32)], axis=1)
    assert np.array_equal(oracle.swiglu_rows(gu), G["swiglu_out"].reshape(2, 32))


def test_generators(oracle):
    assert np.array_equal(oracle.xorshift16(64, 0x9E3779B9), G["xorshift16_9e3779b9"])
    assert np.array_equal(oracle.random16(64, 1), G["random16_1"])
    assert np.array_equal(oracle.normal(96, 0x9E3779B9, 1, 1.0), G["normal_x"])
    assert np.array_equal(oracle.normal(96, 0x2545F491, 2, 1.0 / 32.0), G["normal_w"])
    # the reference's autotune inputs lie in [-1, 1); random16 magnitudes in [2^-6, 1)
    v = bf16_to_f32(oracle.xorshift16(4096, 0x9E3779B9))
    assert v.min() >= -1.0 and v.max() <= 1.0
    r = np.abs(bf16_to_f32(oracle.random16(4096, 7)))
    assert r.min() >= 2.0**-6 and r.max() < 1.0
    z = bf16_to_f32(oracle.normal(1 << 16, 3, 0, 1.0))
    assert abs(z.mean()) < 0.02 and abs(z.std() - 1.0) < 0.02


@pytest.mark.parametrize("mode,key", [(OUT_BF16, "gemm_bf16"), (OUT_F32, "gemm_f32"), (OUT_RESIDUAL, "gemm_residual"), (OUT_SWIGLU, "gemm_swiglu")])
def test_gemm_f64_against_exact_rational(oracle, mode, key):
    got = oracle.gemm_f64(G["gemm_x"], G["gemm_w"], mode, G["gemm_y0"])
    if mode == OUT_F32:
        assert np.array_equal(got.view(np.uint32), G[key].view(np.uint32))
    else:
        assert np.array_equal(got, G[key])


def test_gemm_f32_contract_close_to_f64(oracle):
    x = oracle.normal((96, 512), 1, 1, 1.0)
    w = oracle.normal((200, 512), 2, 2, 512**-0.5)
    y0 = oracle.normal((96, 200), 3, 3, 1.0)
    for mode in (OUT_BF16, OUT_RESIDUAL, OUT_SWIGLU):
        a, b = oracle.gemm_f64(x, w, mode, y0), oracle.gemm_f32(x, w, mode, y0)
        c = oracle.compare(a, b)
        assert c.over_1ulp <= 1e-3 * c.count and c.max_abs_err <= c.max_abs_ref / 64
    a, b = oracle.gemm_f64(x, w, OUT_F32), oracle.gemm_f32(x, w, OUT_F32)
    assert np.abs(a - b).max() < 1e-4


def test_gemm_rows_subset_and_ragged_shapes(oracle):
    x = oracle.normal((17, 72), 1, 1, 1.0)
    w = oracle.normal((9, 72), 2, 2, 0.1)
    full = oracle.gemm_f64(x, w)
    part = oracle.gemm_f64_rows(x, w, [0, 5, 16])
    assert np.array_equal(part[[0, 5, 16]], full[[0, 5, 16]]) and not part[1].any()
    one = oracle.gemm_f64(x[:1], w[:1])
    assert one.shape == (1, 1) and one[0, 0] == full[0, 0]


def test_matvec_reference_order_within_contract(oracle):
    x = oracle.normal((1, 1024), 1, 1, 1.0)
    w = oracle.normal((300, 1024), 2, 2, 1 / 32.0)
    a = oracle.gemm_f64(x, w).reshape(-1)
    b = oracle.matvec_ref_order(x, w)
    c = oracle.compare(a, b)
    assert c.over_1ulp <= 1e-3 * c.count and c.max_ulp <= 8


def test_route_known_answers_and_ties(oracle):
    route = oracle.route_topk(G["route_scores"], 4)
    assert np.array_equal(route, G["route_out"])
    # experts ascending within a row; row 1 holds a three-way tie at experts 5, 9, 40
    assert all(np.all(np.diff(r[:4].astype(np.int64)) > 0) for r in route)
    w = route[:, 4:].view(np.float32)
    assert np.all((w > 0) & (w <= 1)) and np.allclose(w.sum(axis=1), 1.0, atol=0.02)
    s = G["route_scores"][1]
    assert s[5] == s[9] == s[40]
    tied = [e for e in (5, 9, 40) if e in route[1, :4]]
    assert tied == sorted(tied) and (len(tied) == 0 or tied[0] == 5 or s[5] == 0)


@pytest.mark.parametrize("bm", [16, 32, 64])
def test_sort_known_answers(oracle, bm):
    lst, tiles = oracle.moe_sort(G["route_out"], 64, 4, bm)
    want_t = G[f"sort_tiles_{bm}"]
    assert np.array_equal(lst, G[f"sort_list_{bm}"]) and np.array_equal(tiles[: len(want_t)], want_t)
    lst, tiles = oracle.moe_sort(G["sort_big_route"], 8, 2, bm)
    want_t = G[f"sort_big_tiles_{bm}"]
    assert np.array_equal(lst, G[f"sort_big_list_{bm}"]) and np.array_equal(tiles[: len(want_t)], want_t)
    # expert 3 holds 40 pairs: ceil(40/bm) tiles, the last one partial
    n = int(tiles[0])
    t3 = [tuple(tiles[1 + 3 * i : 4 + 3 * i]) for i in range(n) if tiles[1 + 3 * i] == 3]
    assert len(t3) == -(-40 // bm) and sum(t[2] for t in t3) == 40 and all(t[2] <= bm for t in t3)


def test_sort_is_a_stable_permutation(oracle):
    scores = oracle.normal((257, 128), 9, 1, 1.0)
    route = oracle.route_topk(scores, 8)
    lst, tiles = oracle.moe_sort(route, 128, 8, 32)
    assert np.array_equal(np.sort(lst), np.arange(257 * 8, dtype=np.uint32))
    e = route[:, :8].reshape(-1)[lst]
    assert np.all(np.diff(e.astype(np.int64)) >= 0)
    for x in np.unique(e):
        assert np.all(np.diff(lst[e == x].astype(np.int64)) > 0)  # pairs ascending inside an expert
    n = int(tiles[0])
    rows = tiles[3 : 3 + 3 * n : 3]
    assert rows.sum() == 257 * 8 and n <= (257 * 8 + 31) // 32 + 128


def test_combine_known_answers(oracle):
    got = oracle.moe_combine(G["combine_ey"], G["route_out"], 4)
    assert np.array_equal(got, G["combine_out"])
    f32 = oracle.moe_combine(G["combine_ey"], G["route_out"], 4, f32=True)
    c = oracle.compare(got, f32)
    # the per-step rounding of the reference chain differs from one rounding by a few bf16 ulps of the
    # largest term (ulps of a cancelled sum can be many)
    assert c.max_abs_err <= c.max_abs_ref / 64


def test_rmsnorm_known_answers(oracle):
    assert np.array_equal(oracle.rmsnorm_rows(G["norm_x"], G["norm_w"], 1e-6, False), G["norm_out"])
    assert np.array_equal(oracle.rmsnorm_rows(G["norm_x"], G["norm_w"], 1e-6, True), G["norm_out_p1"])
    # and what it means: rows of unit root-mean-square times the weight, to bf16 accuracy
    x = (G["norm_x"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    w = (G["norm_w"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    want = x / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6) * (1.0 + w)
    got = (G["norm_out_p1"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.abs(got - want).max() <= np.abs(want).max() * 2.0**-7


def test_argmax_known_answers(oracle):
    assert np.array_equal(oracle.argmax_rows(G["argmax_logits"]), G["argmax_out"])


def test_moe_out_known_answers(oracle):
    got = oracle.moe_out(G["moe_out_xn"], G["moe_out_gate"], G["moe_out_experts"], G["moe_out_shared"], G["moe_out_x"])
    assert np.array_equal(got, G["moe_out_out"])


def test_q4_known_answers(oracle):
    w = G["q4_w"]
    n, k = w.shape
    data, scales = oracle.q4_quantize(w)
    assert np.array_equal(data, G["q4_data"]) and np.array_equal(scales, G["q4_scales"])
    deq = oracle.q4_dequant(data, scales, n, k)
    assert np.array_equal(deq, G["q4_dequant"])
    # the reference's own unit test (q4.rs:113-131): a block on the grid comes back exactly
    assert np.array_equal(deq[1, :32], w[1, :32])
    assert np.array_equal(oracle.matvec_q4(data, scales, G["q4_x"], n, k), G["q4_matvec"])
    assert np.array_equal(oracle.matvec_q4(data, scales, G["q4_x"], n, k, masks=True), G["q4s_matvec"])
    assert np.array_equal(oracle.matmul_q4(data, scales, G["q4_X"], n, k), G["q4_matmul"])
    assert np.array_equal(G["q4_matmul"][0], G["q4_matvec"])
    # the split order (matvec_q4_split): the blocks of a row shared by 2 and by 4 simdgroups
    sw, sx = G["q4split_w"], G["q4split_x"]
    sd, ss = oracle.q4_quantize(sw)
    for sp in (1, 2, 4):
        assert np.array_equal(oracle.matvec_q4(sd, ss, sx, sw.shape[0], sw.shape[1], split=sp) if sp > 1 else oracle.matvec_q4(sd, ss, sx, sw.shape[0], sw.shape[1]), G[f"q4split_{sp}"]), sp
    # quantisation error is small against the weights
    f = lambda a: (a.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.abs(f(deq) - f(w)).max() <= np.abs(f(w)).max() / 7.5


def test_check_rule(oracle):
    ref = G["check_ref"]
    assert oracle.check_1_64(ref, G["check_ok"])[0] is True
    ok, err, scale = oracle.check_1_64(ref, G["check_bad"])
    assert ok is False and err > scale / 64
    nan = ref.copy()
    nan[3] = np.nan
    assert oracle.check_1_64(ref, nan)[0] is False  # a NaN output never passes
    zero = np.zeros(16, dtype=np.float32)
    ok, err, scale = oracle.check_1_64(zero, zero)
    assert ok and scale == np.float32(1e-6)
    b = np.array([0x3F80, 0x4000], dtype=np.uint16)
    assert oracle.check_1_64(b, np.array([0x3F80, 0x4001], dtype=np.uint16))[0] is True
    assert oracle.check_1_64(b, np.array([0x3F80, 0x4010], dtype=np.uint16))[0] is False


def test_moe_pipeline_oracle_consistency(oracle):
    # gather + gate/up + SwiGLU + down + combine on a small block: the expert path equals a dense
    # per-token evaluation of the same experts
    m, h, mi, E, k = 9, 64, 32, 32, 4
    x = oracle.normal((m, h), 1, 1, 1.0)
    wgu = oracle.normal((E * 2 * mi, h), 2, 2, h**-0.5)
    wd = oracle.normal((E * h, mi), 3, 3, mi**-0.5)
    route = oracle.route_topk(oracle.normal((m, E), 4, 4, 1.0), k)
    lst, tiles = oracle.moe_sort(route, E, k, 16)
    egu = oracle.moe_gate_up(x, wgu, lst, tiles, mi, k)
    ehb = oracle.swiglu_slots(egu)
    ey = oracle.moe_down(ehb, wd, lst, tiles, h)
    out = oracle.moe_combine(ey, route, k)
    assert out.shape == (m, h)
    for r in range(m):
        for s in range(k):
            e = int(route[r, s])
            gu = oracle.gemm_f64(x[r : r + 1], wgu[e * 2 * mi : (e + 1) * 2 * mi], OUT_SWIGLU)
            y = oracle.gemm_f64(gu, wd[e * h : (e + 1) * h])
            assert np.array_equal(y[0], ey[r * k + s])
