"""Generates tests/golden/golden.npz: known-answer vectors for the matrix-multiply path.

The reference (herbert-metal-bf16) holds no fixture for this path and its kernels cannot run off
an Apple GPU, so these vectors come from an INDEPENDENT restatement of its rules in numpy /
pure Python (this file), written from the reference source:
  * round to nearest even f32 -> bf16        src/core/bf16.rs:13-23
  * epilogues Bf16 / F32 / Residual / Swiglu  src/metal/kernels.rs:30-42,217-234; prefill.rs:2790-2818
  * route (softmax, top-k, renormalise)       src/metal/qwen_kernels.rs:1802-1878
  * sort and tile table                       src/metal/prefill.rs:1303-1442
  * combine                                   src/metal/qwen_kernels.rs:2119-2161
  * check rule                                src/metal/qwen.rs:2519-2531
  * input generators                          src/metal/qwen.rs:2613-2626; src/bin/herbert-metal-probe.rs:435-462
The C oracle (oracle/hb_oracle.c) is tested against this file's output; the two share no code.

    python tests/golden/make_golden.py
"""
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def f32_bits(x):
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def bits_f32(b):
    return struct.unpack("<f", struct.pack("<I", b & 0xFFFFFFFF))[0]


def rne_bf16(x):
    """bits>>16, +1 when the round bit is set and (sticky != 0 or the kept lsb is 1)."""
    bits = f32_bits(np.float32(x))
    lsb, rnd, sticky = (bits >> 16) & 1, (bits >> 15) & 1, bits & 0x7FFF
    r = bits >> 16
    if rnd == 1 and (sticky != 0 or lsb == 1):
        r += 1
    return r & 0xFFFF


def widen(h):
    return np.float32(bits_f32(int(h) << 16))


def rne_bf16_array(a):
    return np.array([rne_bf16(v) for v in np.asarray(a, dtype=np.float32).ravel()], dtype=np.uint16).reshape(np.shape(a))


def widen_array(a):
    return (np.asarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def exp_f32(x):
    """The contract's exp: a fixed sequence of f32 operations (see oracle/hb_oracle.h)."""
    f = np.float32
    x = f(x)
    if x > f(88.72283):
        return f(np.inf)
    if x < f(-103.98):
        return f(0.0)

    def fma(a, b, c):  # exact product and sum in float64 (24x24-bit product fits), one rounding to f32
        # a*b is exact in f64; adding c may round in f64 before the f32 rounding: use integers of the
        # exact rational instead.
        from fractions import Fraction

        v = Fraction(float(a)) * Fraction(float(b)) + Fraction(float(c))
        return round_fraction_f32(v)

    n = f(np.rint(f(x * f(1.44269504088896341))))
    r = fma(n, f(-0.693359375), x)
    r = fma(n, f(2.12194440e-4), r)
    p = f(1.9875691500e-4)
    for c in (1.3981999507e-3, 8.3334519073e-3, 4.1665795894e-2, 1.6666665459e-1, 5.0000001201e-1):
        p = fma(p, r, f(c))
    r2 = f(r * r)
    p = fma(p, r2, r)
    p = f(p + f(1.0))
    k = int(n)
    k1 = int(k / 2)  # C division truncates toward zero
    k2 = k - k1
    return f(f(p * f(2.0 ** k1)) * f(2.0 ** k2))


def round_fraction_f32(v):
    """A Fraction rounded to nearest-even f32 (normal range)."""
    from fractions import Fraction

    if v == 0:
        return np.float32(0.0)
    sign = -1 if v < 0 else 1
    v = abs(v)
    e = 0
    while v >= 2:
        v /= 2
        e += 1
    while v < 1:
        v *= 2
        e -= 1
    scaled = v * (1 << 23)
    q = int(scaled)
    rem = scaled - q
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and (q & 1)):
        q += 1
    return np.float32(sign * q * 2.0 ** (e - 23))


def sigmoid_f32(x):
    f = np.float32
    e = exp_f32(f(-x))
    return f(f(1.0) / f(f(1.0) + e))


def swiglu(gh, uh):
    f = np.float32
    g, u = widen(gh), widen(uh)
    return rne_bf16(f(f(g * sigmoid_f32(g)) * u))


def xorshift16(count, seed):
    out = []
    for _ in range(count):
        seed ^= (seed << 13) & 0xFFFFFFFF
        seed ^= seed >> 17
        seed ^= (seed << 5) & 0xFFFFFFFF
        out.append(rne_bf16(np.float32(np.float32(seed >> 8) / np.float32(1 << 23)) - np.float32(1.0)))
    return np.array(out, dtype=np.uint16)


def random16(count, seed):
    out, s = [], seed
    for _ in range(count):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        r = s >> 32
        sign = r >> 31
        e = 9 + ((r >> 24) & 7) % 6
        out.append((sign << 15) | ((e + 112) << 7) | (r & 0x7F))
    return np.array(out, dtype=np.uint16)


def splitmix64(z):
    z = (z + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return z ^ (z >> 31)


def fill_normal(count, seed, tensor_id, sigma):
    out = []
    for i in range(count):
        base = (seed ^ (tensor_id << 40) ^ i) & 0xFFFFFFFFFFFFFFFF
        total = 0
        for j in range(3):
            u = splitmix64((base * 3 + j) & 0xFFFFFFFFFFFFFFFF)
            total += (u & 0xFFFF) + ((u >> 16) & 0xFFFF) + ((u >> 32) & 0xFFFF) + ((u >> 48) & 0xFFFF)
        z = (total - 393210.0) / 65536.0
        out.append(rne_bf16(np.float32(z * sigma)))
    return np.array(out, dtype=np.uint16)


def gemm_f64(x, w, out, y0=None):
    """Exact dot products (float64 of small-K bf16 inputs is exact enough to be order-free), one rounding."""
    from fractions import Fraction

    xf, wf = widen_array(x).astype(np.float64), widen_array(w).astype(np.float64)
    m, n = x.shape[0], w.shape[0]
    acc = [[sum(Fraction(a) * Fraction(b) for a, b in zip(xf[r], wf[c])) for c in range(n)] for r in range(m)]

    def to_bf16(v):  # a Fraction rounded once to bf16 (8 significant bits)
        if v == 0:
            return 0
        sign = 0x8000 if v < 0 else 0
        v = abs(v)
        e = 0
        while v >= 2:
            v /= 2
            e += 1
        while v < 1:
            v *= 2
            e -= 1
        scaled = v * 128
        q = int(scaled)
        rem = scaled - q
        if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and (q & 1)):
            q += 1
        if q == 256:
            q, e = 128, e + 1
        return sign | ((e + 127) << 7) | (q - 128)

    if out == "f32":
        return np.array([[round_fraction_f32(v) for v in row] for row in acc], dtype=np.float32)
    b = np.array([[to_bf16(v) for v in row] for row in acc], dtype=np.uint16)
    if out == "bf16":
        return b
    if out == "residual":
        return rne_bf16_array(widen_array(y0) + widen_array(b))
    if out == "swiglu":
        half = n // 2
        return np.array([[swiglu(b[r, c], b[r, half + c]) for c in range(half)] for r in range(m)], dtype=np.uint16)
    raise ValueError(out)


def butterfly_sum(v):
    a = [np.float32(t) for t in v]
    for off in (16, 8, 4, 2, 1):
        a = [np.float32(a[i] + a[i ^ off]) for i in range(32)]
    return a[0]


def route_topk(scores, top_k):
    f = np.float32
    rows, experts = scores.shape
    out = np.zeros((rows, 2 * top_k), dtype=np.uint32)
    for r in range(rows):
        s = [widen(h) for h in scores[r]]
        mx = max(s)
        ex = [exp_f32(f(v - mx)) for v in s]
        total = butterfly_sum(ex[0:32])
        for g in range(1, experts // 32):
            total = f(total + butterfly_sum(ex[32 * g : 32 * g + 32]))
        p = [f(e / total) for e in ex]
        chosen, vals = [], []
        for _ in range(top_k):
            best, idx = f(-2.0), 0
            for e in range(experts):
                if p[e] > best:
                    best, idx = p[e], e
            p[idx] = f(-1.0)
            chosen.append(idx)
            vals.append(best)
        tot = f(0.0)
        for v in vals:
            tot = f(tot + v)
        for i in range(top_k):
            w = widen(rne_bf16(f(vals[i] / tot)))
            rank = sum(1 for j in range(top_k) if j != i and chosen[j] < chosen[i])
            out[r, rank] = chosen[i]
            out[r, top_k + rank] = f32_bits(w)
    return out


def moe_sort(route, experts, top_k, bm):
    rows = route.shape[0]
    pairs = [(int(route[i // top_k, i % top_k]), i) for i in range(rows * top_k)]
    lst, tiles = [], []
    for e in range(experts):
        mine = [i for (x, i) in pairs if x == e]
        start = len(lst)
        for j in range(0, len(mine), bm):
            tiles.append((e, start + j, min(bm, len(mine) - j)))
        lst.extend(mine)
    table = [len(tiles)] + [v for t in tiles for v in t]
    return np.array(lst, dtype=np.uint32), np.array(table, dtype=np.uint32)


def moe_combine(ey, route, top_k):
    f = np.float32
    rows, d = route.shape[0], ey.shape[1]
    out = np.zeros((rows, d), dtype=np.uint16)
    for r in range(rows):
        for i in range(d):
            acc = f(0.0)
            for s in range(top_k):
                y = widen(ey[r * top_k + s, i])
                w = f(bits_f32(int(route[r, top_k + s])))
                c = widen(rne_bf16(f(y * w)))
                acc = widen(rne_bf16(f(acc + c)))
            out[r, i] = rne_bf16(acc)
    return out


def fma_f32(a, b, c):
    """fmaf: a * b + c rounded once (exact rational arithmetic)."""
    from fractions import Fraction

    return round_fraction_f32(Fraction(float(a)) * Fraction(float(b)) + Fraction(float(c)))


def group_sum256(lanes):
    """256 per-thread values: simd_sum of each 32 (xor butterfly), the 8 partials folded in order."""
    f = np.float32
    acc = butterfly_sum(lanes[0:32])
    for gidx in range(1, 8):
        acc = f(acc + butterfly_sum(lanes[32 * gidx : 32 * gidx + 32]))
    return acc


def rmsnorm_rows(x, w, eps, plus_one):
    f = np.float32
    rows, d = x.shape
    out = np.zeros((rows, d), dtype=np.uint16)
    for r in range(rows):
        lanes = []
        for lane in range(256):
            a = f(0.0)
            for i in range(lane, d, 256):
                v = widen(x[r, i])
                a = fma_f32(v, v, a)
            lanes.append(a)
        ss = group_sum256(lanes)
        mm = f(f(ss * f(1.0 / d)) + f(eps))
        inv = f(f(1.0) / np.sqrt(mm, dtype=np.float32))
        for i in range(d):
            wf = widen(w[i])
            if plus_one:
                wf = f(wf + f(1.0))
            out[r, i] = rne_bf16(f(f(widen(x[r, i]) * inv) * wf))
    return out


def argmax_rows(logits):
    out = []
    for row in logits:
        best, best_i = np.float32(-np.inf), 0xFFFFFFFF
        for i, h in enumerate(row):
            v = widen(h)
            if v > best:
                best, best_i = v, i
        out.append(best_i)
    return np.array(out, dtype=np.uint32)


def moe_out(xn, gate, experts, shared, x):
    f = np.float32
    rows, d = x.shape
    out = np.zeros((rows, d), dtype=np.uint16)
    for r in range(rows):
        lanes = []
        for lane in range(256):
            a = f(0.0)
            for i in range(lane, d, 256):
                a = fma_f32(widen(xn[r, i]), widen(gate[i]), a)
            lanes.append(a)
        logit = widen(rne_bf16(group_sum256(lanes)))
        gsig = widen(rne_bf16(sigmoid_f32(logit)))
        for i in range(d):
            sh = widen(rne_bf16(f(gsig * widen(shared[r, i]))))
            o = widen(rne_bf16(f(widen(experts[r, i]) + sh)))
            out[r, i] = rne_bf16(f(widen(x[r, i]) + o))
    return out


def q4_quantize(w):
    """q4.rs:16-103 restated: (data bytes [n*k/2], f16 scale bits [n*k/32])."""
    f = np.float32
    n, k = w.shape
    data = np.zeros(n * k // 2, dtype=np.uint8)
    scales = np.zeros(n * k // 32, dtype=np.uint16)
    flat = w.reshape(-1)
    for blk in range(n * k // 32):
        v = [widen(h) for h in flat[32 * blk : 32 * blk + 32]]
        m = f(0.0)
        for x in v:
            if abs(x) > abs(m):
                m = x
        best_e, best_d, best_q = float("inf"), 0, [8] * 32
        if m != 0.0:
            for c in (-8, 7, -7, 6, -6, 5, -5, 4, -4, 3, -3, 2, -2, 1, -1):
                dh = np.float16(f(m / f(c)))
                dq = f(dh)
                if dq == 0.0 or not np.isfinite(dq):
                    continue
                inv = f(f(1.0) / dq)
                e, q = 0.0, []
                for x in v:
                    t = f(x * inv)
                    qi = float(np.sign(t) * np.floor(abs(float(t)) + 0.5))  # half away from zero
                    qi = max(-8.0, min(7.0, qi))
                    q.append(int(qi) + 8)
                    r = float(f(x - f(dq * f(qi))))
                    e += r * r
                if e < best_e:
                    best_e, best_d, best_q = e, int(dh.view(np.uint16)), q
        else:
            best_e = 0.0
        for i in range(4):
            for b in range(4):
                data[16 * blk + 4 * i + b] = ((best_q[8 * i + b] ^ 8) & 15) | (((best_q[8 * i + 4 + b] ^ 8) & 15) << 4)
        scales[blk] = best_d
    return data, scales


def q4_value(data, blk, e):
    i, j = e // 8, e % 8
    byte = int(data[16 * blk + 4 * i + (j % 4)])
    nib = (byte & 15) if j < 4 else (byte >> 4)
    return np.float32((nib ^ 8) - 8)


def q4_dequant(data, scales, n, k):
    f = np.float32
    out = np.zeros(n * k, dtype=np.uint16)
    for blk in range(n * k // 32):
        d = f(np.uint16(scales[blk]).view(np.float16))
        for e in range(32):
            out[32 * blk + e] = rne_bf16(f(d * q4_value(data, blk, e)))
    return out.reshape(n, k)


def q4_matvec(data, scales, x, n, k, split=1):
    """kernels.rs:526-632 (rows = 1): lanes over blocks, FMA chains in the reference's element order, butterfly.
    split > 1 (matvec_q4_split, kernels.rs:472-500, 896-928): block b to simdgroup (b / 32) % split, each simdgroup's
    butterfly sum, the partials added in simdgroup order."""
    f = np.float32
    nblk = k // 32
    out = np.zeros(n, dtype=np.uint16)
    for row in range(n):
      total = None
      for sub in range(split):
        lanes = []
        for lane in range(32):
            acc = f(0.0)
            for b in range(lane + 32 * sub, nblk, 32 * split):
                blk = row * nblk + b
                part = f(0.0)
                for i in range(4):
                    for byte in range(4):
                        for e in (8 * i + byte, 8 * i + 4 + byte):
                            part = fma_f32(q4_value(data, blk, e), widen(x[32 * b + e]), part)
                acc = fma_f32(f(np.uint16(scales[blk]).view(np.float16)), part, acc)
            lanes.append(acc)
        s_ = butterfly_sum(lanes)
        total = s_ if total is None else f(total + s_)
      out[row] = rne_bf16(total)
    return out


def q4s_matvec(data, scales, x, n, k):
    """kernels.rs:455-462, 1387-1424 (matvec_q4s): the masks' order of sums."""
    f = np.float32
    nblk = k // 32
    out = np.zeros(n, dtype=np.uint16)
    for row in range(n):
        lanes = []
        for lane in range(32):
            acc = f(0.0)
            for b in range(lane, nblk, 32):
                blk = row * nblk + b
                xs = [widen(x[32 * b + e]) for e in range(32)]
                sx = xs[0]
                for v in xs[1:]:
                    sx = f(sx + v)
                part = f(0.0)
                for i in range(4):
                    word = int.from_bytes(bytes(int(v) for v in data[16 * blk + 4 * i : 16 * blk + 4 * i + 4]), "little") ^ 0x88888888
                    for j in range(8):
                        shift = 8 * j if j < 4 else 8 * (j - 4) + 4
                        val = f(word & (15 << shift))
                        part = fma_f32(val, f(xs[8 * i + j] * f(2.0 ** -shift)), part)
                part = fma_f32(f(-8.0), sx, part)
                acc = fma_f32(f(np.uint16(scales[blk]).view(np.float16)), part, acc)
            lanes.append(acc)
        out[row] = rne_bf16(butterfly_sum(lanes))
    return out


def main():
    g = {}
    # RNE known answers: (f32 bits, bf16 bits) - ties to even, carries, signed zero, subnormal, infinity.
    rne_in = [0x3F800000, 0x3F808000, 0x3F818000, 0x3F808001, 0x3F807FFF, 0x3FFF8000, 0x7F7F8000, 0x00000000, 0x80000000,
              0x00008000, 0x00018000, 0x7F800000, 0xFF800000, 0x3F7FFFFF, 0xC0490FDB, 0x477FE000, 0x33800000]
    g["rne_in"] = np.array(rne_in, dtype=np.uint32)
    g["rne_out"] = np.array([rne_bf16(bits_f32(b)) for b in rne_in], dtype=np.uint16)
    assert list(g["rne_out"][:7]) == [0x3F80, 0x3F80, 0x3F82, 0x3F81, 0x3F80, 0x4000, 0x7F80]
    # exp and SwiGLU
    xs = np.array([-20.0, -5.5, -1.0, -0.3465, 0.0, 1e-3, 0.5, 1.0, 3.25, 10.0, 44.4, 88.0, -87.0, -100.0], dtype=np.float32)
    g["exp_in"] = xs
    g["exp_out"] = np.array([exp_f32(v) for v in xs], dtype=np.float32)
    gh = fill_normal(64, 11, 1, 2.0)
    uh = fill_normal(64, 11, 2, 1.5)
    g["swiglu_g"], g["swiglu_u"] = gh, uh
    g["swiglu_out"] = np.array([swiglu(a, b) for a, b in zip(gh, uh)], dtype=np.uint16)
    # generators
    g["xorshift16_9e3779b9"] = xorshift16(64, 0x9E3779B9)
    g["random16_1"] = random16(64, 1)
    g["normal_x"] = fill_normal(96, 0x9E3779B9, 1, 1.0)
    g["normal_w"] = fill_normal(96, 0x2545F491, 2, 1.0 / 32.0)
    # a small GEMM in the four output modes (exact rational dot products)
    m, n, k = 5, 12, 40
    x = fill_normal(m * k, 0x9E3779B9, 1, 1.0).reshape(m, k)
    w = fill_normal(n * k, 0x2545F491, 2, k ** -0.5).reshape(n, k)
    y0 = fill_normal(m * n, 0x85EBCA6B, 5, 1.0).reshape(m, n)
    g["gemm_x"], g["gemm_w"], g["gemm_y0"] = x, w, y0
    g["gemm_bf16"] = gemm_f64(x, w, "bf16")
    g["gemm_f32"] = gemm_f64(x, w, "f32")
    g["gemm_residual"] = gemm_f64(x, w, "residual", y0)
    g["gemm_swiglu"] = gemm_f64(x, w, "swiglu")
    # MoE: route, sort (three tile sizes), combine
    rows, experts, top_k, d = 6, 64, 4, 16
    scores = fill_normal(rows * experts, 0xC2B2AE35, 3, 1.0).reshape(rows, experts)
    scores[1, 5] = scores[1, 9]  # exact ties: the lowest index must win
    scores[1, 40] = scores[1, 9]
    route = route_topk(scores, top_k)
    g["route_scores"], g["route_out"] = scores, route
    for bm in (16, 32, 64):
        # a skewed route so that one expert spans several tiles
        skew = route.copy()
        lst, table = moe_sort(skew, experts, top_k, bm)
        g[f"sort_list_{bm}"], g[f"sort_tiles_{bm}"] = lst, table
    big = np.zeros((40, 2 * 2), dtype=np.uint32)  # 40 rows, top_k 2: expert 3 gets every row, expert 0 or 7 the other slot
    for r in range(40):
        big[r, 0], big[r, 1] = (0, 3) if r % 3 else (3, 7)
    g["sort_big_route"] = big
    for bm in (16, 32, 64):
        lst, table = moe_sort(big, 8, 2, bm)
        g[f"sort_big_list_{bm}"], g[f"sort_big_tiles_{bm}"] = lst, table
    ey = fill_normal(rows * top_k * d, 0x85EBCA6B, 9, 1.0).reshape(rows * top_k, d)
    g["combine_ey"] = ey
    g["combine_out"] = moe_combine(ey, route, top_k)
    # check rule
    ref = widen_array(fill_normal(256, 5, 1, 1.0)).astype(np.float32)
    scale = np.abs(ref).max()
    ok = ref.copy()
    ok[17] += scale / 64.0 * 0.99
    bad = ref.copy()
    bad[17] += scale / 64.0 * 1.02
    g["check_ref"], g["check_ok"], g["check_bad"] = ref, ok, bad
    # the rows around the products: RMSNorm (both weight conventions), argmax (ties, -inf, NaN), the MoE block's end
    rows, d = 3, 768
    nx = fill_normal(rows * d, 0x9E3779B9, 21, 1.5).reshape(rows, d)
    nw = fill_normal(d, 0x2545F491, 22, 0.2)
    g["norm_x"], g["norm_w"] = nx, nw
    g["norm_out"] = rmsnorm_rows(nx, nw, 1e-6, False)
    g["norm_out_p1"] = rmsnorm_rows(nx, nw, 1e-6, True)
    lg = fill_normal(5 * 300, 0xC2B2AE35, 23, 3.0).reshape(5, 300)
    lg[0, 7] = lg[0, 250] = 0x4120    # 10.0 twice, above everything else in the row: the first index wins
    lg[1, :] = 0xFF80                 # all -inf: no index
    lg[2, 3] = 0x7FC0                 # a NaN never wins
    lg[3, 100], lg[3, 299] = 0x0000, 0x8000  # +0 and -0 compare equal
    lg[3, [i for i in range(300) if i not in (100, 299)]] = 0xBF80
    lg[4, 299] = 0x7F80               # +inf in the last place
    g["argmax_logits"], g["argmax_out"] = lg, argmax_rows(lg)
    assert list(g["argmax_out"][:2]) == [7, 0xFFFFFFFF] and g["argmax_out"][3] == 100 and g["argmax_out"][4] == 299
    mo = [fill_normal(rows * d, 0x85EBCA6B, 24 + i, s).reshape(rows, d) for i, s in enumerate((1.0, 0.7, 0.5, 1.0))]
    mg = fill_normal(d, 0x2545F491, 29, d ** -0.5)
    g["moe_out_xn"], g["moe_out_experts"], g["moe_out_shared"], g["moe_out_x"], g["moe_out_gate"] = mo[0], mo[1], mo[2], mo[3], mg
    g["moe_out_out"] = moe_out(mo[0], mg, mo[1], mo[2], mo[3])
    # Q4_0: quantise a small matrix (one block on an exact grid, one all-zero block), decode it, multiply by a vector
    qn, qk = 5, 96
    qw = fill_normal(qn * qk, 0x2545F491, 31, 0.05).reshape(qn, qk)
    grid = [rne_bf16(np.float32((i * 7 % 16 - 8) / 64.0)) for i in range(32)]
    qw[1, 0:32] = np.array(grid, dtype=np.uint16)
    qw[2, 32:64] = 0
    qd, qs = q4_quantize(qw)
    g["q4_w"], g["q4_data"], g["q4_scales"] = qw, qd, qs
    g["q4_dequant"] = q4_dequant(qd, qs, qn, qk)
    assert np.array_equal(g["q4_dequant"][1, 0:32], qw[1, 0:32]) and not g["q4_dequant"][2, 32:64].any()
    qx = fill_normal(qk, 0x9E3779B9, 32, 1.0)
    g["q4_x"], g["q4_matvec"] = qx, q4_matvec(qd, qs, qx, qn, qk)
    g["q4s_matvec"] = q4s_matvec(qd, qs, qx, qn, qk)
    # matmul_q4 (kernels.rs:983-1071): three rows at a row stride of 104, every row summed as matvec_q4 sums its one
    qX = np.zeros((3, 104), dtype=np.uint16)
    qX[0, :qk] = qx
    qX[1:, :] = fill_normal(2 * 104, 0x9E3779B9, 33, 1.0).reshape(2, 104)
    g["q4_X"] = qX
    g["q4_matmul"] = np.stack([q4_matvec(qd, qs, qX[r, :qk], qn, qk) for r in range(3)])
    # matvec_q4_split: 80 blocks a row, so that with two and with four simdgroups a row every one of them has blocks
    sn, sk = 3, 2560
    sw = fill_normal(sn * sk, 0x2545F491, 34, 0.05).reshape(sn, sk)
    sd, ss = q4_quantize(sw)
    sx = fill_normal(sk, 0x9E3779B9, 35, 1.0)
    g["q4split_w"], g["q4split_x"] = sw, sx
    g["q4split_1"], g["q4split_2"], g["q4split_4"] = (q4_matvec(sd, ss, sx, sn, sk, sp) for sp in (1, 2, 4))
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **g)
    print("wrote", os.path.join(HERE, "golden.npz"), "with", len(g), "arrays")


if __name__ == "__main__":
    main()
