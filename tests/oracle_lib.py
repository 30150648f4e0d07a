"""ctypes binding of the CPU oracle (oracle/hb_oracle.c) for the tests.

The oracle is test infrastructure: it is loaded here, by the smoke run and by
the benchmark's CPU-baseline leg, never by the library under test.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle")

OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU = 0, 1, 2, 3


class Cmp(C.Structure):
    _fields_ = [
        ("count", C.c_size_t),
        ("over_1ulp", C.c_size_t),
        ("mismatched", C.c_size_t),
        ("max_ulp", C.c_uint32),
        ("max_abs_err", C.c_float),
        ("max_abs_ref", C.c_float),
    ]


def build(native: bool = False) -> str:
    """Compile the oracle if its library is missing or older than its source."""
    name = "libhb_oracle_native.so" if native else "libhb_oracle.so"
    so = os.path.join(_DIR, "_build", name)
    src = [os.path.join(_DIR, f) for f in ("hb_oracle.c", "hb_oracle.h")]
    if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in src):
        subprocess.run(["make", "-C", _DIR, "native" if native else "all"], check=True, capture_output=True)
    return so


_u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def load(native: bool = False) -> C.CDLL:
    lib = C.CDLL(build(native))
    lib.hbo_bf16_to_f32.restype = C.c_float
    lib.hbo_bf16_to_f32.argtypes = [C.c_uint16]
    lib.hbo_f32_to_bf16.restype = C.c_uint16
    lib.hbo_f32_to_bf16.argtypes = [C.c_float]
    lib.hbo_round_bf16.restype = C.c_float
    lib.hbo_round_bf16.argtypes = [C.c_float]
    lib.hbo_f64_to_bf16.restype = C.c_uint16
    lib.hbo_f64_to_bf16.argtypes = [C.c_double]
    lib.hbo_expf.restype = C.c_float
    lib.hbo_expf.argtypes = [C.c_float]
    lib.hbo_sigmoid.restype = C.c_float
    lib.hbo_sigmoid.argtypes = [C.c_float]
    lib.hbo_swiglu_one.restype = C.c_uint16
    lib.hbo_swiglu_one.argtypes = [C.c_uint16, C.c_uint16]
    for f in (lib.hbo_gemm_f64, lib.hbo_gemm_f32):
        f.restype = None
        f.argtypes = [_u16p, _u16p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.hbo_gemm_f64_rows.restype = None
    lib.hbo_gemm_f64_rows.argtypes = [_u16p, _u16p, C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.hbo_matvec_ref_order.restype = None
    lib.hbo_matvec_ref_order.argtypes = [_u16p, _u16p, _u16p, C.c_int, C.c_int]
    lib.hbo_swiglu_rows.restype = None
    lib.hbo_swiglu_rows.argtypes = [_u16p, _u16p, C.c_int, C.c_int]
    lib.hbo_route_topk.restype = None
    lib.hbo_route_topk.argtypes = [_u16p, _u32p, C.c_int, C.c_int, C.c_int]
    lib.hbo_moe_sort.restype = C.c_int
    lib.hbo_moe_sort.argtypes = [_u32p, C.c_int, C.c_int, C.c_int, C.c_int, _u32p, _u32p]
    lib.hbo_moe_gate_up.restype = None
    lib.hbo_moe_gate_up.argtypes = [_u16p, _u16p, _u32p, _u32p, _u16p, C.c_int, C.c_int, C.c_int]
    lib.hbo_swiglu_slots.restype = None
    lib.hbo_swiglu_slots.argtypes = [_u16p, _u16p, C.c_int, C.c_int]
    lib.hbo_moe_down.restype = None
    lib.hbo_moe_down.argtypes = [_u16p, _u16p, _u32p, _u32p, _u16p, C.c_int, C.c_int]
    for f in (lib.hbo_moe_combine, lib.hbo_moe_combine_f32):
        f.restype = None
        f.argtypes = [_u16p, _u32p, _u16p, C.c_int, C.c_int, C.c_int]
    lib.hbo_rmsnorm_rows.restype = None
    lib.hbo_rmsnorm_rows.argtypes = [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_float, C.c_int]
    lib.hbo_argmax_rows.restype = None
    lib.hbo_argmax_rows.argtypes = [_u16p, _u32p, C.c_int, C.c_int]
    lib.hbo_moe_out.restype = None
    lib.hbo_moe_out.argtypes = [_u16p, _u16p, _u16p, _u16p, _u16p, C.c_int, C.c_int]
    _u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
    lib.hbo_q4_quantize.restype = None
    lib.hbo_q4_quantize.argtypes = [_u16p, C.c_int, C.c_int, _u8p, _u16p]
    lib.hbo_q4_dequant.restype = None
    lib.hbo_q4_dequant.argtypes = [_u8p, _u16p, C.c_int, C.c_int, _u16p]
    lib.hbo_matmul_q4.restype = None
    lib.hbo_matmul_q4.argtypes = [_u8p, _u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    for f in (lib.hbo_matvec_q4, lib.hbo_matvec_q4s):
        f.restype = None
        f.argtypes = [_u8p, _u16p, _u16p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    lib.hbo_matvec_q4_split.restype = None
    lib.hbo_matvec_q4_split.argtypes = [_u8p, _u16p, _u16p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.hbo_check_1_64.restype = C.c_int
    lib.hbo_check_1_64.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    lib.hbo_fill_normal.restype = None
    lib.hbo_fill_normal.argtypes = [_u16p, C.c_size_t, C.c_uint64, C.c_uint64, C.c_double]
    lib.hbo_fill_xorshift16.restype = C.c_uint32
    lib.hbo_fill_xorshift16.argtypes = [_u16p, C.c_size_t, C.c_uint32]
    lib.hbo_fill_random16.restype = None
    lib.hbo_fill_random16.argtypes = [_u16p, C.c_size_t, C.c_uint64]
    lib.hbo_compare_bf16.restype = None
    lib.hbo_compare_bf16.argtypes = [_u16p, _u16p, C.c_size_t, C.POINTER(Cmp)]
    lib.hbo_threads.restype = C.c_int
    return lib


# Seeds of the synthetic tensors (the first two are the reference's own
# autotune seeds, qwen.rs:2607 and :2427).
SEED_X, SEED_W, SEED_Y, SEED_ROUTER = 0x9E3779B9, 0x2545F491, 0x85EBCA6B, 0xC2B2AE35


class Oracle:
    """Thin numpy-facing wrapper; every array is uint16 (bf16 bits) unless said."""

    def __init__(self, native: bool = False):
        self.lib = load(native)

    def threads(self) -> int:
        return int(self.lib.hbo_threads())

    def normal(self, shape, seed, tensor_id=0, sigma=1.0) -> np.ndarray:
        a = np.empty(shape, dtype=np.uint16)
        self.lib.hbo_fill_normal(a, a.size, seed, tensor_id, float(sigma))
        return a

    def xorshift16(self, shape, seed) -> np.ndarray:
        a = np.empty(shape, dtype=np.uint16)
        self.lib.hbo_fill_xorshift16(a, a.size, seed)
        return a

    def random16(self, shape, seed) -> np.ndarray:
        a = np.empty(shape, dtype=np.uint16)
        self.lib.hbo_fill_random16(a, a.size, seed)
        return a

    def _gemm(self, fn, x, w, out, y0):
        m, k = x.shape
        n = w.shape[0]
        assert w.shape[1] == k
        if out == OUT_F32:
            y = np.zeros((m, n), dtype=np.float32)
        elif out == OUT_SWIGLU:
            y = np.zeros((m, n // 2), dtype=np.uint16)
        elif out == OUT_RESIDUAL:
            y = np.ascontiguousarray(y0).copy()
        else:
            y = np.zeros((m, n), dtype=np.uint16)
        fn(np.ascontiguousarray(x), np.ascontiguousarray(w), y.ctypes.data, m, n, k, out)
        return y

    def gemm_f64(self, x, w, out=OUT_BF16, y0=None):
        return self._gemm(self.lib.hbo_gemm_f64, x, w, out, y0)

    def gemm_f32(self, x, w, out=OUT_BF16, y0=None):
        return self._gemm(self.lib.hbo_gemm_f32, x, w, out, y0)

    def gemm_f64_rows(self, x, w, rows, out=OUT_BF16, y0=None):
        """Full-size output array in which only `rows` are computed."""
        m, k = x.shape
        n = w.shape[0]
        rows = np.ascontiguousarray(np.asarray(rows, dtype=np.int32))
        if out == OUT_F32:
            y = np.zeros((m, n), dtype=np.float32)
        elif out == OUT_SWIGLU:
            y = np.zeros((m, n // 2), dtype=np.uint16)
        elif out == OUT_RESIDUAL:
            y = np.ascontiguousarray(y0).copy()
        else:
            y = np.zeros((m, n), dtype=np.uint16)
        self.lib.hbo_gemm_f64_rows(np.ascontiguousarray(x), np.ascontiguousarray(w), y.ctypes.data, rows, len(rows), n, k, out)
        return y

    def matvec_ref_order(self, x, w):
        n, k = w.shape
        y = np.zeros(n, dtype=np.uint16)
        self.lib.hbo_matvec_ref_order(np.ascontiguousarray(x.reshape(-1)), np.ascontiguousarray(w), y, n, k)
        return y

    def swiglu_rows(self, gu):
        m, n2 = gu.shape
        h = np.zeros((m, n2 // 2), dtype=np.uint16)
        self.lib.hbo_swiglu_rows(np.ascontiguousarray(gu), h, m, n2 // 2)
        return h

    def route_topk(self, scores, top_k):
        rows, experts = scores.shape
        route = np.zeros((rows, 2 * top_k), dtype=np.uint32)
        self.lib.hbo_route_topk(np.ascontiguousarray(scores), route, rows, experts, top_k)
        return route

    def moe_sort(self, route, experts, top_k, bm):
        rows = route.shape[0]
        pairs = rows * top_k
        max_tiles = (pairs + bm - 1) // bm + experts
        lst = np.zeros(pairs, dtype=np.uint32)
        tiles = np.zeros(1 + 3 * max_tiles, dtype=np.uint32)
        self.lib.hbo_moe_sort(np.ascontiguousarray(route), rows, experts, top_k, bm, lst, tiles)
        return lst, tiles

    def moe_gate_up(self, x, wgu, lst, tiles, mi, top_k):
        h = x.shape[1]
        egu = np.zeros((len(lst), 2 * mi), dtype=np.uint16)
        self.lib.hbo_moe_gate_up(np.ascontiguousarray(x), np.ascontiguousarray(wgu), lst, tiles, egu, h, mi, top_k)
        return egu

    def swiglu_slots(self, egu):
        pairs, mi2 = egu.shape
        ehb = np.zeros((pairs, mi2 // 2), dtype=np.uint16)
        self.lib.hbo_swiglu_slots(np.ascontiguousarray(egu), ehb, pairs, mi2 // 2)
        return ehb

    def moe_down(self, ehb, wd, lst, tiles, h):
        pairs, mi = ehb.shape
        ey = np.zeros((pairs, h), dtype=np.uint16)
        self.lib.hbo_moe_down(np.ascontiguousarray(ehb), np.ascontiguousarray(wd), lst, tiles, ey, h, mi)
        return ey

    def moe_combine(self, ey, route, top_k, f32=False):
        rows = route.shape[0]
        d = ey.shape[1]
        out = np.zeros((rows, d), dtype=np.uint16)
        fn = self.lib.hbo_moe_combine_f32 if f32 else self.lib.hbo_moe_combine
        fn(np.ascontiguousarray(ey), np.ascontiguousarray(route), out, rows, d, top_k)
        return out

    def rmsnorm_rows(self, x, w, eps=1e-6, plus_one=False):
        rows, d = x.shape
        y = np.zeros((rows, d), dtype=np.uint16)
        self.lib.hbo_rmsnorm_rows(np.ascontiguousarray(x), np.ascontiguousarray(w), y, rows, d, float(eps), int(plus_one))
        return y

    def argmax_rows(self, logits):
        rows, n = logits.shape
        idx = np.zeros(rows, dtype=np.uint32)
        self.lib.hbo_argmax_rows(np.ascontiguousarray(logits), idx, rows, n)
        return idx

    def moe_out(self, xn, gate, experts, shared, x):
        rows, d = x.shape
        out = np.ascontiguousarray(x).copy()
        self.lib.hbo_moe_out(np.ascontiguousarray(xn), np.ascontiguousarray(gate), np.ascontiguousarray(experts), np.ascontiguousarray(shared), out, rows, d)
        return out

    def q4_quantize(self, w):
        """(data uint8 [n*k/2], scales f16 bits uint16 [n*k/32]) of W [n][k] bf16 (reference src/metal/q4.rs)."""
        n, k = w.shape
        data = np.zeros(n * k // 2, dtype=np.uint8)
        scales = np.zeros(n * k // 32, dtype=np.uint16)
        self.lib.hbo_q4_quantize(np.ascontiguousarray(w), n, k, data, scales)
        return data, scales

    def q4_dequant(self, data, scales, n, k):
        out = np.zeros((n, k), dtype=np.uint16)
        self.lib.hbo_q4_dequant(data, scales, n, k, out)
        return out

    def matmul_q4(self, data, scales, x, n, k, ldy=None):
        """Y [m][ldy] (bf16 bits; columns past n stay 0) for X [m][ldx] (reference matmul_q4, src/metal/kernels.rs:983)."""
        x = np.ascontiguousarray(x)
        m, ldx = x.shape
        ldy = ldy or n
        y = np.zeros((m, ldy), dtype=np.uint16)
        self.lib.hbo_matmul_q4(data, scales, x, y, n, k, m, ldx, ldy)
        return y

    def matvec_q4(self, data, scales, x, n, k, out=OUT_BF16, y0=None, masks=False, split=1):
        y = np.zeros(n, dtype=np.float32 if out == OUT_F32 else np.uint16) if y0 is None else np.ascontiguousarray(y0).copy()
        if split > 1:
            assert not masks
            self.lib.hbo_matvec_q4_split(data, scales, np.ascontiguousarray(x), y.ctypes.data, n, k, out, split)
        else:
            (self.lib.hbo_matvec_q4s if masks else self.lib.hbo_matvec_q4)(data, scales, np.ascontiguousarray(x), y.ctypes.data, n, k, out)
        return y

    def check_1_64(self, ref, got):
        f32_out = ref.dtype == np.float32
        err, scale = C.c_float(), C.c_float()
        ok = self.lib.hbo_check_1_64(ref.ctypes.data, np.ascontiguousarray(got).ctypes.data, ref.size, int(f32_out), C.byref(err), C.byref(scale))
        return bool(ok), err.value, scale.value

    def compare(self, ref, got) -> Cmp:
        c = Cmp()
        self.lib.hbo_compare_bf16(np.ascontiguousarray(ref).reshape(-1), np.ascontiguousarray(got).reshape(-1), ref.size, C.byref(c))
        return c


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def assert_within_contract(cmp: Cmp, what: str = "") -> None:
    """<= 1 bf16 ulp on >= 99.9 % of elements and max|err| <= max|ref|/64."""
    frac = cmp.over_1ulp / max(cmp.count, 1)
    assert frac <= 1e-3, f"{what}: {cmp.over_1ulp}/{cmp.count} elements over 1 bf16 ulp (max {cmp.max_ulp} ulp)"
    assert cmp.max_abs_err <= cmp.max_abs_ref / 64.0, f"{what}: max err {cmp.max_abs_err} over 1/64 of {cmp.max_abs_ref}"
