"""Python face of libhb200.so: a thin ctypes binding of include/hb200.h.

The directory name is not a Python identifier; load it with

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("hb200", ".../herbert-metal-bf16_b200/__init__.py")
    hb200 = importlib.util.module_from_spec(spec); sys.modules["hb200"] = hb200; spec.loader.exec_module(hb200)

Everything computes on the GPU through the C ABI. There is no CPU path: a missing library or a
missing sm_100 device raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libhb200.so")

OK, INVALID, UNSUPPORTED, BACKEND, OOM, KERNEL = range(6)
OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU = range(4)
ROWS_DENSE, ROWS_GATHER, ROWS_SCATTER, ROWS_SORTED = range(4)
X_PLAIN, X_NORM, X_SWIGLU = range(3)
OUT_NAMES = {OUT_BF16: "Bf16", OUT_F32: "F32", OUT_RESIDUAL: "Residual", OUT_SWIGLU: "Swiglu"}


class HbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"hb200 status {status}: {message}")
        self.status = status
        self.message = message


class Range(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("size", C.c_size_t)]


class Op(C.Structure):
    _fields_ = [("kernel", C.c_void_p), ("args", C.POINTER(Range)), ("nargs", C.c_int), ("m", C.c_uint32)]


class GemmDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("k", "n", "out", "rows_mode", "top_k", "experts", "bm", "tile_n", "stages", "cta_pair", "m_first", "rows_max", "stream_k", "merge_runs", "y_shards", "y_group_rows", "y_signal", "split_k")]


class MatvecDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("k", "n", "out", "rows_max", "rows_per_warp", "split", "persist", "x_stationary", "tensor_core", "argmax", "x_src", "norm_eps_bits", "norm_plus_one")]


class ExpertIo(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("experts", "top_k", "h", "mi", "m")] + [
        (n, Range) for n in ("route", "list", "tiles", "x", "wgu", "wdown", "ehb", "ey", "egu", "xs")
    ]


class ExpertPick(C.Structure):
    _fields_ = [("bm", C.c_uint32), ("sort", C.c_void_p), ("gather", C.c_void_p), ("gate_up", C.c_void_p), ("swiglu", C.c_void_p), ("down", C.c_void_p)]


_lib = None


def build(force: bool = False) -> str:
    import importlib.util

    spec = importlib.util.spec_from_file_location("hb200_build", os.path.join(_HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(force=force)


def lib() -> C.CDLL:
    """The loaded library; raises when it has not been built (no fallback of any kind)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise HbError(BACKEND, f"{LIB_PATH} is missing: build it with `python herbert-metal-bf16_b200/build.py` (there is no CPU path)")
    L = C.CDLL(LIB_PATH)
    vp, u32, sz, ci = C.c_void_p, C.c_uint32, C.c_size_t, C.c_int
    pvp = C.POINTER(C.c_void_p)
    sigs = {
        "hb_open": (ci, [ci, pvp]),
        "hb_close": (ci, [vp]),
        "hb_last_error": (C.c_char_p, [vp]),
        "hb_describe": (ci, [vp, C.c_char_p, sz]),
        "hb_set_stream": (ci, [vp, vp]),
        "hb_alloc": (ci, [vp, sz, pvp]),
        "hb_set_alloc_limit": (ci, [vp, sz]),
        "hb_upload": (ci, [vp, vp, vp, sz]),
        "hb_download": (ci, [vp, vp, vp, sz]),
        "hb_memset": (ci, [vp, vp, ci, sz]),
        "hb_sync": (ci, [vp]),
        "hb_launch_count": (C.c_uint64, [vp]),
        "hb_ipc_export": (ci, [vp, vp, vp]),
        "hb_ipc_open": (ci, [vp, vp, pvp]),
        "hb_ipc_close": (ci, [vp, vp]),
        "hb_ep_dispatch_get": (ci, [vp, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_ep_return_get": (ci, [vp, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_ep_plan_get": (ci, [vp, u32, u32, u32, u32, u32, pvp]),
        "hb_ep_combine_get": (ci, [vp, u32, u32, u32, pvp]),
        "hb_ep_combine_sync_get": (ci, [vp, u32, u32, u32, u32, pvp]),
        "hb_ep_dispatch_direct_get": (ci, [vp, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_ep_plan_direct_get": (ci, [vp, u32, u32, u32, u32, u32, pvp]),
        "hb_tp_reduce_get": (ci, [vp, u32, u32, u32, u32, pvp]),
        "hb_tp_sum_get": (ci, [vp, u32, u32, u32, u32, pvp]),
        "hb_tp_sum_sync_get": (ci, [vp, u32, u32, u32, u32, pvp]),
        "hb_tp_sum_stream_get": (ci, [vp, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_dequant_q4_get": (ci, [vp, u32, u32, pvp]),
        "hb_matvec_q4_get": (ci, [vp, u32, u32, u32, u32, u32, pvp]),
        "hb_matvec_q4_split_get": (ci, [vp, u32, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_matmul_q4_get": (ci, [vp, u32, u32, u32, u32, u32, pvp]),
        "hb_gemm_q4_get": (ci, [vp, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_select_gemm_q4": (ci, [vp, u32, u32, u32, Range, Range, Range, Range, Range, u32, pvp, C.POINTER(ci)]),
        "hb_rmsnorm_get": (ci, [vp, u32, C.c_float, u32, pvp]),
        "hb_argmax_get": (ci, [vp, u32, u32, pvp]),
        "hb_moe_out_get": (ci, [vp, u32, pvp]),
        "hb_peer_sync_get": (ci, [vp, u32, u32, u32, pvp]),
        "hb_set_peer_wait_ms": (ci, [vp, u32]),
        "hb_set_launch_overlap": (ci, [vp, ci]),
        "hb_graph_record": (ci, [vp, C.POINTER(Op), ci, pvp]),
        "hb_graph_launch": (ci, [vp, vp]),
        "hb_graph_time": (ci, [vp, vp, ci, C.POINTER(C.c_double)]),
        "hb_graph_free": (ci, [vp, vp]),
        "hb_event_new": (ci, [vp, pvp]),
        "hb_event_free": (ci, [vp, vp]),
        "hb_lane_record": (ci, [vp, ci, vp]),
        "hb_lane_wait": (ci, [vp, ci, vp]),
        "hb_event_sync": (ci, [vp, vp]),
        "hb_upload_async": (ci, [vp, vp, vp, sz]),
        "hb_download_async": (ci, [vp, vp, vp, sz]),
        "hb_host_alloc": (ci, [vp, sz, pvp]),
        "hb_host_free": (ci, [vp, vp]),
        "hb_gemm_get": (ci, [vp, C.POINTER(GemmDesc), pvp]),
        "hb_matvec_get": (ci, [vp, C.POINTER(MatvecDesc), pvp]),
        "hb_swiglu_get": (ci, [vp, u32, pvp]),
        "hb_route_get": (ci, [vp, u32, u32, pvp]),
        "hb_moe_sort_get": (ci, [vp, u32, u32, u32, u32, pvp]),
        "hb_moe_tiles": (u32, [u32, u32, u32, u32]),
        "hb_moe_gather_get": (ci, [vp, u32, u32, pvp]),
        "hb_moe_combine_get": (ci, [vp, u32, u32, u32, pvp]),
        "hb_experts_matvec_get": (ci, [vp, u32, u32, u32, u32, u32, u32, u32, pvp]),
        "hb_epilogue_get": (ci, [vp, u32, u32, pvp]),
        "hb_gemm_static_scratch": (ci, [vp, u32, u32, u32, u32, Range, Range, Range]),
        "hb_kernel_name": (C.c_char_p, [vp]),
        "hb_launch": (ci, [vp, vp, C.POINTER(Range), ci, u32]),
        "hb_run": (ci, [vp, C.POINTER(Op), ci]),
        "hb_time": (ci, [vp, C.POINTER(Op), ci, ci, C.POINTER(C.c_double)]),
        "hb_tune_new": (ci, [pvp]),
        "hb_tune_free": (None, [vp]),
        "hb_tune_apply": (ci, [vp, C.c_char_p, C.c_char_p, sz]),
        "hb_tune_get": (ci, [vp, C.c_char_p, C.POINTER(u32)]),
        "hb_tune_summary": (ci, [vp, C.c_char_p, sz]),
        "hb_tune_gemm_timed": (ci, [vp]),
        "hb_selector_new": (ci, [vp, vp, pvp]),
        "hb_selector_free": (None, [vp]),
        "hb_selector_log": (C.c_char_p, [vp]),
        "hb_selector_buckets": (ci, [vp, C.POINTER(u32), ci]),
        "hb_fill_random16": (ci, [vp, Range, u32]),
        "hb_select_gemm": (ci, [vp, u32, u32, u32, Range, Range, Range, u32, pvp]),
        "hb_select_gate_up": (ci, [vp, u32, u32, Range, Range, Range, Range, u32, pvp, C.POINTER(ci)]),
        "hb_select_matvec": (ci, [vp, u32, u32, u32, u32, C.POINTER(Range), ci, Range, Range, pvp]),
        "hb_select_matvec_x": (ci, [vp, u32, u32, u32, u32, u32, u32, u32, C.POINTER(Range), ci, Range, Range, Range, pvp]),
        "hb_select_axis": (ci, [vp, C.c_char_p, C.c_char_p, C.POINTER(C.POINTER(Op)), C.POINTER(ci), C.POINTER(u32), ci, u32, C.POINTER(u32)]),
        "hb_select_experts": (ci, [vp, C.POINTER(ExpertIo), C.POINTER(ExpertPick)]),
        "hb_selector_inject_wrong": (ci, [vp, ci]),
        "hb_check_rule": (ci, [vp, vp, sz, ci, C.POINTER(ci), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(L, name)  # AttributeError here = the library does not export what the header declares
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


EXPORTS = [
    "hb_open", "hb_close", "hb_last_error", "hb_describe", "hb_set_stream", "hb_alloc", "hb_set_alloc_limit", "hb_upload",
    "hb_download", "hb_memset", "hb_sync", "hb_launch_count", "hb_event_new", "hb_event_free", "hb_lane_record", "hb_lane_wait", "hb_event_sync",
    "hb_upload_async", "hb_download_async", "hb_host_alloc", "hb_host_free", "hb_ipc_export", "hb_ipc_open", "hb_ipc_close",
    "hb_ep_dispatch_get", "hb_ep_plan_get", "hb_ep_return_get", "hb_ep_combine_get", "hb_ep_combine_sync_get", "hb_ep_dispatch_direct_get", "hb_ep_plan_direct_get", "hb_tp_reduce_get", "hb_tp_sum_get", "hb_tp_sum_sync_get", "hb_tp_sum_stream_get", "hb_dequant_q4_get", "hb_matvec_q4_get", "hb_matvec_q4_split_get", "hb_matmul_q4_get", "hb_gemm_q4_get", "hb_select_gemm_q4", "hb_rmsnorm_get", "hb_argmax_get", "hb_moe_out_get", "hb_peer_sync_get", "hb_set_peer_wait_ms", "hb_gemm_get", "hb_matvec_get", "hb_swiglu_get", "hb_route_get",
    "hb_moe_sort_get", "hb_moe_tiles", "hb_moe_gather_get", "hb_moe_combine_get", "hb_experts_matvec_get", "hb_epilogue_get", "hb_gemm_static_scratch", "hb_kernel_name", "hb_launch", "hb_run", "hb_time", "hb_set_launch_overlap", "hb_graph_record", "hb_graph_launch", "hb_graph_time", "hb_graph_free",
    "hb_tune_new", "hb_tune_free", "hb_tune_apply", "hb_tune_get", "hb_tune_summary", "hb_tune_gemm_timed", "hb_selector_new",
    "hb_selector_free", "hb_selector_log", "hb_selector_buckets", "hb_fill_random16", "hb_select_gemm", "hb_select_gate_up",
    "hb_select_matvec", "hb_select_matvec_x", "hb_select_axis", "hb_select_experts", "hb_selector_inject_wrong", "hb_check_rule",
]


LANE_KERNELS, LANE_UPLOAD, LANE_DOWNLOAD = 0, 1, 2


class Event:
    """A mark in a lane of a Context: record it on one lane, make another lane (or the host) wait for it."""

    def __init__(self, ctx: "Context", h):
        self.ctx, self.h = ctx, h

    def record(self, lane: int) -> "Event":
        self.ctx._check(lib().hb_lane_record(self.ctx.h, lane, self.h))
        return self

    def wait(self, lane: int) -> None:
        self.ctx._check(lib().hb_lane_wait(self.ctx.h, lane, self.h))

    def sync(self) -> None:
        self.ctx._check(lib().hb_event_sync(self.ctx.h, self.h))

    def free(self) -> None:
        if self.h:
            lib().hb_event_free(self.ctx.h, self.h)
            self.h = None


class StreamedBlocks:
    """Runs the same kernels over a stream of host blocks, the copies of one block under the kernels of another.

    `sets` is a list (two or more) of (ops, device_in, device_out): the same kernels bound to separate device
    buffers. step(i, host_in, host_out) enqueues upload -> kernels -> download of block i on buffer set
    i % len(sets) and returns without waiting; the upload waits for the kernels that last read that set's input,
    the kernels wait for the upload and for the download that last read that set's output. wait(i) blocks the
    host until block i's result is in host_out.
    """

    def __init__(self, ctx: "Context", sets):
        assert len(sets) >= 2
        self.ctx, self.sets = ctx, sets
        self.prepared = [ctx.make_ops(ops) + (len(ops),) for ops, _, _ in sets]  # the hb_op arrays, built once
        self.up = [ctx.event() for _ in sets]
        self.done = [ctx.event() for _ in sets]
        self.down = [ctx.event() for _ in sets]

    def step(self, i: int, host_in: np.ndarray, host_out: np.ndarray) -> None:
        s = i % len(self.sets)
        ops, d_in, d_out = self.sets[s]
        self.done[s].wait(LANE_UPLOAD)      # the kernels that read this input two blocks ago
        self.ctx.upload_async(d_in, host_in)
        self.up[s].record(LANE_UPLOAD)
        self.up[s].wait(LANE_KERNELS)
        self.down[s].wait(LANE_KERNELS)     # the download that read this output two blocks ago
        arr, _keep, nops = self.prepared[s]
        self.ctx._check(lib().hb_run(self.ctx.h, arr, nops))
        self.done[s].record(LANE_KERNELS)
        self.done[s].wait(LANE_DOWNLOAD)
        self.ctx.download_async(host_out, d_out)
        self.down[s].record(LANE_DOWNLOAD)

    def wait(self, i: int) -> None:
        self.down[i % len(self.sets)].sync()

    def close(self) -> None:
        for e in self.up + self.done + self.down:
            e.free()


class Buffer:
    """A device range owned by a Context (or wrapping foreign device memory)."""

    def __init__(self, ctx: "Context", ptr: int, size: int):
        self.ctx, self.ptr, self.size = ctx, ptr, size

    def range(self, offset: int = 0, size: int | None = None) -> Range:
        size = self.size - offset if size is None else size
        assert 0 <= offset and offset + size <= self.size, "range outside its buffer"
        return Range(self.ptr + offset, size)

    def upload(self, a: np.ndarray, offset: int = 0) -> "Buffer":
        a = np.ascontiguousarray(a)
        assert offset + a.nbytes <= self.size
        self.ctx._check(lib().hb_upload(self.ctx.h, self.ptr + offset, a.ctypes.data, a.nbytes))
        return self

    def download(self, dtype, shape, offset: int = 0) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert offset + out.nbytes <= self.size
        self.ctx._check(lib().hb_download(self.ctx.h, out.ctypes.data, self.ptr + offset, out.nbytes))
        return out

    def zero(self) -> None:
        self.ctx._check(lib().hb_memset(self.ctx.h, self.ptr, 0, self.size))


class Kernel:
    def __init__(self, ctx: "Context", handle: int):
        self.ctx, self.h = ctx, handle

    @property
    def name(self) -> str:
        return lib().hb_kernel_name(self.h).decode()

    def __call__(self, m: int, *bufs) -> None:
        self.ctx.launch(self, m, *bufs)


def _as_range(b) -> Range:
    if isinstance(b, Range):
        return b
    if isinstance(b, Buffer):
        return b.range()
    ptr, size = b
    return Range(int(ptr), int(size))


class Context:
    """hb_ctx: one device, one stream. Not thread-safe."""

    def __init__(self, device: int = 0):
        L = lib()
        h = C.c_void_p()
        st = L.hb_open(device, C.byref(h))
        if st != OK:
            raise HbError(st, L.hb_last_error(None).decode())
        self.h = h

    def close(self) -> None:
        if self.h:
            lib().hb_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, st: int) -> None:
        if st != OK:
            raise HbError(st, lib().hb_last_error(self.h).decode())

    def describe(self) -> str:
        buf = C.create_string_buffer(256)
        self._check(lib().hb_describe(self.h, buf, 256))
        return buf.value.decode()

    def set_stream(self, cuda_stream: int | None) -> None:
        self._check(lib().hb_set_stream(self.h, cuda_stream))

    def alloc(self, nbytes: int) -> Buffer:
        p = C.c_void_p()
        self._check(lib().hb_alloc(self.h, nbytes, C.byref(p)))
        return Buffer(self, p.value, nbytes)

    def wrap(self, ptr: int, nbytes: int) -> Buffer:
        return Buffer(self, ptr, nbytes)

    def to_device(self, a: np.ndarray) -> Buffer:
        a = np.ascontiguousarray(a)
        return self.alloc(max(a.nbytes, 16)).upload(a)

    def sync(self) -> None:
        self._check(lib().hb_sync(self.h))

    def memset(self, buf: "Buffer", value: int = 0) -> None:
        self._check(lib().hb_memset(self.h, buf.ptr, value, buf.size))

    def launch_count(self) -> int:
        return int(lib().hb_launch_count(self.h))

    # ---- peer memory
    def ipc_export(self, buf: "Buffer") -> bytes:
        h = C.create_string_buffer(64)
        self._check(lib().hb_ipc_export(self.h, buf.ptr, h))
        return h.raw

    def ipc_open(self, handle: bytes, nbytes: int) -> "Buffer":
        p = C.c_void_p()
        self._check(lib().hb_ipc_open(self.h, handle, C.byref(p)))
        return Buffer(self, p.value, nbytes)

    def ipc_close(self, buf: "Buffer") -> None:
        self._check(lib().hb_ipc_close(self.h, buf.ptr))

    def ep_dispatch(self, h, top_k, experts, world, rank, cap, direct=False) -> "Kernel":
        return self._get(lib().hb_ep_dispatch_direct_get if direct else lib().hb_ep_dispatch_get, h, top_k, experts, world, rank, cap)

    def ep_return(self, h, top_k, experts, world, rank, cap) -> "Kernel":
        return self._get(lib().hb_ep_return_get, h, top_k, experts, world, rank, cap)

    def ep_combine(self, h, top_k, world, sync_rank=None) -> "Kernel":
        """sync_rank: this rank, for the form that carries the barrier before it (hb_ep_combine_sync_get)."""
        if sync_rank is not None:
            return self._get(lib().hb_ep_combine_sync_get, h, top_k, world, sync_rank)
        return self._get(lib().hb_ep_combine_get, h, top_k, world)

    def set_peer_wait_ms(self, ms: int) -> None:
        self._check(lib().hb_set_peer_wait_ms(self.h, ms))

    def peer_sync(self, words, world, rank) -> "Kernel":
        return self._get(lib().hb_peer_sync_get, words, world, rank)

    def dequant_q4(self, k, n) -> "Kernel":
        return self._get(lib().hb_dequant_q4_get, k, n)

    def matvec_q4(self, k, n, out=OUT_BF16, rows_per_warp=2, masks=0, split=1, persist=0) -> "Kernel":
        if split > 1 or persist:
            return self._get(lib().hb_matvec_q4_split_get, k, n, out, rows_per_warp, masks, split, persist)
        return self._get(lib().hb_matvec_q4_get, k, n, out, rows_per_warp, masks)

    def matmul_q4(self, k, n, m, ldx=0, ldy=0) -> "Kernel":
        return self._get(lib().hb_matmul_q4_get, k, n, m, ldx or k, ldy or n)

    def gemm_q4(self, k, n, out=OUT_BF16, tile_n=0, m_first=1, rows_max=2048) -> "Kernel":
        return self._get(lib().hb_gemm_q4_get, k, n, out, tile_n, m_first, rows_max)

    def rmsnorm(self, d, eps=1e-6, plus_one=False) -> "Kernel":
        return self._get(lib().hb_rmsnorm_get, d, C.c_float(eps), 1 if plus_one else 0)

    def argmax(self, n, rows_max=1) -> "Kernel":
        return self._get(lib().hb_argmax_get, n, rows_max)

    def moe_out(self, d) -> "Kernel":
        return self._get(lib().hb_moe_out_get, d)

    def tp_sum(self, n, out, world, rank, sync=False) -> "Kernel":
        """sync: the form that carries the step's two barriers (hb_tp_sum_sync_get; bindings staging, peers_y, peers_flags, ctl)."""
        return self._get(lib().hb_tp_sum_sync_get if sync else lib().hb_tp_sum_get, n, out, world, rank)

    def tp_sum_stream(self, n, out, world, rank, group_rows=256, sync=1) -> "Kernel":
        return self._get(lib().hb_tp_sum_stream_get, n, out, world, rank, group_rows, sync)

    def tp_reduce(self, n, out, world, rank) -> "Kernel":
        return self._get(lib().hb_tp_reduce_get, n, out, world, rank)

    def ep_plan(self, experts, world, rank, bm, cap, direct=False) -> "Kernel":
        return self._get(lib().hb_ep_plan_direct_get if direct else lib().hb_ep_plan_get, experts, world, rank, bm, cap)

    # ---- copy lanes (kernels 0, upload 1, download 2): in-order queues tied together by events
    def event(self) -> "Event":
        e = C.c_void_p()
        self._check(lib().hb_event_new(self.h, C.byref(e)))
        return Event(self, e)

    def host_array(self, shape, dtype=np.uint16) -> np.ndarray:
        """Page-locked host memory as a numpy array; it lives as long as the context."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self._check(lib().hb_host_alloc(self.h, n, C.byref(p)))
        raw = (C.c_uint8 * n).from_address(p.value)
        return np.frombuffer(raw, dtype=dtype).reshape(shape)

    def upload_async(self, dst: Buffer, src: np.ndarray) -> None:
        assert src.flags.c_contiguous and src.nbytes <= dst.size
        self._check(lib().hb_upload_async(self.h, dst.ptr, src.ctypes.data, src.nbytes))

    def download_async(self, dst: np.ndarray, src: Buffer) -> None:
        assert dst.flags.c_contiguous and dst.nbytes <= src.size
        self._check(lib().hb_download_async(self.h, dst.ctypes.data, src.ptr, dst.nbytes))

    # ---- kernels
    def _get(self, fn, *args) -> Kernel:
        k = C.c_void_p()
        self._check(fn(self.h, *args, C.byref(k)))
        return Kernel(self, k.value)

    def gemm(self, k, n, out=OUT_BF16, rows_max=2048, tile_n=0, stages=0, cta_pair=0, m_first=1, rows_mode=ROWS_DENSE, top_k=0, experts=0, bm=0, merge_runs=0, stream_k=0, y_shards=0, y_group_rows=0, y_signal=0, split_k=0) -> Kernel:
        d = GemmDesc(k, n, out, rows_mode, top_k, experts, bm, tile_n, stages, cta_pair, m_first, rows_max, stream_k, merge_runs, y_shards, y_group_rows, y_signal, split_k)
        return self._get(lib().hb_gemm_get, C.byref(d))

    def matvec(self, k, n, out=OUT_BF16, rows_max=1, rows_per_warp=2, split=1, persist=0, x_stationary=0, tensor_core=0, argmax=0, x_src=X_PLAIN, norm_eps_bits=0,
               norm_plus_one=0) -> Kernel:
        d = MatvecDesc(k, n, out, rows_max, rows_per_warp, split, persist, x_stationary, tensor_core, argmax, x_src, norm_eps_bits, norm_plus_one)
        return self._get(lib().hb_matvec_get, C.byref(d))

    def swiglu_rows(self, n) -> Kernel:
        return self._get(lib().hb_swiglu_get, n)

    def route(self, experts, top_k) -> Kernel:
        return self._get(lib().hb_route_get, experts, top_k)

    def moe_sort(self, experts, top_k, rows_max, bm) -> Kernel:
        return self._get(lib().hb_moe_sort_get, experts, top_k, rows_max, bm)

    def moe_gather(self, h, top_k) -> Kernel:
        return self._get(lib().hb_moe_gather_get, h, top_k)

    def experts_matvec(self, k, n, top_k, experts, x_row, x_stride=0, rows_per_warp=2) -> Kernel:
        return self._get(lib().hb_experts_matvec_get, k, n, top_k, experts, x_row, x_stride, rows_per_warp)

    def moe_combine(self, d, top_k, f32_sum=0) -> Kernel:
        return self._get(lib().hb_moe_combine_get, d, top_k, f32_sum)

    def epilogue(self, n, out=OUT_BF16) -> Kernel:
        return self._get(lib().hb_epilogue_get, n, out)

    def launch(self, kernel: Kernel, m: int, *bufs) -> None:
        arr = (Range * len(bufs))(*[_as_range(b) for b in bufs])
        self._check(lib().hb_launch(self.h, kernel.h, arr, len(bufs), m))

    def make_ops(self, ops):
        """ops: list of (kernel, m, bufs...) -> (Op array, keepalive)."""
        keep = []
        arr = (Op * len(ops))()
        for i, (kern, m, *bufs) in enumerate(ops):
            ra = (Range * len(bufs))(*[_as_range(b) for b in bufs])
            keep.append(ra)
            arr[i] = Op(kern.h, ra, len(bufs), m)
        return arr, keep

    def run(self, ops) -> None:
        arr, keep = self.make_ops(ops)
        self._check(lib().hb_run(self.h, arr, len(ops)))

    def set_launch_overlap(self, on: bool) -> None:
        self._check(lib().hb_set_launch_overlap(self.h, 1 if on else 0))

    def record(self, ops) -> "Graph":
        """The op sequence as one replayable object (hb_graph_record)."""
        arr, keep = self.make_ops(ops)
        g = C.c_void_p()
        self._check(lib().hb_graph_record(self.h, arr, len(ops), C.byref(g)))
        return Graph(self, g, keep)

    def time(self, ops, reps: int = 1) -> float:
        """GPU seconds of `reps` runs of the op sequence (events on the stream)."""
        arr, keep = self.make_ops(ops)
        sec = C.c_double()
        self._check(lib().hb_time(self.h, arr, len(ops), reps, C.byref(sec)))
        return sec.value


class Graph:
    """A recorded op sequence: launch() replays it with one call, time(reps) gives the GPU seconds of `reps` replays."""

    def __init__(self, ctx: Context, h, keep):
        self.ctx, self.h, self.keep = ctx, h, keep

    def launch(self) -> None:
        self.ctx._check(lib().hb_graph_launch(self.ctx.h, self.h))

    def time(self, reps: int = 1) -> float:
        sec = C.c_double()
        self.ctx._check(lib().hb_graph_time(self.ctx.h, self.h, reps, C.byref(sec)))
        return sec.value

    def free(self) -> None:
        if self.h:
            lib().hb_graph_free(self.ctx.h, self.h)
            self.h = None


class Tune:
    """hb_tune: the reference's --tune key=value settings for this path."""

    def __init__(self, settings: str = ""):
        h = C.c_void_p()
        st = lib().hb_tune_new(C.byref(h))
        if st != OK:
            raise HbError(st, "hb_tune_new failed")
        self.h = h
        if settings:
            self.apply(settings)

    def apply(self, settings: str) -> None:
        err = C.create_string_buffer(512)
        st = lib().hb_tune_apply(self.h, settings.encode(), err, 512)
        if st != OK:
            raise HbError(st, err.value.decode())

    def get(self, key: str) -> int:
        v = C.c_uint32()
        st = lib().hb_tune_get(self.h, key.encode(), C.byref(v))
        if st != OK:
            raise HbError(st, f"--tune {key}: unknown")
        return v.value

    def summary(self) -> str:
        buf = C.create_string_buffer(4096)
        lib().hb_tune_summary(self.h, buf, 4096)
        return buf.value.decode()

    def gemm_timed(self) -> bool:
        return bool(lib().hb_tune_gemm_timed(self.h))

    def __del__(self):
        try:
            if self.h:
                lib().hb_tune_free(self.h)
                self.h = None
        except Exception:
            pass


class Selector:
    """hb_selector: the load-time selection loop (candidates, 1/64 check, timing, cached picks)."""

    def __init__(self, ctx: Context, tune: Tune):
        h = C.c_void_p()
        ctx._check(lib().hb_selector_new(ctx.h, tune.h, C.byref(h)))
        self.ctx, self.h, self._tune = ctx, h, tune

    def close(self) -> None:
        if self.h:
            lib().hb_selector_free(self.h)
            self.h = None

    def log(self) -> str:
        return lib().hb_selector_log(self.h).decode()

    def buckets(self) -> list[int]:
        arr = (C.c_uint32 * 64)()
        n = lib().hb_selector_buckets(self.h, arr, 64)
        return [arr[i] for i in range(n)]

    def inject_wrong(self, enable: bool = True) -> None:
        self.ctx._check(lib().hb_selector_inject_wrong(self.h, int(enable)))

    def gemm(self, k, n, out, w, x, y, m) -> Kernel:
        p = C.c_void_p()
        self.ctx._check(lib().hb_select_gemm(self.h, k, n, out, _as_range(w), _as_range(x), _as_range(y), m, C.byref(p)))
        return Kernel(self.ctx, p.value)

    def gate_up(self, k, inter, w, x, gu, h, m) -> list[Kernel]:
        ks = (C.c_void_p * 2)()
        n = C.c_int()
        self.ctx._check(lib().hb_select_gate_up(self.h, k, inter, _as_range(w), _as_range(x), _as_range(gu), _as_range(h), m, ks, C.byref(n)))
        return [Kernel(self.ctx, ks[i]) for i in range(n.value)]

    def matvec(self, k, n, out, rows, w_copies, x, y) -> Kernel:
        arr = (Range * len(w_copies))(*[_as_range(w) for w in w_copies])
        p = C.c_void_p()
        self.ctx._check(lib().hb_select_matvec(self.h, k, n, out, rows, arr, len(w_copies), _as_range(x), _as_range(y), C.byref(p)))
        return Kernel(self.ctx, p.value)

    def gemm_q4(self, k, n, out, wq, scales, w_bf16, x, y, m) -> list[Kernel]:
        """[fused] (bindings W, X, Y, scales) or [dequant, gemm] (bindings W, scales, w_bf16 and w_bf16, X, Y)."""
        ks = (C.c_void_p * 2)()
        nk = C.c_int()
        wb = _as_range(w_bf16) if w_bf16 is not None else Range(None, 0)
        self.ctx._check(lib().hb_select_gemm_q4(self.h, k, n, out, _as_range(wq), _as_range(scales), wb, _as_range(x), _as_range(y), m, ks, C.byref(nk)))
        return [Kernel(self.ctx, ks[i]) for i in range(nk.value)]

    def matvec_x(self, k, n, out, rows, x_src, norm_eps_bits, norm_plus_one, w_copies, x, y, norm_w=None) -> Kernel:
        """The form of a projection whose input is made inside the kernel (x_src X_NORM: x is the residual stream and
        norm_w the norm's weights; X_SWIGLU: x holds rows of [gate | up])."""
        arr = (Range * len(w_copies))(*[_as_range(w) for w in w_copies])
        p = C.c_void_p()
        nw = _as_range(norm_w) if norm_w is not None else Range(None, 0)
        self.ctx._check(lib().hb_select_matvec_x(self.h, k, n, out, rows, x_src, norm_eps_bits, norm_plus_one, arr, len(w_copies), _as_range(x), _as_range(y), nw, C.byref(p)))
        return Kernel(self.ctx, p.value)

    def axis(self, axis: str, key: str, variants, values, position: int = 0) -> int:
        """One axis of the decode step's load-time timing: `variants` are op lists [(kernel, m, bufs...), ...], one per
        value (None: that form is unavailable); returns the value to use."""
        made = [self.ctx.make_ops(v) if v else None for v in variants]
        arrs = (C.POINTER(Op) * len(variants))(*[C.cast(m_[0], C.POINTER(Op)) if m_ else None for m_ in made])
        nops = (C.c_int * len(variants))(*[len(v) if v else 0 for v in variants])
        vals = (C.c_uint32 * len(values))(*values)
        best = C.c_uint32()
        self.ctx._check(lib().hb_select_axis(self.h, axis.encode(), key.encode(), arrs, nops, vals, len(variants), position, C.byref(best)))
        return best.value

    def experts(self, experts, top_k, h, mi, m, route, lst, tiles, x, wgu, wdown, ehb, ey, egu=None, xs=None):
        """Returns dict(bm, sort, gather, gate_up, swiglu, down); gather and swiglu may be None."""
        none = Range(None, 0)
        io = ExpertIo(experts, top_k, h, mi, m, *[_as_range(b) if b is not None else none for b in (route, lst, tiles, x, wgu, wdown, ehb, ey, egu, xs)])
        pick = ExpertPick()
        self.ctx._check(lib().hb_select_experts(self.h, C.byref(io), C.byref(pick)))
        k = lambda h: Kernel(self.ctx, h) if h else None
        return dict(bm=pick.bm, sort=k(pick.sort), gather=k(pick.gather), gate_up=k(pick.gate_up), swiglu=k(pick.swiglu), down=k(pick.down))


def fill_random16(ctx: Context, buf, seed: int) -> None:
    ctx._check(lib().hb_fill_random16(ctx.h, _as_range(buf), seed))


def check_rule(reference: np.ndarray, got: np.ndarray):
    """check_candidates' rule on host arrays: (eligible, err, scale)."""
    f32_out = reference.dtype == np.float32
    e, err, scale = C.c_int(), C.c_float(), C.c_float()
    reference = np.ascontiguousarray(reference)
    got = np.ascontiguousarray(got)
    st = lib().hb_check_rule(reference.ctypes.data, got.ctypes.data, reference.size, int(f32_out), C.byref(e), C.byref(err), C.byref(scale))
    if st != OK:
        raise HbError(st, "hb_check_rule failed")
    return bool(e.value), err.value, scale.value
