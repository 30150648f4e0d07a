"""Benchmark of the bf16 matrix-multiply hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout. A step is one pass of the 9B-class layer GEMM set at M = 2048 rows
(the layer set: qkv 4096->6144, o_proj 4096->4096 + residual, fused gate/up 4096->2x12288 with
SiLU*mul, down 12288->4096 + residual) through the C ABI of libhb200.so, kernels chosen by the
load-time selection loop. `value` is TFLOP/s over all ranks with inputs resident in HBM, timed with
CUDA events on the launching stream; `e2e` is the same step with the block's activations copied in
from pinned host memory and the result copied back inside the timed region. The decode matvec
(config 2), the 27B-class tensor-parallel FFN (config 4) and the MoE block (config 5) are measured
beside it and reported under "extra". Inputs are seeded synthetic tensors of the reference's shapes
(no checkpoints exist here): X ~ N(0,1), W ~ N(0,1/sqrt(K)), bf16.

--impl reference times the CPU restatement of the same contract (oracle/, OpenMP on every host
core) on a bounded row sample of the same workload: the reference's own kernels exist only as
Metal shaders and cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, ROWS = 4096, 12288, 2048
# (name, K, N, out) of the layer's four projections; out: 0 Bf16, 2 Residual, 3 Swiglu
LAYER = [("qkv", HIDDEN, 6144, 0), ("o_proj", HIDDEN, HIDDEN, 2), ("gate_up", HIDDEN, 2 * INTER, 3), ("down", INTER, HIDDEN, 2)]
STEP_FLOP = sum(2.0 * ROWS * k * n for _, k, n, _ in LAYER)
METRIC = "bf16 prefill GEMM TFLOP/s/GPU"


def workload_config(n_gpus: int) -> dict:
    """The `config` object of the JSON line: the same for this library's arm and for the CPU arm."""
    return {"workload": "9B-class layer GEMM set, M=2048: qkv 4096->6144, o 4096->4096 +residual, gate/up 4096->2x12288 SiLU*mul, down 12288->4096 +residual",
            "rows": ROWS, "hidden": HIDDEN, "intermediate": INTER, "parallelism": f"replicas x{n_gpus}" if n_gpus > 1 else "1 GPU",
            "l2": "386 MB of weights per step: inputs larger than L2"}


def host_threads() -> int:
    """The host cores this process may use. A launcher that starts one process per GPU exports OMP_NUM_THREADS=1
    for all of them; the CPU arm runs on one rank alone and takes every core it is allowed."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            p.update({k: float(d[k]) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in d})
            p["source"] = "measured"
        except Exception:
            pass
    return p


class ClockSampler(threading.Thread):
    """SM clock and throttle reasons read through NVML while the timed loops run (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.active = threading.Event()
        self.stop = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # no NVML: the clocks key says so
            self.err = str(e)

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self.stop.is_set():
            if self.active.is_set():
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    try:
                        r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                    except Exception:
                        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(0.002)

    def summary(self):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + getattr(self, "err", "")}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def bind_near_gpu(index: int):
    """With several ranks on one host, every rank's page-locked buffers should live in the memory of the socket its GPU
    hangs on: eight ranks copying through one socket's memory share its bandwidth and the link between the sockets.
    Restricts this process to the CPUs NVML names as the GPU's own (a property of the process, not of the GPU), so
    that the buffers it allocates afterwards are placed there. Returns the number of CPUs, or None when NVML cannot say."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def run_reference(args):
    """The CPU arm: the contract restated in C (oracle/), all host threads, every row of the workload when the
    host gets through it in time (a row sample otherwise)."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = host_threads()
    os.environ["OMP_NUM_THREADS"] = str(threads)  # before the OpenMP runtime starts: the launcher may have set it to 1
    import ctypes

    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle

    o = Oracle(native=True)
    try:  # and for a runtime that had read the old value already
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(threads)
    except OSError:
        pass
    rng = np.random.default_rng(0)

    def bf16(a):
        b = a.astype(np.float32).view(np.uint32)
        return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)

    ws = [bf16(rng.standard_normal((n, k), dtype=np.float32) * k**-0.5) for _, k, n, _ in LAYER]

    def inputs(rows):
        return [bf16(rng.standard_normal((rows, k), dtype=np.float32)) for _, k, _, _ in LAYER], bf16(rng.standard_normal((rows, HIDDEN), dtype=np.float32))

    def step(xs, y0):
        for (name, k, n, out), w, x in zip(LAYER, ws, xs):
            o.gemm_f32(x, w, out, y0 if out == 2 else None)

    # all 2048 rows unless the run (steps + warm-up) would then take more than about four minutes on this host
    probe = inputs(64)
    step(*probe)
    t0 = time.perf_counter()
    step(*probe)
    per_row = (time.perf_counter() - t0) / 64
    rows = ROWS
    while rows > 64 and per_row * rows * (args.steps + args.warmup) > 240.0:
        rows //= 2
    xs, y0 = inputs(rows)
    for _ in range(args.warmup):
        step(xs, y0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(xs, y0)
    dt = (time.perf_counter() - t0) / args.steps
    flop = STEP_FLOP * rows / ROWS
    value = flop / dt / 1e12
    sample = f"{rows} of {ROWS} rows of every GEMM of the layer set (same K and N), f32 accumulate, one RNE"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args.gpus),
        "note": "the reference's kernels are Metal shaders and cannot run here; this is the CPU restatement of its contract (oracle/hb_oracle.c, OpenMP)",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": o.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# The one JSON line goes to the process's real stdout; everything else that writes to file descriptor 1 (NCCL prints its
# version banner there) is sent to stderr, so that stdout holds exactly the line.
_REAL_STDOUT = None


def emit(line: dict) -> None:
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--plain-launches", action="store_true", help="never launch the step's kernels overlapped")
    ap.add_argument("--no-extra", action="store_true", help="skip the matvec / MoE / tensor-parallel sections")
    ap.add_argument("--tune", default="", help="engine tune keys, e.g. gemm.auto=0 to skip the load-time timing")
    ap.add_argument("--form", default="", choices=["", "pair", "sk", "one"], help="with --case gate_up/down/layer: the GEMM form (one = one CTA per 128x256 tile)")
    ap.add_argument("--case", default="", choices=["", "layer", "gate_up", "down", "down512k2", "matvec", "matvec8", "matvec8fit", "moe", "q4", "q4m8", "q4gemm512"],
                    help="run one small case of one kernel a few times and exit (the command profiled under ncu)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if args.case:
        run_case(args)
        return

    import numpy as np
    import torch

    from __graft_entry__ import load_package

    hb = load_package()
    rank, world, local = dist_env()
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    numa = bind_near_gpu(local) if world > 1 else None  # before any page-locked buffer is made: first touch places it
    ctx = hb.Context(local)
    pk = peaks()
    sampler = ClockSampler(local)
    sampler.start()

    def wrap(t):
        return ctx.wrap(t.data_ptr(), t.numel() * t.element_size())

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(sec):
        if world == 1:
            return sec
        t = torch.tensor([sec], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- the layer GEMM set: weights and activations resident in HBM (386 MB of weights per step: larger than L2)
    g = torch.Generator(device=dev)
    g.manual_seed(0x9E3779B9 + rank)
    weights = [(torch.randn(n, k, device=dev, generator=g) * k**-0.5).bfloat16() for _, k, n, _ in LAYER]
    x = torch.randn(ROWS, HIDDEN, device=dev, generator=g).bfloat16()
    qkv = torch.zeros(ROWS, 6144, device=dev, dtype=torch.bfloat16)
    resid = torch.randn(ROWS, HIDDEN, device=dev, generator=g).bfloat16()
    hmid = torch.zeros(ROWS, INTER, device=dev, dtype=torch.bfloat16)
    gu_scratch = torch.zeros(ROWS, 2 * INTER, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()

    tune = hb.Tune(args.tune)
    sel = hb.Selector(ctx, tune)
    t_sel = time.perf_counter()
    k_qkv = sel.gemm(HIDDEN, 6144, 0, wrap(weights[0]), wrap(x), wrap(qkv), ROWS)
    k_o = sel.gemm(HIDDEN, HIDDEN, 2, wrap(weights[1]), wrap(x), wrap(resid), ROWS)
    k_gu = sel.gate_up(HIDDEN, INTER, wrap(weights[2]), wrap(x), wrap(gu_scratch), wrap(hmid), ROWS)
    k_down = sel.gemm(INTER, HIDDEN, 2, wrap(weights[3]), wrap(hmid), wrap(resid), ROWS)
    t_sel = time.perf_counter() - t_sel
    ops = [(k_qkv, ROWS, wrap(weights[0]), wrap(x), wrap(qkv)), (k_o, ROWS, wrap(weights[1]), wrap(x), wrap(resid))]
    if len(k_gu) == 2:
        ops += [(k_gu[0], ROWS, wrap(weights[2]), wrap(x), wrap(gu_scratch)), (k_gu[1], ROWS, wrap(gu_scratch), wrap(hmid))]
    else:
        ops += [(k_gu[0], ROWS, wrap(weights[2]), wrap(x), wrap(hmid))]
    ops += [(k_down, ROWS, wrap(weights[3]), wrap(hmid), wrap(resid))]
    picks = {"qkv": k_qkv.name, "o_proj": k_o.name, "gate_up": "+".join(k.name for k in k_gu), "down": k_down.name}

    # Overlapped launches (each GEMM requests its first weight stages under the tail of the one before and waits for it
    # inside): the same bits, checked here on one step from the same start; used for the timed region when faster.
    resid0 = resid.clone()
    outs_ = []
    for on in (False, True):
        resid.copy_(resid0)
        torch.cuda.synchronize()
        ctx.set_launch_overlap(on)
        ctx.run(ops)
        ctx.sync()
        outs_.append((resid.clone(), qkv.clone(), hmid.clone()))
    if not all(torch.equal(a_, b_) for a_, b_ in zip(*outs_)):
        raise RuntimeError("overlapped launches changed the step's result")
    del outs_
    t_launch = {}
    for on in (False, True):
        ctx.set_launch_overlap(on)
        ctx.time(ops, 3)
        t_launch["overlapped" if on else "plain"] = max_over_ranks(ctx.time(ops, 5)) / 5
    overlap = t_launch["overlapped"] < t_launch["plain"] and not args.plain_launches
    ctx.set_launch_overlap(overlap)
    resid.copy_(resid0)

    ctx.time(ops, args.warmup)
    barrier()
    sampler.active.set()
    launches0 = ctx.launch_count()
    sec = ctx.time(ops, args.steps)  # CUDA events on the launching stream around the K steps
    launches = ctx.launch_count() - launches0
    barrier()
    sec = max_over_ranks(sec)
    ms_per_step = sec / args.steps * 1e3
    value = STEP_FLOP * world / (sec / args.steps) / 1e12
    # the same loop for 200 steps: long enough for the power cap to set the clock (the figure the sustained peak bounds)
    long_steps = max(200, args.steps)
    barrier()
    sec_long = max_over_ranks(ctx.time(ops, long_steps))
    barrier()

    # ---- end to end: activations in from page-locked host memory, result back out, every step.
    # Serial: upload, kernels, download, one after the other. Streamed: the same three per step through the
    # library's copy lanes with two sets of device buffers, so the copies of one step run under the kernels
    # of its neighbours; the host reads step i's result before it enqueues step i + 2.
    x_host = torch.empty(ROWS, HIDDEN, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    y_host = torch.empty(ROWS, HIDDEN, dtype=torch.bfloat16).pin_memory()
    d_x, d_resid = wrap(x), wrap(resid)
    L = hb.lib()
    io_bytes = ROWS * HIDDEN * 2

    def serial_step():
        ctx._check(L.hb_upload(ctx.h, d_x.ptr, x_host.data_ptr(), io_bytes))
        ctx.run(ops)
        ctx._check(L.hb_download(ctx.h, y_host.data_ptr(), d_resid.ptr, io_bytes))

    for _ in range(3):
        serial_step()
    barrier()
    n_e2e = max(3, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        serial_step()
    torch.cuda.synchronize()
    serial_sec = max_over_ranks((time.perf_counter() - t0) / n_e2e)

    x2 = x.clone()
    resid2 = resid.clone()
    ops2 = [(k, m, *[wrap(x2) if r.ptr == d_x.ptr else wrap(resid2) if r.ptr == d_resid.ptr else r for r in rs]) for (k, m, *rs) in ops]
    xh = ctx.host_array((2, ROWS, HIDDEN))
    yh = ctx.host_array((2, ROWS, HIDDEN))
    xh[:] = x_host.view(torch.uint16).numpy()
    blocks = hb.StreamedBlocks(ctx, [(ops, d_x, d_resid), (ops2, wrap(x2), wrap(resid2))])
    n_str = max(4, args.steps)

    def streamed(n):
        for i in range(n):
            if i >= 2:
                blocks.wait(i - 2)  # the host has step i-2's result before its buffers are used again
            blocks.step(i, xh[i % 2], yh[i % 2])
        blocks.wait(n - 2)
        blocks.wait(n - 1)

    streamed(4)
    ctx.sync()
    barrier()
    t0 = time.perf_counter()
    streamed(n_str)
    str_sec = max_over_ranks((time.perf_counter() - t0) / n_str)
    ctx.sync()
    blocks.close()
    sampler.active.clear()
    barrier()
    e2e = {"value": STEP_FLOP * world / str_sec / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": io_bytes, "d2h_bytes_per_step": io_bytes,
           "ms_per_step": str_sec * 1e3, "steps": n_str, "mode": "streamed: copy lanes, 2 buffer sets, host reads every result",
           "cpus_near_gpu": numa,
           "serial": {"value": STEP_FLOP * world / serial_sec / 1e12, "ms_per_step": serial_sec * 1e3, "steps": n_e2e}}

    per_gpu_tflops = value / world
    roofline = {
        "bound": "tensor", "achieved": per_gpu_tflops, "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": per_gpu_tflops / pk["bf16_tflops"],
        "traffic": traffic_of(picks),
        "traffic_source": "ncu captures of these kernel forms summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum per launch), not measured in this run",
        "sustained": {"steps": long_steps, "ms_per_step": sec_long / long_steps * 1e3, "tflops_per_gpu": STEP_FLOP / (sec_long / long_steps) / 1e12,
                      "frac_of_sustained_peak": STEP_FLOP / (sec_long / long_steps) / 1e12 / pk["bf16_tflops_sustained"],
                      "frac_of_burst_peak": STEP_FLOP / (sec_long / long_steps) / 1e12 / pk["bf16_tflops"]},
        "kernel": "gemm_bf16_tn_pair_kernel" if all(v.startswith("gemm_pair_") for v in picks.values()) else "gemm_bf16_tn_kernel / gemm_bf16_tn_pair_kernel", "peak_source": pk["source"] + " (burst cuBLAS bf16)",
        "frac_of_sustained_peak": per_gpu_tflops / pk["bf16_tflops_sustained"], "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
        "algorithmic_flop_per_launch": STEP_FLOP / 4, "launches_per_step": len(ops),
        # operands once: 2(MK + NK + M N_out) bytes, plus the residual read where there is one, averaged over the four
        "algorithmic_bytes_per_launch": sum(2.0 * (ROWS * k + n * k + ROWS * (n // 2 if o == 3 else n) * (2 if o == 2 else 1)) for _, k, n, o in LAYER) / 4,
    }

    ctx.set_launch_overlap(False)  # (the sections below set it themselves where they use it)
    roofline["launches"] = {"mode": "overlapped" if overlap else "plain", "us_per_step": {k_: v * 1e6 for k_, v in t_launch.items()}}
    extra = {"selection_seconds": t_sel, "picks": picks}
    if not args.no_extra:
        try:
            # the same layer set at the other block sizes of config 3 (64 and 512 rows), kernels picked per size
            small = {}
            for rows_s in (64, 512):
                xs_ = x[:rows_s].contiguous()
                qkv_, res_, hm_, gu_ = qkv[:rows_s], resid[:rows_s].clone(), hmid[:rows_s], gu_scratch[:rows_s]
                ks = [sel.gemm(HIDDEN, 6144, 0, wrap(weights[0]), wrap(xs_), wrap(qkv_), rows_s), sel.gemm(HIDDEN, HIDDEN, 2, wrap(weights[1]), wrap(xs_), wrap(res_), rows_s)]
                kg = sel.gate_up(HIDDEN, INTER, wrap(weights[2]), wrap(xs_), wrap(gu_), wrap(hm_), rows_s)
                kd = sel.gemm(INTER, HIDDEN, 2, wrap(weights[3]), wrap(hm_), wrap(res_), rows_s)
                ops_s = [(ks[0], rows_s, wrap(weights[0]), wrap(xs_), wrap(qkv_)), (ks[1], rows_s, wrap(weights[1]), wrap(xs_), wrap(res_))]
                ops_s += [(kg[0], rows_s, wrap(weights[2]), wrap(xs_), wrap(gu_)), (kg[1], rows_s, wrap(gu_), wrap(hm_))] if len(kg) == 2 else [(kg[0], rows_s, wrap(weights[2]), wrap(xs_), wrap(hm_))]
                ops_s += [(kd, rows_s, wrap(weights[3]), wrap(hm_), wrap(res_))]
                modes_s = {}
                for on in (False, True):  # plain launches, then overlapped ones (the kernels that can wait for their predecessor themselves do)
                    ctx.set_launch_overlap(on)
                    ctx.time(ops_s, 5)
                    barrier()
                    modes_s["overlapped" if on else "plain"] = max_over_ranks(ctx.time(ops_s, 50) / 50)
                ctx.set_launch_overlap(False)
                sec_s = min(modes_s.values())
                flop_s = STEP_FLOP * rows_s / ROWS
                wbytes_s = sum(2.0 * n * k for _, k, n, _ in LAYER)
                small[f"M{rows_s}"] = {"us": sec_s * 1e6, "tflops": flop_s / sec_s / 1e12, "weight_gbs": wbytes_s / sec_s / 1e9,
                                       "frac_hbm_weights": wbytes_s / sec_s / 1e9 / pk["hbm_gbs"], "frac_bf16_peak": flop_s / sec_s / 1e12 / pk["bf16_tflops"],
                                       "picks": [o[0].name for o in ops_s], "launches_us": {k_: v * 1e6 for k_, v in modes_s.items()}}
            extra["layer_set_small_blocks"] = small
        except Exception as e:
            extra["small_error"] = repr(e)
        try:
            extra.update(bench_extra(hb, ctx, sel, torch, dev, wrap, pk, rank, world, barrier, max_over_ranks))
        except Exception as e:  # the headline stands on its own
            extra["error"] = repr(e)
        try:
            extra.update(bench_sharded(hb, ctx, torch, dev, pk, rank, world, barrier, max_over_ranks))
        except Exception as e:
            extra["sharded_error"] = repr(e)

    # the other half of the metric (the decode matvec against the HBM roofline) and the sharded configurations, in the
    # object of the line that records them
    roofline.update(summaries(extra, pk))

    cpu = None
    if rank == 0 and world == 1:
        cpu = cpu_baseline()

    sampler.stop.set()
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world),
            "e2e": e2e, "gpu_launches": launches, "clocks": sampler.summary(), "roofline": roofline, "cpu_baseline": cpu, "extra": extra,
        }
        emit(line)
    sel.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def summaries(extra: dict, pk: dict) -> dict:
    """What the sections beside the headline measured, in short: the decode matvec (HBM-bound: us, GB/s of algorithmic
    bytes, fraction of the measured copy bandwidth, picked form), the short prefill blocks, the decode layer chain, the
    MoE block, and the two sharded configurations with their parity against the f64 product."""
    out = {}
    mv = {}
    for key, n in (("matvec_4096x12288", 12288), ("matvec_4096x151936", 151936)):
        for mk, v in (extra.get(key) or {}).items():
            mv[f"n{n}_{mk}"] = {"us": v["us"], "gbs": v["gbs"], "frac": v["frac_hbm"], "form": v["form"]}
    if mv:
        out["matvec"] = dict(mv, bound="hbm", peak=pk["hbm_gbs"], unit="GB/s", k=4096, bytes="2(NK + MK + MN) per launch")
    small = extra.get("layer_set_small_blocks")
    if small:
        out["short_blocks"] = {k_: {"us": v["us"], "tflops": v["tflops"], "frac_bf16_peak": v["frac_bf16_peak"], "frac_hbm_weights": v["frac_hbm_weights"]} for k_, v in small.items()}
    dec = extra.get("decode_layer_9b")
    if dec:
        out["decode_layer_9b"] = {k_: {"us_per_layer": v["us_per_layer"], "frac_hbm": v["frac_hbm"], "kernels_per_layer": v["kernels_per_layer"], "dec.fnorm": v.get("dec.fnorm"), "dec.fswi": v.get("dec.fswi"),
                                        "variants_us": {n_: min(t_.values()) for n_, t_ in (v.get("variants_us") or {}).items()}} for k_, v in dec.items()}
    moe = extra.get("moe_2048tok_256e_top8")
    if moe:
        out["moe_block"] = {"us": moe["us"], "weight_gbs": moe["weight_gbs"], "frac_hbm": moe["frac_hbm"], "kernels": len(moe["us_per_kernel"])}
    q4 = extra.get("matvec_q4_4096")
    if q4:
        out["matvec_q4"] = {k_: {"us": v["us"], "frac_hbm": v["frac_hbm"]} for k_, v in q4.items()}
    if extra.get("gemm_q4_gate_up_4096x24576"):
        out["gemm_q4"] = extra["gemm_q4_gate_up_4096x24576"]
    sh = {}
    for key, name in (("tp_ffn_27b_m2048", "tp_ffn_27b"), ("moe_ep_2048tok", "moe_ep")):
        v = extra.get(key)
        if v:
            sh[name] = {k_: v.get(k_) for k_ in ("n_gpus", "us", "t1_us", "efficiency", "kernels_per_step", "kernels_us", "forms_us", "nccl_form_us", "parity") if k_ in v}
    weak = extra.get("moe_ep_weak_2048tok_per_gpu")
    if weak:
        sh["moe_ep_weak"] = {"n_gpus": weak["n_gpus"], "us": weak["us"], "tokens_per_s_total": weak["tokens_per_s_total"]}
    if sh:
        out["sharded"] = dict(sh, scaling="strong: global M = 2048 rows; efficiency = t1 / (n_gpus * us), t1 the same code on one GPU in the same job")
    for k_ in ("error", "sharded_error", "small_error"):
        if k_ in extra:
            out[k_] = extra[k_]
    return out


def run_case(args):
    """One kernel on one case, a handful of launches, a few hundred MB to 1.3 GB on the device (operands larger
    than L2): the command an ncu capture runs. Prints the case's CUDA-event time."""
    import torch

    from __graft_entry__ import load_package

    hb = load_package()
    dev = torch.device("cuda", 0)
    ctx = hb.Context(0)
    g = torch.Generator(device=dev)
    g.manual_seed(7)

    def wrap(t):
        return ctx.wrap(t.data_ptr(), t.numel() * t.element_size())

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).bfloat16()

    reps = 5
    if args.case in ("gate_up", "down"):
        k, n, out = (HIDDEN, 2 * INTER, 3) if args.case == "gate_up" else (INTER, HIDDEN, 2)
        w, x = rnd(n, k, scale=k**-0.5), rnd(ROWS, k)
        y = rnd(ROWS, n // 2 if out == 3 else n)
        torch.cuda.synchronize()
        form = {"": {}, "one": {}, "pair": {"cta_pair": 1}, "sk": {"stream_k": 1}}[args.form]
        kern = ctx.gemm(k, n, out, rows_max=ROWS, **form)
        ops = [(kern, ROWS, wrap(w), wrap(x), wrap(y))]
        work = {"flop": 2.0 * ROWS * k * n}
    elif args.case == "layer":
        # the bench's step in its picked forms: the four GEMMs of one layer on the CTA-pair kernel
        ws = [rnd(n, k, scale=k**-0.5) for _, k, n, _ in LAYER]
        x, hmid = rnd(ROWS, HIDDEN), rnd(ROWS, INTER)
        qkv, resid = rnd(ROWS, 6144), rnd(ROWS, HIDDEN)
        torch.cuda.synchronize()
        form = {"": {"cta_pair": 1}, "pair": {"cta_pair": 1}, "sk": {"stream_k": 1}, "one": {}}[args.form]
        ks = [ctx.gemm(k, n, out, rows_max=ROWS, **form) for _, k, n, out in LAYER]
        ops = [(ks[0], ROWS, wrap(ws[0]), wrap(x), wrap(qkv)), (ks[1], ROWS, wrap(ws[1]), wrap(x), wrap(resid)),
               (ks[2], ROWS, wrap(ws[2]), wrap(x), wrap(hmid)), (ks[3], ROWS, wrap(ws[3]), wrap(hmid), wrap(resid))]
        work = {"flop": STEP_FLOP}
    elif args.case in ("q4", "q4m8"):
        # the one-row product from Q4_0 weights at the LM-head shape (350 MB of nibbles and scales); q4m8: eight rows
        k, n = 4096, 151936
        blocks = n * k // 32
        wq = torch.randint(0, 256, (blocks * 16,), device=dev, dtype=torch.uint8, generator=g)
        sq = (torch.rand(blocks, device=dev, generator=g) * 0.01 + 0.001).half()
        mq = 8 if args.case == "q4m8" else 1
        x, y = rnd(mq, k), torch.zeros(mq, n, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        kq = ctx.matmul_q4(k, n, mq) if mq > 1 else ctx.matvec_q4(k, n, 0, 2)
        ops = [(kq, mq, wrap(wq), wrap(x), wrap(y), wrap(sq))]
        work = {"bytes": blocks * 18.0 + mq * (2.0 * k + 2.0 * n)}
    elif args.case == "down512k2":
        # a short prefill block on the CTA-pair kernel with K cut in two: 512 rows of the down projection
        k, n, rows = INTER, HIDDEN, 512
        w, x, y = rnd(n, k, scale=k**-0.5), rnd(rows, k), rnd(rows, n)
        torch.cuda.synchronize()
        ops = [(ctx.gemm(k, n, 2, rows_max=rows, cta_pair=1, split_k=2), rows, wrap(w), wrap(x), wrap(y))]
        work = {"flop": 2.0 * rows * k * n}
    elif args.case == "q4gemm512":
        # the prefill GEMM from Q4_0 weights that decodes while it stages: 512 rows of gate/up (56.6 MB of nibbles and scales)
        k, n, rows = HIDDEN, 2 * INTER, 512
        blocks = n * k // 32
        wq = torch.randint(0, 256, (blocks * 16,), device=dev, dtype=torch.uint8, generator=g)
        sq = (torch.rand(blocks, device=dev, generator=g) * 0.01 + 0.001).half()
        x, y = rnd(rows, k), torch.zeros(rows, n, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        ops = [(ctx.gemm_q4(k, n, 0, tile_n=256, rows_max=rows), rows, wrap(wq), wrap(x), wrap(y), wrap(sq))]
        work = {"flop": 2.0 * rows * k * n}
    elif args.case in ("matvec", "matvec8", "matvec8fit"):
        m = 1 if args.case == "matvec" else 8
        k, n = 4096, 151936
        w, x = rnd(n, k, scale=k**-0.5), rnd(8, k)
        y = torch.zeros(8, n, device=dev, dtype=torch.bfloat16)
        torch.cuda.synchronize()
        # one row: a warp per two weight rows on the CUDA cores; eight rows: the weight stream on the tensor cores
        kern = (ctx.matvec(k, n, 0, rows_max=m, rows_per_warp=2, split=2) if m == 1 else
                ctx.matvec(k, n, 0, rows_max=m, tensor_core=3 if args.case == "matvec8fit" else 1, split=4))
        ops = [(kern, m, wrap(w), wrap(x), wrap(y))]
        work = {"bytes": 2.0 * (n * k + m * k + m * n)}
    else:
        m, h, mi, E, top_k, bm = 2048, 2048, 512, 256, 8, 64
        pairs = m * top_k
        x, wgu, wd = rnd(m, h), rnd(E * 2 * mi, h, scale=h**-0.5), rnd(E * h, mi, scale=mi**-0.5)
        scores = rnd(m, E)
        route = torch.zeros(m, 2 * top_k, device=dev, dtype=torch.int32)
        lst = torch.zeros(pairs, device=dev, dtype=torch.int32)
        tiles = torch.zeros(1 + 3 * hb.lib().hb_moe_tiles(m, top_k, E, bm), device=dev, dtype=torch.int32)
        ehb, ey, out = rnd(pairs, mi), rnd(pairs, h), rnd(m, h)
        torch.cuda.synchronize()
        kw = dict(rows_max=m, top_k=top_k, experts=E, bm=bm)
        ops = [(ctx.route(E, top_k), m, wrap(scores), wrap(route)), (ctx.moe_sort(E, top_k, m, bm), m, wrap(route), wrap(lst), wrap(tiles)),
               (ctx.gemm(h, 2 * mi, 3, rows_mode=hb.ROWS_GATHER, merge_runs=1, **kw), m, wrap(wgu), wrap(x), wrap(ehb), wrap(lst), wrap(tiles)),
               (ctx.gemm(mi, h, 0, rows_mode=hb.ROWS_SCATTER, merge_runs=1, **kw), m, wrap(wd), wrap(ehb), wrap(ey), wrap(lst), wrap(tiles)),
               (ctx.moe_combine(h, top_k), m, wrap(ey), wrap(route), wrap(out))]
        work = {"bytes": 2.0 * E * 3 * mi * h}
    ctx.time(ops, 2)
    sec = ctx.time(ops, reps) / reps
    line = {"case": args.case, "kernels": [o[0].name for o in ops], "us": sec * 1e6}
    if "flop" in work:
        line["tflops"] = work["flop"] / sec / 1e12
    else:
        line["gbs"] = work["bytes"] / sec / 1e9
    emit(line)
    ctx.close()


# dram__bytes_read.sum + dram__bytes_write.sum per launch (MB) of each projection of the step, from the ncu captures
# summarised in profiles/: the CTA-pair kernel and the one-CTA 128x256 kernel. `roofline.traffic` is the mean over the
# four launches of the forms the selection picked (None when a pick has no capture).
TRAFFIC_MB = {"gemm_pair": {"qkv": 72.3, "o_proj": 70.0, "gate_up": 257.8, "down": 236.4},
              "gemm_tc_t128x256": {"qkv": 71.8, "o_proj": 67.5, "gate_up": 252.1, "down": 232.4}}


def traffic_of(picks):
    total = 0.0
    for name, kernel in picks.items():
        form = "gemm_pair" if kernel.startswith("gemm_pair_") else "gemm_tc_t128x256" if kernel.startswith("gemm_tc_") and "_t128x256_" in kernel else None
        if form is None or name not in TRAFFIC_MB[form]:
            return None
        total += TRAFFIC_MB[form][name]
    return total / len(picks) * 1e6


def bench_extra(hb, ctx, sel, torch, dev, wrap, pk, rank, world, barrier, max_over_ranks):
    """Decode matvec (config 2) and the MoE block (config 5) on every rank's own GPU."""
    out = {}
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    # -- the small dense GEMM the CPU restatement runs whole: M=512, K=1024, N=4096 (4.3 GFLOP: 64 tiles of 128x256, a launch-bound case)
    try:
        w1 = (torch.randn(4096, 1024, device=dev, generator=g) / 32.0).bfloat16()
        x1 = torch.randn(512, 1024, device=dev, generator=g).bfloat16()
        y1 = torch.zeros(512, 4096, device=dev, dtype=torch.bfloat16)
        k1 = sel.gemm(1024, 4096, 0, wrap(w1), wrap(x1), wrap(y1), 512)
        gr = ctx.record([(k1, 512, wrap(w1), wrap(x1), wrap(y1))] * 8)
        gr.time(3)
        barrier()
        sec1 = max_over_ranks(gr.time(20) / (20 * 8))
        gr.free()
        out["config1_gemm_512x1024x4096"] = {"us": sec1 * 1e6, "tflops": 2.0 * 512 * 1024 * 4096 / sec1 / 1e12, "form": k1.name}
    except Exception as e:
        out["config1_error"] = repr(e)
    # -- matvec: K=4096, N=12288, M in {1,4,8}; four weight copies walked in turn so that W streams from HBM
    k, n = 4096, 12288
    copies = [(torch.randn(n, k, device=dev, generator=g) * k**-0.5).bfloat16() for _ in range(4)]
    xs = torch.randn(8, k, device=dev, generator=g).bfloat16()
    y = torch.zeros(8, n, device=dev, dtype=torch.bfloat16)
    mv = {}
    for m in (1, 4, 8):
        kern = sel.matvec(k, n, 0, m, [wrap(c) for c in copies], wrap(xs), wrap(y))
        ops = [(kern, m, wrap(c), wrap(xs), wrap(y)) for c in copies]
        # replayed as one recorded sequence, as a decode step is: a 20 us kernel enqueued one call at a time would
        # be timed at the host's launch rate; once with plain launches, once with each kernel launched ahead of its
        # predecessor's end (it waits inside before it touches an activation or an output)
        secs = {}
        for mode in ("plain", "overlapped"):
            ctx.set_launch_overlap(mode == "overlapped")
            gr = ctx.record(ops)
            gr.time(5)
            barrier()
            secs[mode] = max_over_ranks(gr.time(50) / (50 * len(copies)))
            gr.free()
        ctx.set_launch_overlap(False)
        sec = min(secs.values())
        bytes_ = 2.0 * (n * k + m * k + m * n)
        mv[f"m{m}"] = {"us": sec * 1e6, "gbs": bytes_ / sec / 1e9, "frac_hbm": bytes_ / sec / 1e9 / pk["hbm_gbs"], "form": kern.name,
                       "us_plain_launches": secs["plain"] * 1e6, "us_overlapped_launches": secs["overlapped"] * 1e6}
    out["matvec_4096x12288"] = mv
    del copies
    # the LM-head-like matrix is larger than L2 on its own
    n2 = 151936
    w2 = (torch.randn(n2, k, device=dev, generator=g) * k**-0.5).bfloat16()
    y2 = torch.zeros(8, n2, device=dev, dtype=torch.bfloat16)
    mv2 = {}
    for m in (1, 4, 8):
        kern = sel.matvec(k, n2, 0, m, [wrap(w2)], wrap(xs), wrap(y2))
        ops = [(kern, m, wrap(w2), wrap(xs), wrap(y2))]
        ctx.time(ops, 3)
        barrier()
        sec = max_over_ranks(ctx.time(ops, 20) / 20)
        bytes_ = 2.0 * (n2 * k + m * k + m * n2)
        mv2[f"m{m}"] = {"us": sec * 1e6, "gbs": bytes_ / sec / 1e9, "frac_hbm": bytes_ / sec / 1e9 / pk["hbm_gbs"], "form": kern.name}
    out["matvec_4096x151936"] = mv2
    # the same product from Q4_0 weights (4.5 bits per weight: 16 bytes of nibbles and an f16 scale per 32 weights; any
    # bytes are valid nibbles, so the synthetic weights are random bytes and small random scales)
    try:
        q4 = {}
        for nq in (12288, n2):
            blocks = nq * k // 32
            copies_q = 6 if nq == 12288 else 1
            wq = [torch.randint(0, 256, (blocks * 16,), device=dev, dtype=torch.uint8, generator=g) for _ in range(copies_q)]
            sq = (torch.rand(blocks, device=dev, generator=g) * 0.01 + 0.001).half()
            yq = torch.zeros(nq, device=dev, dtype=torch.bfloat16)
            best = None
            for rows, masks in ((1, 0), (2, 0), (4, 0), (2, 1), (4, 1)):
                kq = ctx.matvec_q4(k, nq, 0, rows, masks)
                ops_q = [(kq, 1, wrap(w_), wrap(xs), wrap(yq), wrap(sq)) for w_ in wq]
                gr = ctx.record(ops_q)
                gr.time(3)
                barrier()
                sec_q = max_over_ranks(gr.time(20) / (20 * copies_q))
                gr.free()
                if best is None or sec_q < best[0]:
                    best = (sec_q, kq.name)
            qbytes = blocks * 18.0 + 2.0 * k + 2.0 * nq
            q4[f"n{nq}"] = {"us": best[0] * 1e6, "gbs": qbytes / best[0] / 1e9, "frac_hbm": qbytes / best[0] / 1e9 / pk["hbm_gbs"], "form": best[1],
                            "bf16_equivalent_gbs": 2.0 * nq * k / best[0] / 1e9}
            # the rows of a short block at once (matmul_q4): each block of weights decoded once for all of them
            for mq in (2, 4, 8):
                xq = torch.randn(mq, k, device=dev, generator=g).bfloat16()
                ymq = torch.zeros(mq, nq, device=dev, dtype=torch.bfloat16)
                kq = ctx.matmul_q4(k, nq, mq)
                gr = ctx.record([(kq, mq, wrap(w_), wrap(xq), wrap(ymq), wrap(sq)) for w_ in wq])
                gr.time(3)
                barrier()
                sec_q = max_over_ranks(gr.time(20) / (20 * copies_q))
                gr.free()
                q4[f"n{nq}"][f"m{mq}_us"] = sec_q * 1e6
            del wq, sq
        out["matvec_q4_4096"] = q4
    except Exception as e:
        out["q4_error"] = repr(e)
    # the prefill GEMM from Q4_0 weights: dequant_q4 into a bf16 copy + the bf16 GEMM, against the GEMM that decodes
    # while it stages (q4.fuse), at the gate/up shape of the layer, 2048 and 512 rows
    try:
        kq_, nq_ = HIDDEN, 2 * INTER
        blocks = nq_ * kq_ // 32
        wq_ = torch.randint(0, 256, (blocks * 16,), device=dev, dtype=torch.uint8, generator=g)
        sq_ = (torch.rand(blocks, device=dev, generator=g) * 0.01 + 0.001).half()
        wb_ = torch.zeros(nq_, kq_, device=dev, dtype=torch.bfloat16)
        gus_ = torch.zeros(2048, nq_, device=dev, dtype=torch.bfloat16)
        q4g = {}
        for rows_q in (2048, 512, 128):
            xq_ = torch.randn(rows_q, kq_, device=dev, generator=g).bfloat16()
            hq_ = torch.zeros(rows_q, INTER, device=dev, dtype=torch.bfloat16)
            k_dq = ctx.dequant_q4(kq_, nq_)
            k_dq(1, wrap(wq_), wrap(sq_), wrap(wb_))
            k_bf = sel.gate_up(kq_, INTER, wrap(wb_), wrap(xq_), wrap(gus_[:rows_q]), wrap(hq_), rows_q)
            apart = [(k_dq, 1, wrap(wq_), wrap(sq_), wrap(wb_))]
            apart += [(k_bf[0], rows_q, wrap(wb_), wrap(xq_), wrap(gus_[:rows_q])), (k_bf[1], rows_q, wrap(gus_[:rows_q]), wrap(hq_))] if len(k_bf) == 2 else [(k_bf[0], rows_q, wrap(wb_), wrap(xq_), wrap(hq_))]
            res_q = {}
            for name, ops_q in [("dequant+gemm", apart)] + [(f"fused128x{tn}", [(ctx.gemm_q4(kq_, nq_, 3, tile_n=tn, rows_max=rows_q), rows_q, wrap(wq_), wrap(xq_), wrap(hq_), wrap(sq_))]) for tn in (256, 128)]:
                ctx.time(ops_q, 3)
                barrier()
                res_q[name] = max_over_ranks(ctx.time(ops_q, 10) / 10) * 1e6
            best = min(res_q, key=res_q.get)
            q4g[f"M{rows_q}"] = {"us": res_q, "picked": best, "tflops": 2.0 * rows_q * kq_ * nq_ / (res_q[best] * 1e-6) / 1e12,
                                 "dequant_alone_us": ctx.time(apart[:1], 10) / 10 * 1e6}
        out["gemm_q4_gate_up_4096x24576"] = q4g
        del wq_, sq_, wb_, gus_
    except Exception as e:
        out["q4_gemm_error"] = repr(e)
    # the LM head with the greedy pick: projection + argmax as two kernels, and the projection that folds the argmax in
    idx = torch.zeros(8, device=dev, dtype=torch.int32)
    form = dict(rows_per_warp=2, split=2)
    apart = [(ctx.matvec(k, n2, 0, rows_max=1, **form), 1, wrap(w2), wrap(xs), wrap(y2)), (ctx.argmax(n2, rows_max=1), 1, wrap(y2), wrap(idx))]
    fused = [(ctx.matvec(k, n2, 0, rows_max=1, argmax=1, **form), 1, wrap(w2), wrap(xs), wrap(y2), wrap(idx))]
    lm = {}
    for name, ops in (("apart", apart), ("fused", fused)):
        gr = ctx.record(ops)
        gr.time(3)
        barrier()
        lm[name + "_us"] = max_over_ranks(gr.time(20) / 20) * 1e6
        gr.free()
    lm["fused_form"] = fused[0][0].name
    out["lm_head_argmax_m1"] = lm
    del w2, y2
    # -- the matrix products of one 9B-class layer at decode time (1, 4 and 8 rows), with the norms before them, as one
    # recorded sequence over four layers' worth of weights (1.5 GB: every byte streams from HBM). The forms are chosen
    # as the engine chooses them at load: every projection's form by hb_select_matvec(_x), then the step's axes
    # (the norms apart or inside the projections: dec.fnorm; the SwiGLU in gate/up's epilogue or in down's input:
    # dec.fswi) on the whole chain by hb_select_axis.
    try:
        import struct

        layers = 4
        eps_bits = struct.unpack("<I", struct.pack("<f", 1e-6))[0]
        wl = [[(torch.randn(nn, kk, device=dev, generator=g) * kk**-0.5).bfloat16() for _, kk, nn, _ in LAYER] for _ in range(layers)]
        nw = (torch.randn(HIDDEN, device=dev, generator=g) * 0.1).bfloat16()
        dec = {}
        for m in (1, 4, 8):
            xd = torch.randn(m, HIDDEN, device=dev, generator=g).bfloat16()
            attn = torch.randn(m, HIDDEN, device=dev, generator=g).bfloat16()  # stands for the attention's output, the o projection's input
            xn = torch.zeros_like(xd)
            qkvd = torch.zeros(m, 6144, device=dev, dtype=torch.bfloat16)
            hd = torch.zeros(m, INTER, device=dev, dtype=torch.bfloat16)
            gud = torch.zeros(m, 2 * INTER, device=dev, dtype=torch.bfloat16)
            copies = lambda i: [wrap(wl[l][i]) for l in range(layers)]
            k_q = sel.matvec(HIDDEN, 6144, 0, m, copies(0), wrap(xn), wrap(qkvd))
            k_o = sel.matvec(HIDDEN, HIDDEN, 2, m, copies(1), wrap(attn), wrap(xd))
            k_g = sel.matvec(HIDDEN, 2 * INTER, 3, m, copies(2), wrap(xn), wrap(hd))
            k_d = sel.matvec(INTER, HIDDEN, 2, m, copies(3), wrap(hd), wrap(xd))
            k_n = ctx.rmsnorm(HIDDEN, 1e-6, True)
            k_qf = sel.matvec_x(HIDDEN, 6144, 0, m, hb.X_NORM, eps_bits, 1, copies(0), wrap(xd), wrap(qkvd), wrap(nw))
            k_gf = sel.matvec_x(HIDDEN, 2 * INTER, 3, m, hb.X_NORM, eps_bits, 1, copies(2), wrap(xd), wrap(hd), wrap(nw))

            def chain_ops(fnorm, fswi=0, kq=None, ko=None, kg=None, kd=None):
                ops_c = []
                for l in range(layers):
                    if fnorm:
                        ops_c += [(kq or k_qf, m, wrap(wl[l][0]), wrap(xd), wrap(qkvd), wrap(nw)), (ko or k_o, m, wrap(wl[l][1]), wrap(attn), wrap(xd))]
                    else:
                        ops_c += [(k_n, m, wrap(xd), wrap(nw), wrap(xn)), (kq or k_q, m, wrap(wl[l][0]), wrap(xn), wrap(qkvd)), (ko or k_o, m, wrap(wl[l][1]), wrap(attn), wrap(xd))]
                    if fswi:  # gate/up writes [gate | up], down makes the SwiGLU where it loads its input
                        gsrc = [(k_gpf, m, wrap(wl[l][2]), wrap(xd), wrap(gud), wrap(nw))] if fnorm else [(k_n, m, wrap(xd), wrap(nw), wrap(xn)), (k_gp, m, wrap(wl[l][2]), wrap(xn), wrap(gud))]
                        ops_c += gsrc + [(k_ds, m, wrap(wl[l][3]), wrap(gud), wrap(xd))]
                    elif fnorm:
                        ops_c += [(kg or k_gf, m, wrap(wl[l][2]), wrap(xd), wrap(hd), wrap(nw)), (kd or k_d, m, wrap(wl[l][3]), wrap(hd), wrap(xd))]
                    else:
                        ops_c += [(k_n, m, wrap(xd), wrap(nw), wrap(xn)), (kg or k_g, m, wrap(wl[l][2]), wrap(xn), wrap(hd)), (kd or k_d, m, wrap(wl[l][3]), wrap(hd), wrap(xd))]
                return ops_c

            def replay(ops_c):
                res = {}
                for mode in ("plain", "overlapped"):  # overlapped: each kernel is launched ahead of its predecessor's end and waits inside
                    ctx.set_launch_overlap(mode == "overlapped")
                    gr = ctx.record(ops_c)
                    gr.time(3)
                    barrier()
                    res[mode] = max_over_ranks(gr.time(20) / (20 * layers))
                    gr.free()
                ctx.set_launch_overlap(False)
                return res

            ctx.set_launch_overlap(True)  # the axes are timed as the step will run
            fnorm = sel.axis("fnorm", "dec.fnorm", [chain_ops(0), chain_ops(1)], [0, 1], position=0)
            fswi, k_gp = 0, None
            try:  # the SwiGLU made by the down projection: a CUDA-core form, its rows must fit in shared memory
                k_ds = sel.matvec_x(INTER, HIDDEN, 2, m, hb.X_SWIGLU, 0, 0, copies(3), wrap(gud), wrap(xd))
                k_gp = sel.matvec(HIDDEN, 2 * INTER, 0, m, copies(2), wrap(xn), wrap(gud))
                k_gpf = sel.matvec_x(HIDDEN, 2 * INTER, 0, m, hb.X_NORM, eps_bits, 1, copies(2), wrap(xd), wrap(gud), wrap(nw))
                fswi = sel.axis("fswi", "dec.fswi", [chain_ops(fnorm, 0), chain_ops(fnorm, 1)], [0, 1], position=0)
            except hb.HbError:
                pass
            ctx.set_launch_overlap(False)
            variants = {"norms apart": replay(chain_ops(0)), "norms inside the projections": replay(chain_ops(1))}
            if k_gp is not None:
                variants["SwiGLU inside down"] = replay(chain_ops(fnorm, 1))
            picked_ops = chain_ops(fnorm, fswi)
            secs = replay(picked_ops)
            forms = sorted({o[0].name for o in picked_ops})
            # for several rows also the chain of evenly dealt tensor-core streams, whose start-up hides under the kernel
            # before them once launches overlap (each projection's pick above was timed alone)
            alt = None
            if m > 1:
                ka = [ctx.matvec(kk, nn, oo, rows_max=m, tensor_core=2, split=2) for _, kk, nn, oo in LAYER]
                kaf = [ctx.matvec(kk, nn, oo, rows_max=m, tensor_core=2, split=2, x_src=hb.X_NORM, norm_eps_bits=eps_bits, norm_plus_one=1) for _, kk, nn, oo in (LAYER[0], LAYER[2])]
                alt_ops = chain_ops(fnorm, 0, kaf[0] if fnorm else ka[0], ka[1], kaf[1] if fnorm else ka[2], ka[3])
                alt = replay(alt_ops)
                if min(alt.values()) < min(secs.values()):
                    forms = sorted({o[0].name for o in alt_ops})
                    picked_ops = alt_ops
            sec_d = min(list(secs.values()) + (list(alt.values()) if alt else []))
            wb = sum(2.0 * nn * kk for _, kk, nn, _ in LAYER)
            dec[f"m{m}"] = {"us_per_layer": sec_d * 1e6, "weight_gbs": wb / sec_d / 1e9, "frac_hbm": wb / sec_d / 1e9 / pk["hbm_gbs"], "kernels_per_layer": len(picked_ops) // layers,
                            "dec.fnorm": fnorm, "dec.fswi": fswi, "selected_forms_us": {k_: v * 1e6 for k_, v in secs.items()},
                            "variants_us": {k_: {kk_: vv * 1e6 for kk_, vv in v.items()} for k_, v in variants.items()},
                            "balanced_stream_forms_us": {k_: v * 1e6 for k_, v in alt.items()} if alt else None, "forms": forms}
        out["decode_layer_9b"] = dec
        del wl
    except Exception as e:
        out["decode_error"] = repr(e)
    # -- MoE block (config 5): 2048 tokens, hidden 2048, 256 experts, top-8, expert intermediate 512
    m, h, mi, E, top_k = 2048, 2048, 512, 256, 8
    pairs = m * top_k
    x = torch.randn(m, h, device=dev, generator=g).bfloat16()
    wgu = (torch.randn(E * 2 * mi, h, device=dev, generator=g) * h**-0.5).bfloat16()
    wd = (torch.randn(E * h, mi, device=dev, generator=g) * mi**-0.5).bfloat16()
    scores = torch.randn(m, E, device=dev, generator=g).bfloat16()
    route = torch.zeros(m, 2 * top_k, device=dev, dtype=torch.int32)
    lst = torch.zeros(pairs, device=dev, dtype=torch.int32)
    tiles = torch.zeros(1 + 3 * hb.lib().hb_moe_tiles(m, top_k, E, 16), device=dev, dtype=torch.int32)
    ehb = torch.zeros(pairs, mi, device=dev, dtype=torch.bfloat16)
    ey = torch.zeros(pairs, h, device=dev, dtype=torch.bfloat16)
    egu = torch.zeros(pairs, 2 * mi, device=dev, dtype=torch.bfloat16)
    xsb = torch.zeros(pairs, h, device=dev, dtype=torch.bfloat16)
    outb = torch.zeros(m, h, device=dev, dtype=torch.bfloat16)
    k_route = ctx.route(E, top_k)
    k_route(m, wrap(scores), wrap(route))
    ctx.sync()
    pick = sel.experts(E, top_k, h, mi, m, wrap(route), wrap(lst), wrap(tiles), wrap(x), wrap(wgu), wrap(wd), wrap(ehb), wrap(ey), wrap(egu), wrap(xsb))
    ops = [(k_route, m, wrap(scores), wrap(route)), (pick["sort"], m, wrap(route), wrap(lst), wrap(tiles))]
    if pick["gather"]:
        ops += [(pick["gather"], m, wrap(x), wrap(lst), wrap(xsb)), (pick["gate_up"], m, wrap(wgu), wrap(xsb), wrap(ehb), wrap(lst), wrap(tiles))]
    elif pick["swiglu"]:
        ops += [(pick["gate_up"], m, wrap(wgu), wrap(x), wrap(egu), wrap(lst), wrap(tiles)), (pick["swiglu"], pairs, wrap(egu), wrap(ehb))]
    else:
        ops += [(pick["gate_up"], m, wrap(wgu), wrap(x), wrap(ehb), wrap(lst), wrap(tiles))]
    ops += [(pick["down"], m, wrap(wd), wrap(ehb), wrap(ey), wrap(lst), wrap(tiles)), (ctx.moe_combine(h, top_k), m, wrap(ey), wrap(route), wrap(outb))]
    gr = ctx.record(ops)  # the block as one recorded sequence, as a layer of the prefill step would be
    gr.time(3)
    barrier()
    sec_plain = max_over_ranks(gr.time(20) / 20)
    gr.free()
    out_plain = outb.clone()
    # the same sequence with overlapped launches: every kernel sets itself up under the tail of the one before and
    # waits for it inside
    ctx.set_launch_overlap(True)
    try:
        gr = ctx.record(ops)
    finally:
        ctx.set_launch_overlap(False)
    gr.time(3)
    barrier()
    sec_over = max_over_ranks(gr.time(20) / 20)
    gr.free()
    if not torch.equal(out_plain, outb):
        raise RuntimeError("moe block: overlapped launches changed the result")
    sec = min(sec_plain, sec_over)
    wbytes = 2.0 * E * (2 * mi * h + h * mi)
    flop = 2.0 * pairs * (2 * mi) * h + 2.0 * pairs * h * mi
    per_kernel = {}
    for op in ops:
        per_kernel[op[0].name] = ctx.time([op], 20) / 20 * 1e6
    # the whole sparse layer around that block (qwen.rs:2699-2733): router projection h -> E, the block, the shared
    # expert (gate/up + SwiGLU, down), and moe_out (sigmoid gate, sum, residual)
    try:
        wr = (torch.randn(E, h, device=dev, generator=g) * h**-0.5).bfloat16()
        wsg = (torch.randn(2 * mi, h, device=dev, generator=g) * h**-0.5).bfloat16()
        wsd = (torch.randn(h, mi, device=dev, generator=g) * mi**-0.5).bfloat16()
        gate_w = (torch.randn(h, device=dev, generator=g) * h**-0.5).bfloat16()
        resid = torch.randn(m, h, device=dev, generator=g).bfloat16()
        sh_h = torch.zeros(m, mi, device=dev, dtype=torch.bfloat16)
        sh_gu = torch.zeros(m, 2 * mi, device=dev, dtype=torch.bfloat16)
        sh_y = torch.zeros(m, h, device=dev, dtype=torch.bfloat16)
        k_router = sel.gemm(h, E, 0, wrap(wr), wrap(x), wrap(scores), m)
        k_sgu = sel.gate_up(h, mi, wrap(wsg), wrap(x), wrap(sh_gu), wrap(sh_h), m)
        k_sd = sel.gemm(mi, h, 0, wrap(wsd), wrap(sh_h), wrap(sh_y), m)
        full = [(k_router, m, wrap(wr), wrap(x), wrap(scores))] + ops
        full += [(k_sgu[0], m, wrap(wsg), wrap(x), wrap(sh_gu)), (k_sgu[1], m, wrap(sh_gu), wrap(sh_h))] if len(k_sgu) == 2 else [(k_sgu[0], m, wrap(wsg), wrap(x), wrap(sh_h))]
        full += [(k_sd, m, wrap(wsd), wrap(sh_h), wrap(sh_y)), (ctx.moe_out(h), m, wrap(x), wrap(gate_w), wrap(outb), wrap(sh_y), wrap(resid))]
        gr = ctx.record(full)
        gr.time(3)
        barrier()
        sec_full = max_over_ranks(gr.time(20) / 20)
        gr.free()
        out["moe_layer_full_2048tok"] = {"us": sec_full * 1e6, "kernels": len(full), "tokens_per_s": m / sec_full,
                                         "router": k_router.name, "shared_gate_up": "+".join(k_.name for k_ in k_sgu), "shared_down": k_sd.name}
    except Exception as e:
        out["moe_layer_error"] = repr(e)
    out["moe_2048tok_256e_top8"] = {"us": sec * 1e6, "tile_rows": pick["bm"], "weight_gbs": wbytes / sec / 1e9, "frac_hbm": wbytes / sec / 1e9 / pk["hbm_gbs"],
                                    "tflops": flop / sec / 1e12, "us_per_kernel": per_kernel,
                                    "launches_us": {"plain": sec_plain * 1e6, "overlapped": sec_over * 1e6}}
    return out


def contract_report(torch, ref, got, share, rows, reference):
    """The engine's contract on two bf16 tensors (at most 1 ulp apart on all but `share` of the elements, max|err| <=
    max|ref| / 64) as the object the JSON line carries."""
    def ordered(t):  # bf16 bits as integers that grow with the value
        i = t.contiguous().view(torch.int16).int()
        return torch.where(i < 0, -(i & 0x7FFF), i)

    ulp = (ordered(ref) - ordered(got)).abs()
    err = float((ref.float() - got.float()).abs().max())
    scale = max(float(ref.float().abs().max()), 1e-6)
    over = int((ulp > 1).sum())
    return {"rows": rows, "elements": ref.numel(), "bit_equal": int((ulp == 0).sum()), "over_1ulp": over, "max_ulp": int(ulp.max()),
            "max_err_over_scale": err / scale, "within_contract": bool(over <= share * ref.numel() and err <= scale / 64), "allowed_share_over_1ulp": share,
            "reference": reference}


def swiglu_ref(torch, acc16):
    """bf16(g * sigmoid(g) * u) over [gate | up] columns that are bf16 already, in f32 as the epilogue does."""
    n = acc16.shape[1] // 2
    g, u = acc16[:, :n].float(), acc16[:, n:].float()
    return ((g * (1.0 / (1.0 + torch.exp(-g)))) * u).bfloat16()


def bench_sharded(hb, ctx, torch, dev, pk, rank, world, barrier, max_over_ranks):
    """The two configurations that shard (strong scaling, total work fixed): the 27B-class FFN tensor-parallel
    over `world` ranks and the MoE block expert-parallel. At world = 1 the same code runs without an exchange.
    Every rank builds the whole weights from one seed and keeps its shard, so that rank 0 can check sampled rows of
    the sharded result against the f64 product of the unsharded operands; with several ranks the one-GPU time of the
    same code is measured in the same job (t1) for the strong-scaling efficiency t1 / (world * t)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("hb200_dist", os.path.join(ROOT, "herbert-metal-bf16_b200", "dist.py"))
    D = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(D)
    out = {}
    stream = torch.cuda.Stream(dev)
    ctx.sync()
    ctx.set_stream(stream.cuda_stream)

    def dist_all_gather(parts, t):
        import torch.distributed as dist

        dist.all_gather(parts, t)

    try:
        with torch.cuda.stream(stream):
            be = D.GpuBackend(hb, ctx, rows_max=2048)
            g = torch.Generator(device=dev)
            g.manual_seed(99)  # the same tensors on every rank

            def timed(fn, warm, reps):
                for _ in range(warm):
                    fn()
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    fn()
                e1.record(stream)
                e1.synchronize()
                barrier()
                return max_over_ranks(e0.elapsed_time(e1) * 1e-3 / reps)

            def kernels_of(state, body):
                """Every kernel of one step of `state` timed alone (20 launches each, all ranks in step, max over ranks):
                the step's calls are taken down through the state's emitters instead of launched."""
                ops = []
                rec = lambda kern, mm, *ranges: ops.append((kern, mm, *ranges))
                state.emit = rec
                state.pb.emit = rec
                try:
                    body()
                finally:
                    state.emit = D._launch_now
                    state.pb.emit = D._launch_now
                res = []
                for op in ops:
                    stream.synchronize()
                    barrier()
                    ctx.time([op], 2)
                    barrier()
                    res.append({"kernel": op[0].name, "us": max_over_ranks(ctx.time([op], 20) / 20) * 1e6})
                return res

            sample = torch.randperm(2048, generator=torch.Generator().manual_seed(5))[:16].sort().values.to(dev)

            # -- the 27B-class FFN: hidden 5120, intermediate 17408, M = 2048
            m, h, inter = 2048, 5120, 17408
            if inter % world == 0:
                x = torch.randn(m, h, device=dev, generator=g).bfloat16()
                y = torch.randn(m, h, device=dev, generator=g).bfloat16()
                wgu = (torch.randn(2 * inter, h, device=dev, generator=g) * h**-0.5).bfloat16()
                wd = (torch.randn(h, inter, device=dev, generator=g) * inter**-0.5).bfloat16()
                wgu_l, wd_l = D.shard_gate_up(wgu, rank, world), D.shard_down(wd, rank, world)
                flop = 2.0 * m * (2 * inter) * h + 2.0 * m * h * inter
                # the production form: the down GEMM's epilogue stores every block of rows of its f32 partial into the
                # staging buffer of the rank that sums it (reduce-scatter under the GEMM), tp_sum adds the staged blocks
                # in rank order, rounds, adds the residual and stores the bf16 rows into every rank's Y ...
                tp = D.TpPeer(hb, ctx, rank, world, m, h)
                D.tp_peer_connect(tp)
                tp.set_y(y)
                got = D.tp_ffn_peer(tp, x, wgu_l, wd_l).clone()
                # Sampled rows against the f64 product of the unsharded operands, stage by stage as the tests do: the SwiGLU
                # rows every rank made (three roundings: a looser rate, see tests/test_gpu_full_size.py), then the sharded
                # sum over exactly those rows under the engine's contract.
                hm_l = tp.kernels[(h, inter // world)][2][sample].contiguous()
                if world > 1:
                    parts = [torch.empty_like(hm_l) for _ in range(world)]
                    dist_all_gather(parts, hm_l)
                    hm_gpu = torch.cat(parts, dim=1)
                else:
                    hm_gpu = hm_l
                xs_ = x[sample].double()
                hm = swiglu_ref(torch, torch.cat([(xs_ @ wgu[c : c + 8704].double().t()).float().bfloat16() for c in range(0, 2 * inter, 8704)], dim=1))
                parity_swiglu = contract_report(torch, hm, hm_gpu, 3e-3, int(sample.numel()), "f64 gate and up sums of the unsharded weights on the GPU, then the three roundings of the SwiGLU epilogue")
                acc = torch.cat([(hm_gpu.double() @ wd[c : c + 1280].double().t()).float().bfloat16() for c in range(0, h, 1280)], dim=1)
                want = (y[sample].float() + acc.float()).bfloat16()
                parity = contract_report(torch, want, got[sample], 1e-3, int(sample.numel()), "f64 product of all ranks' SwiGLU rows with the unsharded down weights on the GPU, one rounding, residual add")
                parity["gate_up_swiglu_stage"] = parity_swiglu
                # (the step's kernels recorded once and replayed with one call; also launched one by one from the host)
                sec = timed(lambda: D.tp_ffn_peer(tp, x, wgu_l, wd_l, recorded=True), 3, 10)
                sec_loop = timed(lambda: D.tp_ffn_peer(tp, x, wgu_l, wd_l), 3, 10) if world > 1 else sec
                tp_kernels = kernels_of(tp, lambda: D._tp_step_body(tp, x, wgu_l, wd_l, None, False))
                # the other two forms of the exchange over the same kernels: the partial stays local and tp_reduce pulls the
                # blocks it sums from the peers; the GEMM flags finished row groups and the sum runs beside it
                other_forms = {}
                forms_ = (("pull", dict(mode="pull")), ("stream", dict(mode="stream")), ("pushsync", dict(mode="pushsync")),
                          ("push, barrier kernels", dict(mode="push", fold_barriers=False))) if world > 1 else ()
                for mode_, kw_ in forms_:
                    tpl = D.TpPeer(hb, ctx, rank, world, m, h, **kw_)
                    D.tp_peer_connect(tpl)
                    tpl.set_y(y)
                    got_other = D.tp_ffn_peer(tpl, x, wgu_l, wd_l).clone()
                    other_forms[mode_] = timed(lambda: D.tp_ffn_peer(tpl, x, wgu_l, wd_l, recorded=True), 3, 10)
                    if not torch.equal(got_other, got):
                        raise RuntimeError(f"tp_ffn: the {tp.mode} and the {mode_} form differ")
                    barrier()
                    tpl.close()
                sec_pull = other_forms.get("pull", sec)
                # ... and the same FFN with an NCCL all-reduce of the f32 partials and a separate epilogue (the baseline form)
                y2 = y.clone()
                D.tp_ffn(be, x, wgu_l, wd_l, y2)
                same = bool(torch.equal(y2, got))
                # (beyond two ranks NCCL sums the partials in another order than rank 0 + rank 1 + ...: not the same bits)
                diff = float((y2.float() - got.float()).abs().max())
                scale = float(got.float().abs().max())
                sec_nccl = timed(lambda: D.tp_ffn(be, x, wgu_l, wd_l, y2), 3, 10)
                barrier()
                tp.close()
                t1 = sec
                if world > 1:  # the same code on this GPU alone, the whole weights
                    one = D.TpPeer(hb, ctx, 0, 1, m, h)
                    one.connect([one])
                    one.set_y(y)
                    t1 = timed(lambda: D.tp_ffn_peer(one, x, wgu, wd), 3, 10)
                    one.close()
                out["tp_ffn_27b_m2048"] = {"n_gpus": world, "us": sec * 1e6, "t1_us": t1 * 1e6, "efficiency": t1 / (world * sec), "tflops_total": flop / sec / 1e12,
                                           "tflops_per_gpu": flop / sec / 1e12 / world, "frac_of_measured_peak_per_gpu": flop / sec / 1e12 / world / pk["bf16_tflops"],
                                           "nvlink_bytes_per_gpu": (m * h * 4 + m * h * 2) * (world - 1) // world if world > 1 else 0, "scaling": "strong",
                                           "kernels_per_step": tp.kernels_per_step, "parity": parity, "kernels_us": tp_kernels,
                                           "exchange": tp.describe(),
                                           "launched_one_by_one_us": sec_loop * 1e6, "pull_form_us": sec_pull * 1e6,
                                           "forms_us": {tp.mode: sec * 1e6, **{k_: v * 1e6 for k_, v in other_forms.items()}},
                                           "nccl_form_us": sec_nccl * 1e6, "equals_nccl_form_bitwise": same,
                                           "max_abs_diff_vs_nccl_form": diff, "max_abs_value": scale}
                del wgu, wd, wgu_l, wd_l
            # -- the MoE block: 2048 tokens, hidden 2048, 256 experts, top-8, expert intermediate 512
            m, h, mi, E, top_k, bm = 2048, 2048, 512, 256, 8, 64
            if m % world == 0 and E % world == 0:
                rl, epr = m // world, E // world
                x_all = torch.randn(m, h, device=dev, generator=g).bfloat16()
                sc_all = torch.randn(m, E, device=dev, generator=g).bfloat16()
                wgu = (torch.randn(E * 2 * mi, h, device=dev, generator=g) * h**-0.5).bfloat16()
                wd = (torch.randn(E * h, mi, device=dev, generator=g) * mi**-0.5).bfloat16()
                xs, sc = x_all[rank * rl : (rank + 1) * rl].contiguous(), sc_all[rank * rl : (rank + 1) * rl].contiguous()
                wgu_l, wd_l = wgu[rank * epr * 2 * mi : (rank + 1) * epr * 2 * mi], wd[rank * epr * h : (rank + 1) * epr * h]
                wbytes = 2.0 * E * 3 * mi * h
                # the exchange through peer memory by the library's own kernels (the production form) ...
                st = D.EpPeer(hb, ctx, rank, world, rl, h, mi, E, top_k, bm)
                D.ep_peer_connect(st)
                got = D.ep_moe_peer(st, xs, sc, wgu_l, wd_l).clone()
                stream.synchronize()
                # sampled token rows of this rank against the f64 chain over the whole weights, the route as the GPU made it
                rows_s = sample[sample < rl][:8] if world > 1 else sample[:8]
                if rows_s.numel() == 0:
                    rows_s = torch.arange(min(8, rl), device=dev)
                route = st.route[rows_s].cpu()
                want = torch.zeros(rows_s.numel(), h, device=dev, dtype=torch.bfloat16)
                for i in range(rows_s.numel()):
                    xr = xs[rows_s[i]].double()[None]
                    accr = torch.zeros(1, h, device=dev, dtype=torch.bfloat16)
                    for s_ in range(top_k):
                        e = int(route[i, s_])
                        wgt = torch.tensor([int(route[i, top_k + s_])], dtype=torch.int32).view(torch.float32).to(dev)
                        hm = swiglu_ref(torch, (xr @ wgu[e * 2 * mi : (e + 1) * 2 * mi].double().t()).float().bfloat16())
                        yr = (hm.double() @ wd[e * h : (e + 1) * h].double().t()).float().bfloat16()
                        accr = (accr.float() + (yr.float() * wgt).bfloat16().float()).bfloat16()
                    want[i] = accr[0]
                parity = contract_report(torch, want, got[rows_s], 0.05, int(rows_s.numel()), "f64 chain over the unsharded expert weights on the GPU (gate/up, SwiGLU, down, bf16 combine chain: the roundings of three stages compound, so 5 % of the outputs may be over 1 ulp)")
                sec = timed(lambda: D.ep_moe_peer(st, xs, sc, wgu_l, wd_l, recorded=True), 4, 20)
                got_rec = D.ep_moe_peer(st, xs, sc, wgu_l, wd_l, recorded=True).clone()
                if not torch.equal(got_rec, got):
                    raise RuntimeError("ep_moe: the replayed step differs from the step launched kernel by kernel")
                sec_loop = timed(lambda: D.ep_moe_peer(st, xs, sc, wgu_l, wd_l), 3, 20) if world > 1 else sec

                def ep_body():
                    D._ep_step_body(st, xs, sc, wgu_l, wd_l, None, False)
                    st.parity ^= 1  # taken down, not run: the two offset buffers keep their turn

                ep_kernels = kernels_of(st, ep_body)
                # ... and the same block with the rows exchanged by NCCL all-to-all, host-known counts (the baseline form)
                ref = D.ep_moe(be, xs, sc, wgu_l, wd_l, E, top_k, mi, bm)
                same = bool(torch.equal(ref, got))
                sec_nccl = timed(lambda: D.ep_moe(be, xs, sc, wgu_l, wd_l, E, top_k, mi, bm), 2, 5)
                barrier()
                kernels_per_step = st.kernels_per_step
                st.close()
                t1 = sec
                if world > 1:  # the same code on this GPU alone: all tokens, all experts
                    one = D.EpPeer(hb, ctx, 0, 1, m, h, mi, E, top_k, bm)
                    one.connect([one])
                    t1 = timed(lambda: D.ep_moe_peer(one, x_all, sc_all, wgu, wd), 3, 10)
                    one.close()
                out["moe_ep_2048tok"] = {"n_gpus": world, "us": sec * 1e6, "t1_us": t1 * 1e6, "efficiency": t1 / (world * sec), "weight_gbs_total": wbytes / sec / 1e9,
                                         "tokens_per_s": m / sec, "scaling": "strong", "tile_rows": bm, "kernels_per_step": kernels_per_step, "parity": parity, "kernels_us": ep_kernels,
                                         "exchange": "peer-memory stores and loads by the library's kernels: every source owns a region of the owners' buffers (no counts exchanged first), the dispatch flags its landing and the plan waits for the flags, the combine carries the outputs-complete barrier and pulls the expert outputs (no NCCL call in the step); the step replayed as one recorded sequence" if world > 1 else "one GPU: the plain block",
                                         "launched_one_by_one_us": sec_loop * 1e6,
                                         "nccl_form_us": sec_nccl * 1e6, "equals_nccl_form_bitwise": same}
                if world > 1:
                    # weak scaling: 2048 tokens on every rank (the experts still partitioned), peer-memory form. The
                    # buffers hold four times the average number of received rows (an overflow would be reported).
                    try:
                        gl = torch.Generator(device=dev)
                        gl.manual_seed(1000 + rank)
                        xw = torch.randn(m, h, device=dev, generator=gl).bfloat16()
                        sw = torch.randn(m, E, device=dev, generator=gl).bfloat16()
                        stw = D.EpPeer(hb, ctx, rank, world, m, h, mi, E, top_k, bm, cap=min(m * top_k * world, 4 * m * top_k))
                        D.ep_peer_connect(stw)
                        sec_w = timed(lambda: D.ep_moe_peer(stw, xw, sw, wgu_l, wd_l, recorded=True), 4, 10)
                        ctx.sync()
                        barrier()
                        stw.close()
                        out["moe_ep_weak_2048tok_per_gpu"] = {"n_gpus": world, "us": sec_w * 1e6, "tokens_per_s_total": m * world / sec_w, "scaling": "weak",
                                                              "weight_gbs_total": wbytes / sec_w / 1e9}
                        del stw
                    except Exception as e:
                        out["moe_ep_weak_error"] = repr(e)
    finally:
        stream.synchronize()
        ctx.set_stream(None)
    return out


def cpu_baseline():
    """The oracle's f32-accumulate contract kernel on the host cores, on a bounded sample: the small dense GEMM
    (M=512, K=1024, N=4096) repeated, and one matvec pass; about 10-20 s in all."""
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import Oracle

    o = Oracle(native=True)
    rng = np.random.default_rng(0)

    def bf16(a):
        b = a.astype(np.float32).view(np.uint32)
        return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)

    rows = 128
    ws = [bf16(rng.standard_normal((n, k), dtype=np.float32) * k**-0.5) for _, k, n, _ in LAYER]
    xs = [bf16(rng.standard_normal((rows, k), dtype=np.float32)) for _, k, _, _ in LAYER]
    y0 = bf16(rng.standard_normal((rows, HIDDEN), dtype=np.float32))

    def step():
        for (name, k, n, out), w, x in zip(LAYER, ws, xs):
            o.gemm_f32(x, w, out, y0 if out == 2 else None)

    step()
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0 and reps < 50:
        step()
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    value = STEP_FLOP * rows / ROWS / dt / 1e12
    # the small dense GEMM in full (M=512, K=1024, N=4096): the case the CPU restatement runs whole
    w1 = bf16(rng.standard_normal((4096, 1024), dtype=np.float32) / 32.0)
    x1 = bf16(rng.standard_normal((512, 1024), dtype=np.float32))
    o.gemm_f32(x1, w1, 0, None)
    t1 = time.perf_counter()
    for _ in range(10):
        o.gemm_f32(x1, w1, 0, None)
    c1 = (time.perf_counter() - t1) / 10
    return {"value": value, "unit": "TFLOP/s", "cores": o.threads(), "kind": "port",
            "sample": f"{rows} of {ROWS} rows of every GEMM of the layer set, {reps} passes, f32 accumulate + one RNE (oracle/hb_oracle.c, OpenMP)",
            "config1_512x1024x4096_ms": c1 * 1e3, "config1_tflops": 2.0 * 512 * 1024 * 4096 / c1 / 1e12}


if __name__ == "__main__":
    main()
