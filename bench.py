#!/usr/bin/env python
"""Benchmark of the fe2o3 example hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the workload's hot
path over one batch of seeded synthetic input.  `value` is timed with CUDA
events with inputs resident in HBM; `e2e` is the same pass through the public
host API with pinned host buffers, host<->device copies inside the timed
region.  Inputs are synthetic (SplitMix64-keyed generators); no dataset is
involved.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE = "moe_top2_v1"
L2_FLUSH_BYTES = 256 << 20


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) in a thread
    while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index):
        self.index, self.mhz, self.reasons, self.max_mhz = index, [], set(), None
        self.stop_flag, self.thread, self.nv, self.handle = threading.Event(), None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.mhz.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for name, bit in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def start(self):
        if self.nv and self.thread is None:
            self.stop_flag.clear()
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        if self.thread:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            self.thread = None

    def summary(self):
        return {"sm_mhz": float(np.median(self.mhz)) if self.mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.mhz)}


class Harness:
    def __init__(self, rank, world, local_rank):
        import torch
        import fe2o3_b200 as fe
        self.torch, self.fe = torch, fe
        self.rank, self.world = rank, world
        torch.cuda.set_device(local_rank)
        self.ctx = fe.GpuContext(local_rank)
        self.stream = self.ctx.default_stream()  # the legacy default stream, shared with torch
        self.flush_buf = None
        self.clocks = None  # set for the headline workload: sampled over its timed region

    def barrier(self):
        if self.world > 1:
            self.torch.distributed.barrier()
        self.torch.cuda.synchronize()

    def flush_l2(self):
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(L2_FLUSH_BYTES, dtype=self.torch.uint8, device="cuda")
        self.flush_buf.zero_()

    def time_steps(self, step, steps, warmup, flush):
        """Returns per-step device milliseconds (list of `steps`)."""
        fe = self.fe
        for _ in range(warmup):
            if flush:
                self.flush_l2()
            step()
        ev = [(fe.Event(self.ctx), fe.Event(self.ctx)) for _ in range(steps)]
        self.barrier()
        if self.clocks:
            self.clocks.start()
        for s, e in ev:
            if flush:
                self.flush_l2()
            s.record(self.stream)
            step()
            e.record(self.stream)
        self.barrier()
        if self.clocks:
            self.clocks.stop()
        return [e.elapsed_time_ms_since(s) for s, e in ev]

    def max_over_ranks(self, x):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.torch.distributed.all_reduce(t, op=self.torch.distributed.ReduceOp.MAX)
        return float(t.item())


# DRAM bytes (read + write) of one launch of each workload's dominant kernel at the default full size,
# from one-pass ncu captures (dram__bytes_read.sum + dram__bytes_write.sum; summary under profiles/).
# Reported only when the workload runs at exactly that size.
NCU_TRAFFIC = {
    ("masked_reduce_u32", 1 << 28): 2147519744 + 3300352,
    ("row_softmax_v1", 65536 * 1024): 268459008 + 216675072,
    ("device_scan_u32", 1 << 28): 1074060800 + 1014678784,
    ("tiled_gemm_v1", (8192, 8192, 8192)): 1046762752 + 250886400,
    ("flash_attention_v1", (4, 16, 2048, 64)): 50588160 + 2605312,
    # grouped FFN GEMMs of one pass, average of the two launches (GEMM-1, which gathers its rows of x and clears
    # the output, 629 MB; GEMM-2, which adds the weighted rows into the output, 1056 MB)
    ("moe_top2_v1", (16384, 2048, 4096, 8)): (263091712 + 365496064 + 826510336 + 229486592) // 2,
}


def roofline(bound, achieved, peak, unit, traffic=None, peak_source="measured"):
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "traffic": traffic, "traffic_source": "ncu capture summarised under profiles/, not this run" if traffic else None,
            "peak_source": f"of {peak_source}"}


# ------------------------------------------------------------------ workloads

def wl_masked_reduce(h, steps, warmup, n=1 << 28, cpu=True):
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    host_v = ctx.pinned(n, np.uint32)
    host_a = ctx.pinned(n, np.uint32)
    host_o = ctx.pinned(1, np.uint32)
    synth.u32_below(1, 1 + h.rank * 16, n, 1 << 16, out=host_v)
    synth.bernoulli(1, 2 + h.rank * 16, n, 0.75, flag_value=7, packed=False, flags_out=host_a)
    v = fe.DeviceBuffer.zeroed(stream, n, np.uint32)
    a = fe.DeviceBuffer.zeroed(stream, n, np.uint32)
    o = fe.DeviceBuffer.zeroed(stream, 1, np.uint32)
    v.copy_from_host_async(stream, host_v)
    a.copy_from_host_async(stream, host_a)
    stream.synchronize()
    prep = fe.prepare(ctx, "masked_reduce_u32", values=v, active=a, output=o)
    l0 = fe.launch_count()
    ms = h.time_steps(lambda: prep.launch(stream), steps, warmup, flush=False)
    launches = fe.launch_count() - l0 - warmup
    o.copy_to_host_async(stream, host_o)
    stream.synchronize()
    got = int(host_o[0])
    step_ms = h.max_over_ranks(float(np.mean(ms)))
    alg_bytes = n * 8 + 4
    res = {"ms_per_step": step_ms, "value": h.world * n / (step_ms * 1e-3), "unit": "elements/s",
           "launches": launches,
           "roofline": roofline("hbm", alg_bytes / (float(np.mean(ms)) * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s",
                                traffic=NCU_TRAFFIC.get(("masked_reduce_u32", n)), peak_source=peaks["source"]),
           "workload": {"workload": "masked_reduce_u32", "elements": n, "values": "uniform[0,2^16) seed 1",
                        "mask": "Bernoulli(0.75) u32 flags {0,7}", "algorithmic_bytes_per_step": alg_bytes,
                        "l2": "inputs (2 GiB) larger than L2"}}

    # end to end: pinned host -> device, launch, result back to host, every step
    def e2e_step():
        v.copy_from_host_async(stream, host_v)
        a.copy_from_host_async(stream, host_a)
        prep.launch(stream)
        o.copy_to_host_async(stream, host_o)
        stream.synchronize()
    e2e_steps = max(2, min(steps, 5))
    e2e_step()
    h.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    h.barrier()
    e2e_s = h.max_over_ranks((time.perf_counter() - t0) / e2e_steps)
    res["e2e"] = {"value": h.world * n / e2e_s, "unit": "elements/s", "h2d_bytes_per_step": 8 * n,
                  "d2h_bytes_per_step": 4, "ms_per_step": e2e_s * 1e3}
    if cpu and h.rank == 0:
        import oracle
        oracle.build()
        oracle.set_threads(os.cpu_count())
        best, want = None, None
        for _ in range(5):
            t0 = time.perf_counter()
            want = oracle.masked_sum_u32(host_v, host_a, parallel=True)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        res["cpu_baseline"] = {"value": n / best, "unit": "elements/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": f"the full {n}-element workload, best of 5 passes of the OpenMP oracle"}
        res["parity"] = {"bit_exact": got == want, "gpu": got, "oracle": want}
        if got != want:
            raise SystemExit(f"masked_reduce_u32 mismatch: gpu {got} oracle {want}")
    return res


def wl_scan(h, steps, warmup, n=1 << 28, cpu=True):
    """Device-wide inclusive u32 prefix sum: 4 bytes in and 4 bytes out per element."""
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    host_v = ctx.pinned(n, np.uint32)
    synth.u32_below(1, 3, n, 1 << 16, out=host_v)
    host_o = ctx.pinned(n, np.uint32)
    v = fe.DeviceBuffer.from_host(stream, host_v)
    o = fe.DeviceBuffer.zeroed(stream, n, np.uint32)
    prep = fe.prepare(ctx, "device_scan_u32", values=v, output=o, exclusive=0)
    ms = h.time_steps(lambda: prep.launch(stream), steps, warmup, flush=False)
    if ctx.take_kernel_status(stream):
        raise RuntimeError("scan reported a kernel status word")
    step_ms = h.max_over_ranks(float(np.mean(ms)))
    alg = n * 8
    res = {"ms_per_step": step_ms, "value": h.world * n / (step_ms * 1e-3), "unit": "elements/s", "launches": steps,
           "roofline": roofline("hbm", alg / (float(np.mean(ms)) * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s",
                                traffic=NCU_TRAFFIC.get(("device_scan_u32", n)), peak_source=peaks["source"]),
           "workload": {"workload": "device_scan_u32", "elements": n, "values": "uniform[0,2^16) seed 1 domain 3",
                        "algorithmic_bytes_per_step": alg, "l2": "input+output (2 GiB) larger than L2"}}

    def e2e_step():
        v.copy_from_host_async(stream, host_v)
        prep.launch(stream)
        o.copy_to_host_async(stream, host_o)
        stream.synchronize()
    e2e_step()
    t0 = time.perf_counter()
    e2e_step()
    dt = time.perf_counter() - t0
    res["e2e"] = {"value": n / dt, "unit": "elements/s", "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 4 * n}
    if cpu and h.rank == 0:
        import oracle
        t0 = time.perf_counter()
        want = oracle.scan_sum_u32(host_v)
        dt = time.perf_counter() - t0
        res["cpu_baseline"] = {"value": n / dt, "unit": "elements/s", "cores": 1, "kind": "port",
                               "sample": f"the full {n}-element workload, sequential oracle"}
        res["parity"] = {"bit_exact": bool((host_o == want).all())}
    return res


def wl_row_softmax(h, steps, warmup, rows=65536, cols=1024, cpu=True):
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    n = rows * cols
    host_x = ctx.pinned(n, np.float32)
    host_y = ctx.pinned(n, np.float32)
    synth.normal_f32(2, 1, n, 2.0, out=host_x)
    x = fe.DeviceBuffer.zeroed(stream, n, np.float32)
    y = fe.DeviceBuffer.zeroed(stream, n, np.float32)
    x.copy_from_host_async(stream, host_x)
    stream.synchronize()
    prep = fe.prepare(ctx, "row_softmax_v1", input=x, output=y, rows=rows, cols=cols)
    ms = h.time_steps(lambda: prep.launch(stream), steps, warmup, flush=False)
    step_ms = float(np.mean(ms))
    alg = n * 8
    res = {"ms_per_step": step_ms, "value": alg / (step_ms * 1e-3) / 1e9, "unit": "GB/s",
           "roofline": roofline("hbm", alg / (step_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s",
                                traffic=NCU_TRAFFIC.get(("row_softmax_v1", n)), peak_source=peaks["source"]),
           "workload": {"workload": "row_softmax_v1", "rows": rows, "cols": cols, "algorithmic_bytes_per_step": alg,
                        "l2": "input+output (512 MiB) larger than L2"}}
    y.copy_to_host_async(stream, host_y)
    stream.synchronize()
    t0 = time.perf_counter()
    x.copy_from_host_async(stream, host_x)
    prep.launch(stream)
    y.copy_to_host_async(stream, host_y)
    stream.synchronize()
    dt = time.perf_counter() - t0
    res["e2e"] = {"value": alg / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 4 * n}
    if cpu:
        import oracle
        oracle.set_threads(os.cpu_count())
        sample = 4096
        t0 = time.perf_counter()
        st, want = oracle.row_softmax(host_x[: sample * cols].reshape(sample, cols))
        dt = time.perf_counter() - t0
        got = host_y[: sample * cols].reshape(sample, cols)
        rel = float((np.abs(got - want) / np.maximum(np.abs(want), 1e-30)).max())
        res["cpu_baseline"] = {"value": sample * cols * 8 / dt / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
                               "kind": "port", "sample": f"first {sample} rows"}
        res["parity"] = {"max_rel": rel, "tolerance": 1e-5, "ok": bool(st == 0 and rel <= 1e-5)}
    return res


def wl_gemm(h, steps, warmup, m=8192, n=8192, k=8192, cpu=True):
    """C = A*B.  On N GPUs the global A has N*m rows: rank g owns the row block [g*m, (g+1)*m) of A and C
    (its own stream of the generator), B is replicated before timing, and there is no collective in the
    timed region (weak scaling: m rows per GPU)."""
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    # row block g of A is stream (seed 0, domain 1 + 16 g): every rank's block is a pure function of its index
    a_h, b_h = synth.uniform_bf16(0, 1 + 16 * h.rank, m * k), synth.uniform_bf16(0, 2, k * n)
    a, b = fe.DeviceBuffer.from_host(stream, a_h), fe.DeviceBuffer.from_host(stream, b_h)
    c = fe.DeviceBuffer.zeroed(stream, m * n, np.float32)
    prep = fe.prepare(ctx, "tiled_gemm_v1", schedule=fe.SCHEDULE_TCGEN05, a=a, b=b, c=c, m=m, n=n, k=k)
    h.barrier()
    ms = h.time_steps(lambda: prep.launch(stream), steps, warmup, flush=False)
    if ctx.take_kernel_status(stream):
        raise RuntimeError("tensor-core GEMM reported a kernel status word")
    local_ms = float(np.mean(ms))
    step_ms = h.max_over_ranks(local_ms)
    flops = 2.0 * m * n * k
    tf = flops / (local_ms * 1e-3) / 1e12
    res = {"ms_per_step": step_ms, "value": h.world * flops / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "scaling": "weak", "launches": steps,
           "roofline": roofline("tensor", tf, peaks["bf16_tflops"], "TFLOP/s",
                                traffic=NCU_TRAFFIC.get(("tiled_gemm_v1", (m, n, k))), peak_source=peaks["source"]),
           "workload": {"workload": "tiled_gemm_v1", "m": m * h.world, "n": n, "k": k, "dtype": "bf16 in, f32 out",
                        "sharding": f"row blocks of A and C, {m} rows per GPU, B replicated, no collective",
                        "algorithmic_flops_per_step": flops * h.world, "l2": "A+B (256 MiB) larger than L2"}}
    # end to end through the C ABI with host buffers: pinned H2D of A and B, the kernel, D2H of C
    host_a, host_b, host_c = ctx.pinned(m * k, np.uint16), ctx.pinned(k * n, np.uint16), ctx.pinned(m * n, np.float32)
    host_a[:], host_b[:] = a_h, b_h

    def e2e_step():
        a.copy_from_host_async(stream, host_a)
        b.copy_from_host_async(stream, host_b)
        prep.launch(stream)
        c.copy_to_host_async(stream, host_c)
        stream.synchronize()
    e2e_step()
    h.barrier()
    t0 = time.perf_counter()
    for _ in range(3):
        e2e_step()
    h.barrier()
    dt = h.max_over_ranks((time.perf_counter() - t0) / 3)
    res["e2e"] = {"value": h.world * flops / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * (m * k + k * n) * h.world,
                  "d2h_bytes_per_step": 4 * m * n * h.world, "ms_per_step": dt * 1e3}
    if cpu and h.rank == 0:
        import oracle
        oracle.set_threads(os.cpu_count())
        rows = 8
        got = c.to_host_vec(stream)[: rows * n]
        t0 = time.perf_counter()
        want = oracle.gemm_bf16_rows(rows, n, k, a_h[: rows * k], b_h)
        dt = time.perf_counter() - t0
        err = float(np.abs(got - want).max())
        res["cpu_baseline"] = {"value": 2.0 * rows * n * k / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                               "kind": "port", "sample": f"first {rows} rows of C"}
        res["parity"] = {"max_abs": err, "tolerance": 1e-3 * float(np.sqrt(k)) / 3, "ok": bool(err <= 1e-3 * np.sqrt(k) / 3)}
    return res


def wl_attention(h, steps, warmup, batch=4, heads=16, seq=2048, dim=64, cpu=True):
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    n = batch * heads * seq * dim
    host = [ctx.pinned(n, np.uint16) for _ in range(3)]
    for i, buf in enumerate(host):
        synth.normal_bf16(3, 1 + i, n, 1.0, out=buf)
    host_o = ctx.pinned(n, np.float32)
    q, k, v = (fe.DeviceBuffer.from_host(stream, b) for b in host)
    o = fe.DeviceBuffer.zeroed(stream, n, np.float32)
    scale = 1.0 / float(np.sqrt(dim))
    prep = fe.prepare(ctx, "flash_attention_v1", q=q, k=k, v=v, output=o, batch=batch, heads=heads, seq=seq, dim=dim,
                      scale=scale, causal=0, input_dtype=fe.DTYPE_BF16)
    ms = h.time_steps(lambda: prep.launch(stream), steps, warmup, flush=True)
    if ctx.take_kernel_status(stream):
        raise RuntimeError("attention reported a kernel status word")
    step_ms = float(np.mean(ms))
    flops = 4.0 * batch * heads * seq * seq * dim
    tf = flops / (step_ms * 1e-3) / 1e12
    res = {"ms_per_step": step_ms, "value": tf, "unit": "TFLOP/s",
           "roofline": roofline("tensor", tf, peaks["bf16_tflops"], "TFLOP/s",
                                traffic=NCU_TRAFFIC.get(("flash_attention_v1", (batch, heads, seq, dim))),
                                peak_source=peaks["source"]),
           "workload": {"workload": "flash_attention_v1", "batch": batch, "heads": heads, "seq": seq, "dim": dim,
                        "causal": False, "dtype": "bf16 in, f32 out", "algorithmic_flops_per_step": flops,
                        "l2": "256 MiB L2 flush between steps"}}

    def e2e_step():
        for d, s in zip((q, k, v), host):
            d.copy_from_host_async(stream, s)
        prep.launch(stream)
        o.copy_to_host_async(stream, host_o)
        stream.synchronize()
    e2e_step()
    t0 = time.perf_counter()
    for _ in range(3):
        e2e_step()
    dt = (time.perf_counter() - t0) / 3
    res["e2e"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 6 * n, "d2h_bytes_per_step": 4 * n}
    if cpu:
        import oracle
        oracle.set_threads(os.cpu_count())
        # Bounded sample: every query row of eight (batch, head) pairs against all keys, spread over the
        # schedule: early rounds of the persistent kernel and the last round, whose units are split into
        # single 128-row tiles (at the default shape the heads from 55 on).
        S, D, bh = seq, dim, batch * heads
        picks = sorted({0, bh // 7, bh // 3, (bh * 4) // 7, bh - 9 if bh > 9 else 0, bh - 8 if bh > 8 else 0, bh - 4 if bh > 4 else 0,
                        bh - 1})
        f = lambda b, i: synth.bf16_to_f32(b[i * S * D:(i + 1) * S * D]).reshape(1, 1, S, D)
        worst, ok, dt = 0.0, True, 0.0
        for i in picks:
            t0 = time.perf_counter()
            st, want = oracle.flash_attention(f(host[0], i), f(host[1], i), f(host[2], i), scale, False)
            dt += time.perf_counter() - t0
            got = host_o[i * S * D:(i + 1) * S * D].reshape(S, D)
            err = np.abs(got - want[0, 0]) - (2e-3 * np.abs(want).max() + 2e-2 * np.abs(want[0, 0]))
            worst = max(worst, float(np.abs(got - want[0, 0]).max()))
            ok = ok and st == 0 and bool(err.max() <= 0)
        res["cpu_baseline"] = {"value": 4.0 * len(picks) * S * S * D / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
                               "kind": "port",
                               "sample": f"{len(picks)} of {bh} heads, {S} queries x {S} keys each, f64 two-pass oracle"}
        res["parity"] = {"max_abs": worst, "tolerance": "2e-3*max|e| + 2e-2*|e|", "heads_checked": picks, "ok": ok}
        if not ok:
            raise SystemExit(f"flash_attention_v1 mismatch against the oracle on heads {picks}: max_abs {worst}")
    return res


MOE_SHAPE = dict(tokens=16384, d_model=2048, d_ff=4096, experts=8)


def moe_inputs(rank, world, tokens, d_model, d_ff, experts):
    """This rank's shard of the seeded MoE inputs (x rows and expert weights)."""
    from fe2o3_b200 import synth
    t_local, per = tokens // world, experts // world
    full_x = synth.normal_bf16(4, 1, tokens * d_model, 1.0)
    x = full_x[rank * t_local * d_model:(rank + 1) * t_local * d_model]
    wg = synth.normal_bf16(4, 2, d_model * experts, 0.02)
    # expert e's matrices are streams (4, 100 + e) and (4, 200 + e): shards are independent of `world`
    w1 = np.concatenate([synth.normal_bf16(4, 100 + e, d_model * d_ff, 0.02) for e in range(rank * per, (rank + 1) * per)])
    w2 = np.concatenate([synth.normal_bf16(4, 200 + e, d_ff * d_model, 0.02) for e in range(rank * per, (rank + 1) * per)])
    return x, wg, w1, w2


def moe_oracle_tokens(oracle, x_rows, wg, w1_all, w2_all, n, d, f, E):
    """`n` tokens (rows of x) through the CPU oracle: gate, top-2, route weights, expert FFN, combine, with
    room for every route (no drops), which is also what the layer is given.  Tokens are independent
    then, so any subset of a batch can be checked on its own."""
    logits = oracle.moe_gate_logits(x_rows, wg, n, d, E)
    _, routing = oracle.moe_top2_route(logits, n, E, 2 * n)
    w = oracle.moe_route_weights(logits, routing["top2_experts"], n, E)
    compact = oracle.moe_expert_ffn(x_rows, w1_all, w2_all, routing["top2_experts"], routing["inverse"], n, d, f, E)
    _, want = oracle.moe_combine(compact, routing["inverse"], w, n, d)
    return routing["top2_experts"], want.reshape(n, d)


def wl_moe(h, steps, warmup, cpu=True, exchange="auto", **shape):
    fe = h.fe
    from fe2o3_b200.moe import MoeTop2Layer
    shape = {**MOE_SHAPE, **shape}
    T, d, f, E = shape["tokens"], shape["d_model"], shape["d_ff"], shape["experts"]
    peaks = measured_peaks()
    torch = h.torch
    layer = MoeTop2Layer(h.ctx, h.stream, T, d, f, E, rank=h.rank, world=h.world, io_sets=2, exchange=exchange)
    x, wg, w1, w2 = moe_inputs(h.rank, h.world, T, d, f, E)
    layer.load(x, wg, w1, w2)
    h.barrier()      # the ranks have prepared their inputs at different speeds: start the first pass together
    l0 = fe.launch_count()
    layer.forward()  # one eager pass: first-launch set-up happens outside any capture
    h.barrier()
    per_pass = fe.launch_count() - l0
    # the whole pass (all kernels of the layer) replays from one CUDA graph when no stage needs the host
    graphed = os.environ.get("FE2O3_BENCH_NO_GRAPH") is None and layer.capture()
    step = layer.replay if graphed else layer.forward
    ms = h.time_steps(step, steps, warmup, flush=False)
    launches = per_pass * steps
    if h.ctx.take_kernel_status(h.stream):
        raise RuntimeError("MoE reported a kernel status word")
    step_ms = h.max_over_ranks(float(np.mean(ms)))
    flops = T * 2 * 4.0 * d * f + 2.0 * T * d * E
    # Roofline of the dominant kernel: the two grouped FFN GEMMs of this rank on the rows the pass routed,
    # by CUDA events.  One GPU: the pair's duration inside the timed passes, as the pass minus the same pass
    # without the expert FFN, both replayed from CUDA graphs; beside it the pair replayed alone from a graph
    # of its own, which is slower (its first GEMM then finds no token rows in L2 and the GPU stays at its power
    # limit).  Several GPUs: the pair inside passes launched kernel by kernel (its first GEMM waits in the
    # kernel for the other ranks' rows and its second one stores rows into their memory, so it cannot run
    # outside a pass); that waiting is included.
    n_ffn = max(3, min(steps, 10))
    ffn_in_pass_ms = None
    if layer.exchange == "nccl":
        ffn_ms = float(np.mean(h.time_steps(lambda: layer.k_ffn.launch(h.stream), n_ffn, 3, flush=False)))
    elif h.world == 1 and layer.exchange == "none" and graphed:
        side = torch.cuda.Stream()
        pair_graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(pair_graph, stream=side):
            layer.k_ffn.launch(h.ctx.wrap_stream(side.cuda_stream))
        ffn_ms = float(np.mean(h.time_steps(pair_graph.replay, n_ffn, 3, flush=False)))
        # ... and what the pair takes inside the pass: the pass minus the same pass without the expert FFN
        # (gate, routing, route weights), both replayed from CUDA graphs.  Inside the pass the first GEMM finds
        # the token rows in L2 (the gate has just read them) and the GPU is not at its power limit throughout.
        rest_graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(rest_graph, stream=side):
            ss = h.ctx.wrap_stream(side.cuda_stream)
            layer.k_gate.launch(ss)
            layer.k_top2.launch(ss)
            layer.k_weights.launch(ss)
            if not layer.fused_combine:
                layer.k_combine.launch(ss)
        rest_ms = float(np.mean(h.time_steps(rest_graph.replay, n_ffn, 3, flush=False)))
        ffn_in_pass_ms = float(np.mean(ms)) - rest_ms
    else:
        marks = [(fe.Event(h.ctx), fe.Event(h.ctx)) for _ in range(n_ffn + 3)]
        h.barrier()
        for pair in marks:
            layer.forward(ffn_marks=pair)
        h.barrier()
        ffn_ms = float(np.mean([e.elapsed_time_ms_since(b) for b, e in marks[3:]]))
    ffn_rows = int(layer.ffn_rows())
    ffn_alone_ms = ffn_ms if ffn_in_pass_ms else None
    ffn_ms = ffn_in_pass_ms or ffn_ms   # the duration inside the timed region where it could be measured
    ffn_tf = ffn_rows * 4.0 * d * f / (ffn_ms * 1e-3) / 1e12
    sms = int(h.ctx.observe_environment().multiprocessors)
    m_tiles = -(-ffn_rows // 128) + (E // h.world)   # upper bound: one ragged tile per expert segment
    res = {"ms_per_step": step_ms, "value": T / (step_ms * 1e-3), "unit": "tokens/s", "launches": launches,
           "scaling": "strong",
           "roofline": {**roofline("tensor", ffn_tf, peaks["bf16_tflops"], "TFLOP/s",
                                   traffic=NCU_TRAFFIC.get(("moe_top2_v1", (T, d, f, E))) if h.world == 1 else None,
                                   peak_source=peaks["source"]),
                        "kernel": "gemm_tc_kernel<256>, the two grouped FFN GEMMs of the pass, combine included (two launches" +
                                  ("; duration inside the timed passes = pass minus the same pass without the expert FFN, both replayed "
                                   "from CUDA graphs; the pair replayed alone, where the first GEMM finds no token rows in L2, is "
                                   "given beside it)" if ffn_alone_ms else
                                   ", timed inside passes launched kernel by kernel, waits for other ranks included)"),
                        "rows": ffn_rows, "ms_per_pair": ffn_ms,
                        "frac_of_sustained_peak": ffn_tf / peaks["bf16_tflops_sustained"],
                        "ms_per_pair_replayed_alone": ffn_alone_ms,
                        "frac_replayed_alone": (ffn_rows * 4.0 * d * f / (ffn_alone_ms * 1e-3) / 1e12 / peaks["bf16_tflops"])
                        if ffn_alone_ms else None,
                        "whole_pass": {"achieved": flops / (step_ms * 1e-3) / 1e12 / h.world,
                                       "peak": peaks["bf16_tflops_sustained"],
                                       "frac": flops / (step_ms * 1e-3) / 1e12 / h.world / peaks["bf16_tflops_sustained"],
                                       "unit": "TFLOP/s", "peak_source": "of " + peaks["source"] + " (sustained, per GPU)"}},
           "workload": {"workload": "moe_top2_v1", **shape, "gate": "softmax(x*Wg), top-2 renormalised",
                        "ffn": "GELU(erf), bf16 hidden", "parallelism": f"ep{h.world}" if h.world > 1 else "single", "exchange": layer.exchange,
                        "peer_mapping": getattr(layer, "peer_mapping", None),
                        "cuda_graph": bool(graphed), "kernels_per_pass": per_pass,
                        "algorithmic_flops_per_step": flops,
                        "ffn_tiles": {"rows_this_rank": ffn_rows, "tile": "128x256", "sms": sms,
                                      "waves_gemm1": m_tiles * (-(-f // 256)) / sms, "waves_gemm2": m_tiles * (-(-d // 256)) / sms},
                        "share_outside_ffn": max(0.0, 1.0 - ffn_ms / float(np.mean(ms))),
                        "l2": "weights (256 MiB) + activations larger than L2"}}
    # end to end through the C ABI with host buffers: pinned H2D of this rank's tokens into the layer's
    # input buffer, the pass, D2H of its output, all on the layer's stream, every step
    t_local = T // h.world
    host_x = h.ctx.pinned(t_local * d, np.uint16)
    host_x[:] = x
    host_out = h.ctx.pinned(t_local * d, np.float32)

    def e2e_step():
        layer.x_buf.copy_from_host_async(h.stream, host_x)
        step()
        layer.out_buf.copy_to_host_async(h.stream, host_out)
        h.stream.synchronize()
    e2e_step()
    h.barrier()
    t0 = time.perf_counter()
    for _ in range(5):
        e2e_step()
    h.barrier()
    dt = h.max_over_ranks((time.perf_counter() - t0) / 5)
    res["e2e"] = {"value": T / dt, "unit": "tokens/s", "h2d_bytes_per_step": 2 * t_local * d * h.world,
                  "d2h_bytes_per_step": 4 * t_local * d * h.world, "ms_per_step": dt * 1e3,
                  "path": "fe2o3_buf_copy_from_host_async -> pass -> fe2o3_buf_copy_to_host_async -> fe2o3_stream_sync"}
    # The same with two steps in flight: the input of step i+1 goes up and the output of step i-1 comes down on
    # copy streams of their own while step i computes (two input/output buffer pairs, events between the
    # streams).  Every step's tokens and outputs still cross PCIe inside the timed region.
    up, down = h.ctx.create_stream(), h.ctx.create_stream()
    host_outs = [host_out, h.ctx.pinned(t_local * d, np.float32)]
    ev_in, ev_done, ev_out = ([fe.Event(h.ctx) for _ in range(2)] for _ in range(3))

    def pipelined(n):
        for i in range(n):
            b = i & 1
            if i >= 2:
                up.wait_event(ev_done[b])        # the pass two steps back has read this input buffer
            layer.x_bufs[b].copy_from_host_async(up, host_x)
            ev_in[b].record(up)
            h.stream.wait_event(ev_in[b])
            if i >= 2:
                h.stream.wait_event(ev_out[b])   # its output has left this output buffer
            if graphed:
                layer.replay(io=b)
            else:
                layer.forward(io=b)
            ev_done[b].record(h.stream)
            down.wait_event(ev_done[b])
            layer.out_bufs[b].copy_to_host_async(down, host_outs[b])
            ev_out[b].record(down)
        for st in (up, h.stream, down):
            st.synchronize()
    pipelined(2)
    h.barrier()
    n_pipe = 8
    t0 = time.perf_counter()
    pipelined(n_pipe)
    h.barrier()
    dtp = h.max_over_ranks((time.perf_counter() - t0) / n_pipe)
    same = bool(np.array_equal(host_outs[0], host_outs[1]))   # both buffer pairs carried the same tokens
    res["e2e_pipelined"] = {"value": T / dtp, "unit": "tokens/s", "ms_per_step": dtp * 1e3, "steps_in_flight": 2,
                            "h2d_bytes_per_step": 2 * t_local * d * h.world, "d2h_bytes_per_step": 4 * t_local * d * h.world,
                            "both_pairs_equal": same}
    if not same:
        raise SystemExit("pipelined end-to-end passes over the two buffer pairs disagree")
    if cpu:
        # Parity on EVERY rank: a strided sample of each rank's tokens (so rows that crossed NVLink in both
        # directions are covered) is gathered to rank 0 and checked there against the oracle.
        ns = 16 if h.world > 1 else 64
        idx = np.unique(np.linspace(0, t_local - 1, ns).astype(np.int64))
        ns = len(idx)
        out_rows = host_out.reshape(t_local, d)[idx]
        x_rows = np.ascontiguousarray(x.reshape(t_local, d)[idx])
        top2_rows = layer.top2.cpu().numpy().view(np.uint32).reshape(t_local, 2)[idx]
        if h.world > 1:
            def gather(a):   # bytes travel (NCCL has no 16-bit integer type); rank-major result in a's dtype
                a = np.ascontiguousarray(a)
                loc = torch.from_numpy(a.view(np.uint8).reshape(-1)).cuda()
                allr = torch.empty(h.world * loc.numel(), dtype=torch.uint8, device="cuda")
                torch.distributed.all_gather_into_tensor(allr, loc)
                return allr.cpu().numpy().view(a.dtype).reshape((h.world,) + a.shape)
            out_all, x_all, top2_all = gather(out_rows), gather(x_rows), gather(top2_rows)
        else:
            out_all, x_all, top2_all = out_rows[None], x_rows[None], top2_rows[None]
        if h.rank == 0:
            import oracle
            oracle.build()
            oracle.set_threads(os.cpu_count())
            if h.world == 1:
                w1_all, w2_all = w1, w2
            else:
                w1_all = np.concatenate([oracle.synth_normal_bf16(4, 100 + e, d * f, 0.02) for e in range(E)])
                w2_all = np.concatenate([oracle.synth_normal_bf16(4, 200 + e, f * d, 0.02) for e in range(E)])
            per_rank, all_ok, secs = [], True, 0.0
            for r in range(h.world):
                t0 = time.perf_counter()
                want_top2, want = moe_oracle_tokens(oracle, x_all[r].reshape(-1), wg, w1_all, w2_all, ns, d, f, E)
                secs += time.perf_counter() - t0
                got = out_all[r].reshape(ns, d)
                routing_ok = bool((top2_all[r].reshape(-1) == want_top2).all())
                err = np.abs(got - want) - (2e-3 * np.abs(want).max() + 2e-2 * np.abs(want))
                ok = routing_ok and bool(err.max() <= 0)
                all_ok = all_ok and ok
                per_rank.append({"rank": r, "tokens_checked": ns, "routing_bit_exact": routing_ok,
                                 "max_abs": float(np.abs(got - want).max()), "ok": ok})
            res["cpu_baseline"] = {"value": ns * h.world / secs, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                   "sample": f"{ns} tokens of each of {h.world} rank(s), spread over the rank's range, "
                                             "through gate, routing, FFN and combine"}
            res["parity"] = {"routing_bit_exact": all(p["routing_bit_exact"] for p in per_rank),
                             "max_abs": max(p["max_abs"] for p in per_rank), "tolerance": "2e-3*max|e| + 2e-2*|e|",
                             "per_rank": per_rank, "ok": all_ok}
            if not all_ok:
                raise SystemExit(f"moe_top2_v1 mismatch against the oracle: {per_rank}")
    if layer.exchange == "peer" and h.world > 1:
        h.barrier()
        layer.close()
    return res


def wl_scalar_gemm_512(h, steps, warmup, cpu=True):
    """BASELINE's first configuration taken literally: f32 C = A*B, M = N = K = 512, A and B uniform
    [-1, 1) from seed 0 (the scalar_gemm_v1 signature).  Single-launch latency, bit-exact against the
    full CPU oracle."""
    fe = h.fe
    from fe2o3_b200 import synth
    ctx, stream = h.ctx, h.stream
    peaks = measured_peaks()
    m = n = k = 512
    a_h, b_h = synth.uniform_f32(0, 1, m * k), synth.uniform_f32(0, 2, k * n)
    a, b = fe.DeviceBuffer.from_host(stream, a_h), fe.DeviceBuffer.from_host(stream, b_h)
    c = fe.DeviceBuffer.zeroed(stream, m * n, np.float32)
    flops = 2.0 * m * n * k
    res = {"workload": {"workload": "scalar_gemm_v1", "m": m, "n": n, "k": k, "dtype": "f32 in, f32 out",
                        "inputs": "uniform[-1,1) seed 0", "l2": "256 MiB L2 flush between launches"}}
    schedules = {}
    for name, sched in (("exact_order", fe.SCHEDULE_EXACT_ORDER), ("tcgen05_split_bf16", fe.SCHEDULE_TCGEN05)):
        try:
            prep = fe.prepare(ctx, "scalar_gemm_v1", schedule=sched, a=a, b=b, c=c, m=m, n=n, k=k)
        except fe.Fe2o3Error as err:
            schedules[name] = {"unavailable": str(err)}
            continue
        ms = h.time_steps(lambda: prep.launch(stream), max(5, min(steps, 20)), warmup, flush=True)
        lat = float(np.median(ms))
        schedules[name] = {"latency_us": lat * 1e3, "tflops": flops / (lat * 1e-3) / 1e12, "launches": prep.geometry.launches,
                           "result": c.to_host_vec(stream)}
    if ctx.take_kernel_status(stream):
        raise RuntimeError("scalar GEMM reported a kernel status word")
    exact = schedules["exact_order"]
    res.update({"ms_per_step": exact["latency_us"] / 1e3, "value": exact["tflops"], "unit": "TFLOP/s",
                "launches": exact["launches"],
                "roofline": {**roofline("tensor", exact["tflops"], peaks["bf16_tflops"], "TFLOP/s", peak_source=peaks["source"]),
                             "note": "exact-order schedule on CUDA cores (bit-identical to the sequential oracle); "
                                     "268 MFLOP in one launch is latency-bound, far from any throughput peak"}})
    host_a, host_b, host_c = ctx.pinned(m * k, np.float32), ctx.pinned(k * n, np.float32), ctx.pinned(m * n, np.float32)
    host_a[:], host_b[:] = a_h, b_h
    prep = fe.prepare(ctx, "scalar_gemm_v1", schedule=fe.SCHEDULE_EXACT_ORDER, a=a, b=b, c=c, m=m, n=n, k=k)

    def e2e_step():
        a.copy_from_host_async(stream, host_a)
        b.copy_from_host_async(stream, host_b)
        prep.launch(stream)
        c.copy_to_host_async(stream, host_c)
        stream.synchronize()
    e2e_step()
    t0 = time.perf_counter()
    for _ in range(10):
        e2e_step()
    dt = (time.perf_counter() - t0) / 10
    res["e2e"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": 4 * (m * k + k * n),
                  "d2h_bytes_per_step": 4 * m * n, "ms_per_step": dt * 1e3}
    if cpu:
        import oracle
        oracle.set_threads(os.cpu_count())
        t0 = time.perf_counter()
        want = oracle.gemm_f32(m, n, k, a_h, b_h, fast=True)
        dt = time.perf_counter() - t0
        bit_exact = bool((host_c.view(np.uint32) == np.asarray(want, np.float32).reshape(-1).view(np.uint32)).all())
        res["cpu_baseline"] = {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": "the full 512^3 product, sequential-k oracle parallel over rows"}
        res["parity"] = {"exact_order_bit_exact": bit_exact, "ok": bit_exact}
        split = schedules.get("tcgen05_split_bf16", {})
        if "result" in split:
            rel = float(np.abs(split["result"] - want.reshape(-1)).max() / np.abs(want).max())
            res["parity"]["tcgen05_split_bf16_max_err_over_max"] = rel
            res["parity"]["ok"] = bit_exact and rel <= 1e-4
        if not res["parity"]["ok"]:
            raise SystemExit(f"scalar_gemm_v1 512^3 mismatch: {res['parity']}")
    res["schedules"] = {k2: {kk: vv for kk, vv in v.items() if kk != "result"} for k2, v in schedules.items()}
    return res


WORKLOADS = {"masked_reduce_u32": wl_masked_reduce, "row_softmax_v1": wl_row_softmax, "tiled_gemm_v1": wl_gemm,
             "flash_attention_v1": wl_attention, "moe_top2_v1": wl_moe, "device_scan_u32": wl_scan,
             "scalar_gemm_v1_512": wl_scalar_gemm_512}
# secondary ops that also run when the bench has several GPUs (the sharded paths)
MULTI_GPU_OPS = ("tiled_gemm_v1",)
UNITS = {"masked_reduce_u32": ("masked u32 reduction throughput", "elements/s", "u32"),
         "moe_top2_v1": ("MoE top-2 layer throughput", "tokens/s", "bf16"),
         "tiled_gemm_v1": ("tiled GEMM throughput", "TFLOP/s", "bf16"),
         "flash_attention_v1": ("flash attention throughput", "TFLOP/s", "bf16"),
         "row_softmax_v1": ("row softmax bandwidth", "GB/s", "f32"),
         "device_scan_u32": ("device-wide u32 prefix sum throughput", "elements/s", "u32"),
         "scalar_gemm_v1_512": ("f32 GEMM 512^3 single-launch throughput", "TFLOP/s", "f32")}


def run_reference_arm(args):
    """The reference's CPU implementation of the headline workload (the oracle port:
    the reference is Rust and cannot be compiled here), all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    oracle.build()
    cores = oracle.set_threads(os.cpu_count())
    # inputs come from the oracle library's restatement of the benchmark generators: the GPU library is
    # not loaded on this arm
    if args.workload == "masked_reduce_u32":
        n = 1 << 28
        v = oracle.synth_u32_below(1, 1, n, 1 << 16)
        a = oracle.synth_bernoulli_flags(1, 2, n, 0.75, 7)
        step = lambda: oracle.masked_sum_u32(v, a, parallel=True)
        units, unit, dtype, scaling = n, "elements/s", "u32", "weak"
        config = {"workload": "masked_reduce_u32", "elements": n}
        sample = "the full 2^28-element workload per step"
    elif args.workload == "moe_top2_v1":
        T, d, f, E = (MOE_SHAPE[k] for k in ("tokens", "d_model", "d_ff", "experts"))
        sample_tokens = 128  # bounded sample of the 16384-token batch per step
        x = oracle.synth_normal_bf16(4, 1, sample_tokens * d, 1.0)   # a prefix of the batch's stream
        wg = oracle.synth_normal_bf16(4, 2, d * E, 0.02)
        w1 = np.concatenate([oracle.synth_normal_bf16(4, 100 + e, d * f, 0.02) for e in range(E)])
        w2 = np.concatenate([oracle.synth_normal_bf16(4, 200 + e, f * d, 0.02) for e in range(E)])

        def step():
            logits = oracle.moe_gate_logits(x, wg, sample_tokens, d, E)
            _, routing = oracle.moe_top2_route(logits, sample_tokens, E, 2 * sample_tokens)
            w = oracle.moe_route_weights(logits, routing["top2_experts"], sample_tokens, E)
            compact = oracle.moe_expert_ffn(x, w1, w2, routing["top2_experts"], routing["inverse"], sample_tokens, d, f, E)
            return oracle.moe_combine(compact, routing["inverse"], w, sample_tokens, d)
        units, unit, dtype, scaling = sample_tokens, "tokens/s", "bf16", "strong"
        config = {"workload": "moe_top2_v1", **MOE_SHAPE}
        sample = f"{sample_tokens} tokens of the batch per step through gate, routing, FFN and combine"
    else:
        emit({"impl": "reference", "unavailable": f"no CPU reference arm for workload {args.workload}"})
        return
    for _ in range(min(args.warmup, 3)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = units / dt
    emit({
        "impl": "reference", "metric": UNITS[args.workload][0], "value": val, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config,
        "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})


emit = None   # set by main(): writes the one JSON line to the process's real stdout


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=HEADLINE)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary ops in the `ops` object")
    ap.add_argument("--small", action="store_true", help="reduced sizes (profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-oracle leg (profiler captures)")
    ap.add_argument("--exchange", default="auto", choices=("auto", "peer", "nccl"),
                    help="moe_top2_v1: exchange between ranks; 'peer' on one GPU runs the expert-parallel kernels "
                         "(dispatch, flag-waiting FFN, scatter epilogue, combine) over the rank's own buffers")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    # stdout carries exactly one line, the JSON result: anything a library prints to file descriptor 1
    # while the bench runs (banners, warnings) goes to stderr instead
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)
    global emit

    def emit(obj):  # noqa: F811
        sys.stdout.flush()
        os.write(result_fd, (json.dumps(obj) + "\n").encode())
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout for the one JSON line
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    h = Harness(rank, world, local_rank)
    kw = {}
    if args.small:
        kw = {"masked_reduce_u32": {"n": 1 << 26}, "device_scan_u32": {"n": 1 << 26}, "row_softmax_v1": {"rows": 32768},
              "tiled_gemm_v1": {"m": 4096, "n": 4096, "k": 4096},
              "moe_top2_v1": {"tokens": 2048}}.get(args.workload, {})
    if args.no_cpu:
        kw["cpu"] = False
    if args.workload == "moe_top2_v1" and args.exchange != "auto":
        kw["exchange"] = args.exchange
    clocks = ClockSampler(local_rank)
    h.clocks = clocks
    res = WORKLOADS[args.workload](h, args.steps, args.warmup, **kw)
    h.clocks = None
    ops = {}
    if not args.no_extra and not args.small:
        for name, fn in WORKLOADS.items():
            if name == args.workload or (world > 1 and name not in MULTI_GPU_OPS):
                continue
            try:
                r = fn(h, min(args.steps, 10), args.warmup)
                ops[name] = {k: r[k] for k in ("value", "unit", "ms_per_step", "scaling", "roofline", "cpu_baseline", "parity",
                                               "e2e", "schedules", "workload")
                             if k in r}
            except Exception as e:  # a secondary op must not take the headline down
                ops[name] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0:
        metric, unit, dtype = UNITS.get(args.workload, (args.workload, res["unit"], "f32"))
        line = {"metric": metric, "value": res["value"], "unit": res["unit"], "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": res.get("scaling", "weak"), "vs_baseline": None, "dtype": dtype, "data": "synthetic",
                "config": res["workload"], "roofline": res["roofline"], "e2e": res.get("e2e"),
                "e2e_pipelined": res.get("e2e_pipelined"), "cpu_baseline": res.get("cpu_baseline"), "gpu_launches": res.get("launches", args.steps),
                "clocks": clocks.summary(), "parity": res.get("parity"), "ops": ops}
        emit(line)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
