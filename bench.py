#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line on stdout (rank 0).  A step is one pass of the hot path over one batch:
one GEMM launch per GPU (or one launch of a bandwidth kernel).  The headline workload is the
bf16 4096^3 GEMM with bf16 output; with N GPUs the problem is M-sharded -- every rank owns a
4096-row block of A and C, B is replicated, and no collective is on the compute path -- so
the job is ``[N*4096, 4096] = A . B^T`` and ``value`` is the whole job's TFLOP/s.

Headline timing: CUDA events on the launching stream around exactly K back-to-back steps, after
W >= 3 warm-up steps, bracketed by a barrier and a device synchronise, max over ranks.
Successive steps rotate over several operand sets whose total footprint exceeds the L2, so no
step finds its inputs cached by the previous one.  ``e2e`` repeats the measurement through the
host-buffer API (pinned host memory -> device -> host every step).  ``cpu_baseline`` and
``--impl reference`` time the reference's CPU computation of the same GEMM (numpy on
float32-upcast inputs) on this machine's cores.

Without ``--workload`` the line also carries, after the headline:

* ``sustained``: the headline kernel over a timed region of several hundred milliseconds, with
  the SM clocks NVML reported during it and the clock the kernel itself measured;
* ``workloads`` (one GPU only): every other configured problem -- fp16 512^3, bf16 8192^3, the
  fused 8192x8192x2048 GEMM, fp8 8192^3, the two decode shapes, vector_add and copy_2d_padded --
  timed by the reference's own protocol (100 launches, each between its own event pair and
  followed by a synchronise, the first 20 dropped, median; bench_harness.py:93-94,181-198 of
  the reference) and checked against the oracle;
* ``strong_65536``: the M = 65536, N = K = 8192 problem split by rows over the N GPUs, same
  protocol, with the all-gather of C timed apart.
"""

from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import math
import os
import re
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1000 * 1000
SM_COUNT = 148
FLOP_PER_CLK_PER_SM = {2: 8192.0, 1: 16384.0}  # dense tensor rate by operand width in bytes
REF_LAUNCHES, REF_DROP = 100, 20  # the reference's timing protocol (bench_harness.py:93-94)
SHORT_KERNEL_MS = 0.1  # below this a leg's headline figure comes from back-to-back launches

# name -> problem per GPU.  `dist`: distribution of A and B; seeds follow the configured ones
# (A from seed, B from seed + 1, bias from seed + 2).
WORKLOADS = {
    "bf16_4096": dict(M=4096, N=4096, K=4096, dtype_ab="bf16", dtype_c="bf16", dist="uniform", seed=1,
                      text="bf16 GEMM C=A.B^T M=N=K=4096 per GPU, U(-1,1) seed 1, fp32 accumulate, bf16 out"),
    "bf16_8192": dict(M=8192, N=8192, K=8192, dtype_ab="bf16", dtype_c="bf16", dist="uniform", seed=1,
                      text="bf16 GEMM M=N=K=8192 per GPU, U(-1,1) seed 1, bf16 out"),
    "fp16_512": dict(M=512, N=512, K=512, dtype_ab="f16", dtype_c="f32", dist="normal", seed=0,
                     text="fp16 GEMM M=N=K=512, N(0,1) seed 0, fp32 out"),
    "fused_8192x8192x2048": dict(M=8192, N=8192, K=2048, dtype_ab="bf16", dtype_c="bf16", dist="normal", seed=2, epilogue="bias_relu",
                                 text="bf16 GEMM [8192,2048].[8192,2048]^T + bias N(0,0.1), ReLU, bf16 out, N(0,1) seed 2"),
    "fp8_8192": dict(M=8192, N=8192, K=8192, dtype_ab="e4m3", dtype_c="bf16", dist="normal", seed=3,
                     text="fp8-e4m3 GEMM M=N=K=8192, per-tensor scales amax/448, N(0,1) seed 3, bf16 out"),
    "int8_8192": dict(M=8192, N=8192, K=8192, dtype_ab="i8", dtype_c="i32", dist="int8", seed=7,
                      text="int8 GEMM M=N=K=8192, integers in [-128,127] seed 7, exact int32 sums out (TFLOP/s reads as TOP/s)"),
    "mxfp8_8192": dict(M=8192, N=8192, K=8192, dtype_ab="mxe4m3", dtype_c="bf16", dist="normal", seed=8,
                       text="block-scaled fp8 GEMM M=N=K=8192 (e4m3 elements, one E8M0 scale per 32 elements of K, scales resident "
                            "on the device), N(0,1) seed 8, bf16 out"),
    "sharded_65536": dict(M=65536, N=8192, K=8192, dtype_ab="bf16", dtype_c="bf16", dist="uniform", seed=4, strong=True,
                          text="bf16 GEMM M=65536 N=K=8192 split by M rows over the GPUs, U(-1,1) seed 4"),
    "decode_16": dict(M=16, N=8192, K=8192, dtype_ab="bf16", dtype_c="bf16", dist="uniform", seed=4, tile_n=128, hbm=True, static_b=True, b_layout="packed",
                      text="bf16 skinny GEMM M=16 N=K=8192, U(-1,1) seed 4; B is the weight matrix: direct-B (packed once, outside "
                           "the timing) and static_b (its first tiles are requested while the previous launch drains)"),
    "decode_128": dict(M=128, N=8192, K=8192, dtype_ab="bf16", dtype_c="bf16", dist="uniform", seed=4, tile_n=128, hbm=True, static_b=True, b_layout="packed",
                       text="bf16 skinny GEMM M=128 N=K=8192, U(-1,1) seed 4; B is the weight matrix: direct-B (packed once) and static_b"),
    "vector_add": dict(n=1 << 28, text="int32 vector_add, 2^28 elements per array, integers from default_rng(5)"),
    "vector_add_64m": dict(n=1 << 26, text="int32 vector_add, 2^26 elements per array (profiling size), integers from default_rng(5)"),
    "copy_2d_padded_8k": dict(M=8192, N=8188, text="fp32 copy_2d_padded 8192x8188 (profiling size), standard normal from default_rng(6)"),
    "copy_2d_padded": dict(M=16384, N=16380, text="fp32 copy_2d_padded 16384x16380 (ragged last column tile), standard normal from default_rng(6)"),
}
DEFAULT_WORKLOAD = "bf16_4096"
# The other configured problems, measured after the headline by the default run on one GPU.
EXTRA_WORKLOADS = ("fp16_512", "bf16_8192", "fused_8192x8192x2048", "fp8_8192", "decode_16", "decode_128", "vector_add", "copy_2d_padded")


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


EIGHT_BIT = ("e4m3", "e5m2", "i8", "mxe4m3", "mxe5m2")  # operand types that run at twice the 16-bit tensor rate


def operands_f32(ops: dict, dtype_ab: str):
    """float32 values of the stored operands (block scales applied)."""
    from aster_b200.dtypes import dequantize_mx, to_f32

    if dtype_ab.startswith("mx"):
        return (dequantize_mx(ops["A"], ops["block_scales_a"], dtype_ab[2:]), dequantize_mx(ops["B"], ops["block_scales_b"], dtype_ab[2:]))
    return to_f32(ops["A"], dtype_ab), to_f32(ops["B"], dtype_ab)


def draw(rng, shape, dist):
    if dist == "uniform":
        return rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)
    if dist == "int8":
        return rng.integers(-128, 128, size=shape).astype(np.float32)
    return rng.standard_normal(size=shape).astype(np.float32)


def host_operands(w: dict, rank: int, rows: int):
    """Seeded synthetic A (this rank's rows), B, bias and scales in storage form."""
    from aster_b200.dtypes import from_f32, quantize_e4m3, quantize_mx
    from aster_b200.sharding import sharded_uniform_rows

    seed = w["seed"]
    if w.get("strong"):
        first = rank * rows
        a = sharded_uniform_rows(seed, first, rows, w["K"], threads=min(8, os.cpu_count() or 1))
    elif rank == 0:
        a = draw(np.random.default_rng(seed), (rows, w["K"]), w["dist"])
    else:
        a = draw(np.random.default_rng([seed, rank]), (rows, w["K"]), w["dist"])
    b = draw(np.random.default_rng(seed + 1), (w["N"], w["K"]), w["dist"])
    out = dict(scale_a=None, scale_b=None, bias=None, block_scales_a=None, block_scales_b=None)
    if w["dtype_ab"].startswith("mx"):
        out["A"], out["block_scales_a"] = quantize_mx(a, w["dtype_ab"][2:])
        out["B"], out["block_scales_b"] = quantize_mx(b, w["dtype_ab"][2:])
    elif w["dtype_ab"] == "e4m3":
        out["A"], sa = quantize_e4m3(a)
        out["B"], sb = quantize_e4m3(b)
        out["scale_a"], out["scale_b"] = float(sa), float(sb)
    else:
        out["A"], out["B"] = from_f32(a, w["dtype_ab"]), from_f32(b, w["dtype_ab"])
    if w.get("epilogue") == "bias_relu":
        out["bias"] = (np.random.default_rng(seed + 2).standard_normal(w["N"]) * 0.1).astype(np.float32)
    return out


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML (read-only) while the
    measurement runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, device: int):
        self.samples = []  # (t, sm_mhz, reasons_mask, power_w)
        self.max_mhz = None
        self.power_limit_w = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            from aster_b200 import _native as nat

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByPciBusId(nat.device_pci_bus_id(device).encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            try:  # read only: the limit the board enforces on itself
                self.power_limit_w = pynvml.nvmlDeviceGetEnforcedPowerLimit(self._h) / 1000.0
            except Exception:
                self.power_limit_w = None
        except Exception as e:  # NVML missing: report no clocks rather than guess
            log(f"clock sampling unavailable: {e}")

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                try:
                    power = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                except Exception:
                    power = None
                self.samples.append((time.perf_counter(), mhz, mask, power))
            except Exception:
                pass
            self._stop.wait(0.002)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
            deadline = time.perf_counter() + 2.0
            while not self.samples and time.perf_counter() < deadline:  # one reading before any timing starts
                time.sleep(0.001)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float) -> dict:
        if self._h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        window = "timed region"
        if not inside:  # region shorter than one NVML read: nearest samples around it
            window = "nearest samples around the timed region"
            inside = sorted(self.samples, key=lambda s: min(abs(s[0] - t0), abs(s[0] - t1)))[:3]
        mask = 0
        for s in inside:
            mask |= s[2]
        powers = [s[3] for s in inside if s[3] is not None]
        mhz = [s[1] for s in inside]
        return {
            "sm_mhz": float(np.median(mhz)) if inside else None,
            "sm_mhz_min": float(min(mhz)) if inside else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(name for bit, name in self.REASONS.items() if mask & bit),
            "power_w_max": max(powers) if powers else None,
            "power_limit_w": self.power_limit_w,
            "samples": len(inside),
            "window": window,
        }


# ---------------------------------------------------------------------------------------------
# distributed plumbing (torch.distributed only for barrier / reductions)
# ---------------------------------------------------------------------------------------------
class Job:
    def __init__(self, gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1 or "TORCHELASTIC_RUN_ID" in os.environ:  # any torchrun launch, also with one rank
            import torch
            import torch.distributed as dist

            torch.cuda.set_device(self.local_rank)
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # NCCL may announce its version on stdout while the communicator comes up; stdout
            # is reserved for the one JSON line, so it is pointed at stderr until then.
            sys.stdout.flush()
            saved = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
                dist.barrier()
                torch.cuda.synchronize()
            finally:
                sys.stdout.flush()
                os.dup2(saved, 1)
                os.close(saved)
            self.dist, self.torch = dist, torch
        elif gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def _reduce(self, x: float, op) -> float:
        if self.dist is None:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(self, x: float) -> float:
        return self._reduce(x, self.dist.ReduceOp.MAX) if self.dist is not None else x

    def all_ranks_true(self, flag: bool) -> bool:
        """True only when `flag` is true on every rank."""
        return self._reduce(1.0 if flag else 0.0, self.dist.ReduceOp.MIN) > 0.5 if self.dist is not None else bool(flag)

    def gather_floats(self, x: float) -> list:
        """The value of every rank, in rank order (on every rank)."""
        if self.dist is None:
            return [float(x)]
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        out = self.torch.empty(self.world, dtype=self.torch.float64, device="cuda")
        self.dist.all_gather_into_tensor(out, t)
        return [float(v) for v in out.tolist()]

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU computation of the path (numpy on float32-upcast inputs)
# ---------------------------------------------------------------------------------------------
def cpu_gemm_seconds(w: dict, rows: int, max_seconds: float, max_reps: int):
    """Times ``oracle.gemm`` (bench_harness.py:821 of the reference: ``A.f32 @ B.f32.T``, plus
    the epilogue) on at most ``rows`` rows of the per-GPU problem.  Returns (best seconds,
    reps, rows used)."""
    from oracle import gemm_oracle as orc

    use_all_host_threads()
    rows = min(rows, w["M"])
    ops = host_operands(w, 0, rows)
    a32, b32 = operands_f32(ops, w["dtype_ab"])
    alpha = 1.0 if ops["scale_a"] is None else float(np.float32(ops["scale_a"]) * np.float32(ops["scale_b"]))
    best, reps, t_start = float("inf"), 0, time.perf_counter()
    while reps < max_reps and (reps == 0 or time.perf_counter() - t_start < max_seconds):
        t0 = time.perf_counter()
        acc = a32 @ b32.T  # upcast excluded from the timing, as in the reference's verify loop
        out = orc.encode(orc.gemm_epilogue(acc, ops["bias"], w.get("epilogue") == "bias_relu", "n", alpha), w["dtype_c"])
        best = min(best, time.perf_counter() - t0)
        reps += 1
    del out
    return best, reps, rows


def use_all_host_threads() -> None:
    """Let the BLAS behind numpy use every core (torchrun pins OMP_NUM_THREADS=1 for its
    children; the reference's bench scripts set the thread count to all cores,
    bench_perf_102_gemm_python_multitile_lds_cdna3.py:24-25)."""
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        pass


def cpu_threads() -> int:
    try:
        from threadpoolctl import threadpool_info

        n = [p.get("num_threads") for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return os.cpu_count() or 1


def common_config(w: dict, name: str, world: int) -> dict:
    """The `config` object, identical for both arms: what is computed, not how."""
    rows = w["M"] // world if w.get("strong") else w["M"]
    return {"workload": w["text"], "name": name, "per_gpu_shape": [rows, w["N"], w["K"]], "global_rows": rows * world,
            "parallelism": f"m-row shards x{world}, B replicated, no collective"}


def run_reference_arm(args, w: dict, name: str) -> dict:
    """--impl reference: every step is the numpy GEMM on a bounded row sample."""
    use_all_host_threads()
    cores = cpu_threads()
    if "K" not in w:
        return {"impl": "reference", "unavailable": "bandwidth workloads have no reference arm here; use the GEMM workloads"}
    # Size the sample so the whole run stays within a couple of minutes.
    probe_rows = min(w["M"], 512)
    t_probe, _, _ = cpu_gemm_seconds(w, probe_rows, 1.0, 1)
    budget = 90.0 / max(1, args.steps + args.warmup)
    rows = int(min(w["M"], max(128, probe_rows * budget / max(t_probe, 1e-6)) // 128 * 128)) or min(w["M"], 128)
    from oracle import gemm_oracle as orc

    ops = host_operands(w, 0, rows)
    a32, b32 = operands_f32(ops, w["dtype_ab"])
    alpha = 1.0 if ops["scale_a"] is None else float(np.float32(ops["scale_a"]) * np.float32(ops["scale_b"]))

    def step():
        acc = a32 @ b32.T
        return orc.encode(orc.gemm_epilogue(acc, ops["bias"], w.get("epilogue") == "bias_relu", "n", alpha), w["dtype_c"])

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    flops = 2.0 * rows * w["N"] * w["K"]
    value = flops * args.steps / dt / 1e12
    sample = f"{rows} of {w['M']} rows of A per step (full B), numpy float32 matmul + epilogue, {args.steps} steps"
    return {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w["dtype_ab"], "data": "synthetic", "impl": "reference",
        "config": common_config(w, name, max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ---------------------------------------------------------------------------------------------
# timing
# ---------------------------------------------------------------------------------------------
class Timed(tuple):
    """(max-over-ranks ms, this rank's ms, host t0, host t1) with ``sm_mhz``: the average SM clock
    of the timed launches as the kernels themselves counted it (0 when no plan was given)."""

    sm_mhz = 0.0


def time_steps(job: Job, run_step, steps: int, warmup: int, plan=None):
    """W warm-up steps, then K steps between two events on the default stream; returns
    (max-over-ranks milliseconds for the K steps, this rank's milliseconds, host t0, host t1).
    With ``plan`` the result's ``sm_mhz`` is the SM clock averaged over exactly the K timed
    launches (the plan's cycle and nanosecond totals are read before and after them)."""
    from aster_b200 import _native as nat
    from aster_b200.execution import GpuEvent
    from aster_b200.gemm import mean_sm_mhz

    for i in range(warmup):
        run_step(i)
    nat.call("b200_device_synchronize")
    before = plan.clock_totals() if plan is not None else None
    job.barrier()
    e0, e1 = GpuEvent(), GpuEvent()
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        run_step(warmup + i)
    e1.record()
    e1.synchronize()
    nat.call("b200_device_synchronize")
    t1 = time.perf_counter()
    job.barrier()
    ms = e1.elapsed_ms(e0)
    out = Timed((job.max_over_ranks(ms), ms, t0, t1))
    if plan is not None:
        out.sm_mhz = mean_sm_mhz(before, plan.clock_totals())
    return out


def time_reference_protocol(run_step, launches: int = REF_LAUNCHES, drop: int = REF_DROP, plan=None) -> dict:
    """The reference's protocol (python/aster/execution/core.py:698-703 and
    bench_harness.py:93-94,181-198): every launch between its own pair of events and followed
    by a synchronise; the first `drop` are warm-up; statistics over the rest, in ms.  With
    ``plan``, ``sm_mhz`` is the SM clock averaged over the kept launches."""
    from aster_b200.execution import GpuEvent
    from aster_b200.gemm import mean_sm_mhz

    e0, e1 = GpuEvent(), GpuEvent()
    times = []
    before = None
    for i in range(launches):
        if i == drop and plan is not None:
            before = plan.clock_totals()
        e0.record()
        run_step(i)
        e1.record()
        e1.synchronize()
        times.append(e1.elapsed_ms(e0))
    sm_mhz = mean_sm_mhz(before, plan.clock_totals()) if before is not None else 0.0
    kept = np.sort(np.asarray(times[drop:], dtype=np.float64))
    pct = lambda q: float(kept[min(len(kept) - 1, int(q * len(kept)))])  # noqa: E731
    return {"launches": launches, "dropped": drop, "p50_ms": pct(0.5), "p0_ms": float(kept[0]), "p10_ms": pct(0.1), "p90_ms": pct(0.9),
            "mean_ms": float(kept.mean()), "stddev_ms": float(kept.std()), "sm_mhz": sm_mhz}


# ---------------------------------------------------------------------------------------------
# GEMM problems resident on the device
# ---------------------------------------------------------------------------------------------
class GemmCase:
    """One workload on one GPU: plan, rotating operand sets larger than the L2, launchers."""

    def __init__(self, w: dict, rank: int, world: int):
        from aster_b200 import _native as nat
        from aster_b200.dtypes import STORAGE
        from aster_b200.execution import GpuBuffer
        from aster_b200.gemm import GemmPlan

        self.w = w
        self.rows = rows = w["M"] // world if w.get("strong") else w["M"]
        self.N, self.K = N, K = w["N"], w["K"]
        self.plan_kw = {k: w[k] for k in ("epilogue", "split_k", "tile_n", "static_b", "b_layout", "stages", "workspace_exchange", "raster_group") if k in w}
        self.plan = plan = GemmPlan(rows, N, K, w["dtype_ab"], w["dtype_c"], **self.plan_kw)
        self.res = res = plan.resources()
        self.ops = ops = host_operands(w, rank, rows)
        self.eb_c = np.dtype(STORAGE[w["dtype_c"]]).itemsize
        self.eb_ab = ops["A"].itemsize
        self.set_bytes = ops["A"].nbytes + ops["B"].nbytes + rows * N * self.eb_c
        self.n_sets = min(max(2, -(-int(1.5 * L2_BYTES) // self.set_bytes)), 64)
        self.sets = []
        for _ in range(self.n_sets):
            dA, dB, dC = GpuBuffer(ops["A"].nbytes), GpuBuffer(ops["B"].nbytes), GpuBuffer(rows * N * self.eb_c)
            dA.copy_from_host(ops["A"])
            dB.copy_from_host(ops["B"])
            if plan.direct_b:
                # Direct-B: the weight matrix is packed once, outside the timing, as the reference
                # preshuffles B on the host before its timed loop (bench_harness.py:567-574).
                packed = GpuBuffer(res.packed_b_bytes)
                plan.pack_b(dB, packed)
                nat.call("b200_device_synchronize")
                dB.free()
                dB = packed
            self.sets.append((dA, dB, dC))
        self.small = {}
        for key in ("bias", "scale_a", "scale_b"):
            if ops[key] is not None:
                arr = np.atleast_1d(np.asarray(ops[key], dtype=np.float32))
                self.small[key] = GpuBuffer(arr.nbytes)
                self.small[key].copy_from_host(arr)
        ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
        self.ws = GpuBuffer(ws_bytes) if ws_bytes else None
        if ops["block_scales_a"] is not None:
            from aster_b200.gemm import mx_scales_bytes, pack_mx_scales

            for key, n_rows in (("block_scales_a", rows), ("block_scales_b", N)):
                raw = GpuBuffer(ops[key].nbytes)
                raw.copy_from_host(ops[key])
                self.small[key] = GpuBuffer(mx_scales_bytes(n_rows, K))
                pack_mx_scales(raw, self.small[key], n_rows, K)
                nat.call("b200_device_synchronize")
                raw.free()
            plan.set_mx_scales(self.small["block_scales_a"], self.small["block_scales_b"])
        small = self.small
        self.bound = [plan.bind(dA, dB, dC, small.get("bias"), small.get("scale_a"), small.get("scale_b"), self.ws) for dA, dB, dC in self.sets]
        self.launches_per_step = 2 if res.split_k > 1 else 1

    def run_step(self, i: int) -> None:
        self.bound[i % self.n_sets]()

    @property
    def flops(self) -> float:
        return 2.0 * self.rows * self.N * self.K

    @property
    def algorithmic_bytes(self) -> float:
        return (self.rows * self.K + self.N * self.K) * self.eb_ab + self.rows * self.N * self.eb_c

    def result(self, set_index: int) -> np.ndarray:
        from aster_b200.dtypes import STORAGE

        out = np.empty((self.rows, self.N), dtype=STORAGE[self.w["dtype_c"]])
        self.sets[set_index % self.n_sets][2].copy_to_host(out)
        return out

    def verify(self, out: np.ndarray, sample_rows: int = 64) -> dict:
        """This rank's result against the oracle on a sample of rows, with the tolerances the
        parity tests use: max |err| <= 2e-3 * sqrt(K) * max|a| * max|b| on fp32 outputs; one bf16
        spacing at the oracle's magnitude plus the summation-order allowance on bf16 outputs;
        2 % relative Frobenius error for scaled and block-scaled fp8 against the oracle on the same
        quantised inputs; equality for integer sums."""
        from oracle import gemm_oracle as orc

        w, ops = self.w, self.ops
        pick = np.sort(np.random.default_rng(0).choice(self.rows, min(self.rows, sample_rows), replace=False))
        sub = dict(ops, A=ops["A"][pick], block_scales_a=None if ops["block_scales_a"] is None else ops["block_scales_a"][pick])
        got = out[pick]
        relu = w.get("epilogue") == "bias_relu"
        if w["dtype_ab"] == "i8":
            want = orc.gemm_i32(sub["A"], ops["B"])
            return {"ok": bool(np.array_equal(got, want)), "criterion": "int32 sums equal", "rows": int(len(pick))}
        a32, b32 = operands_f32(sub, w["dtype_ab"])
        alpha = 1.0 if ops["scale_a"] is None else float(np.float32(ops["scale_a"]) * np.float32(ops["scale_b"]))
        want = orc.gemm_epilogue(a32 @ b32.T, ops["bias"], relu, "n", alpha)
        amax = float(np.abs(a32).max()) * float(np.abs(b32).max())
        if w["dtype_ab"] in EIGHT_BIT:
            want_c = orc.decode(orc.encode(want, w["dtype_c"]), w["dtype_c"])
            rel = orc.rel_frobenius(orc.decode(got, w["dtype_c"]), want_c)
            return {"ok": bool(rel <= 0.02), "criterion": "relative Frobenius error <= 2% vs oracle on the same quantised inputs", "value": rel,
                    "rows": int(len(pick))}
        if w["dtype_c"] == "f32":
            bound = 2e-3 * math.sqrt(self.K) * amax * abs(alpha)
            err = float(np.max(np.abs(got - want)))
            return {"ok": bool(err <= bound), "criterion": "max|err| <= 2e-3*sqrt(K)*max|a|*max|b|", "value": err, "bound": bound, "rows": int(len(pick))}
        slack = 1e-6 * self.K * amax * abs(alpha)
        excess = orc.bf16_output_error(got, want, slack)
        return {"ok": bool(excess <= 0.0), "criterion": "|bf16 out - oracle f32| <= one bf16 spacing + 1e-6*K*max|a|*max|b|", "value": excess,
                "rows": int(len(pick))}

    def free(self) -> None:
        for dA, dB, dC in self.sets:
            dA.free(), dB.free(), dC.free()
        for b in self.small.values():
            b.free()
        if self.ws is not None:
            self.ws.free()
        self.plan.destroy()


def roofline_of(case: GemmCase, ms: float, sustained: bool, sm_mhz: float | None) -> dict:
    """Roofline object of one GEMM launch of `ms` milliseconds."""
    peaks = measured_peaks()
    w = case.w
    eight = w["dtype_ab"] in EIGHT_BIT
    if w.get("hbm"):
        achieved = case.algorithmic_bytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": f"{peaks['_source']} (hbm copy)", "frac_of_nominal": achieved / 8000.0}
    achieved = case.flops / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    if eight:
        peak *= 2.0  # no measured 8-bit figure: twice the measured bf16 cuBLAS rate
    kind = ("sustained" if sustained else "burst") + (" bf16 x2 for 8-bit inputs" if eight else " bf16")
    out = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
           "peak_source": f"{peaks['_source']} ({kind})", "frac_of_nominal": achieved / (4500.0 if eight else 2250.0)}
    if sm_mhz:
        # The tensor pipes' own ceiling at the clock the launch really ran at: SMs x flop/clk x MHz.
        clock_peak = SM_COUNT * FLOP_PER_CLK_PER_SM[1 if eight else 2] * sm_mhz * 1e6 / 1e12
        out["sm_mhz_in_kernel"] = sm_mhz  # SM cycles / nanoseconds counted by the timed launches themselves
        out["frac_of_clock_peak"] = achieved / clock_peak
        out["clock_note"] = "clock of the SM that ran CTA 0; the SMs of one launch differ by up to 4 %, so can the fraction"
    return out


def kernel_source_digest() -> str:
    """Digest of the GEMM kernel sources: a DRAM-traffic figure captured under the profiler is
    only quoted while the kernel is still the one that was captured."""
    h = hashlib.sha256()
    for name in ("gemm_kernel.cuh", "ptx_sm100.cuh", "gemm_sm100.cu", "bandwidth.cu"):
        with open(os.path.join(ROOT, "aster_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def dram_traffic(name: str) -> dict:
    """Per-launch DRAM bytes (read + write) of the workload's dominant kernel from the profiler
    summaries under profiles/ ("traffic-record:" lines), or null when there is no capture or
    the kernel sources have changed since it was taken."""
    digest = kernel_source_digest()
    pdir = os.path.join(ROOT, "profiles")
    stale = None
    for fn in sorted(os.listdir(pdir)) if os.path.isdir(pdir) else []:
        if not fn.endswith((".md", ".txt")):
            continue
        with open(os.path.join(pdir, fn)) as f:
            for line in f:
                m = re.match(r"\s*traffic-record:\s+workload=(\S+)\s+dram_bytes_per_launch=(\S+)\s+kernel_sources=(\S+)", line)
                if m and m.group(1) == name:
                    if m.group(3) == digest:
                        return {"traffic": float(m.group(2)), "traffic_source": f"profiles/{fn} (kernel sources {digest})"}
                    stale = f"profiles/{fn} was captured on kernel sources {m.group(3)}; they are now {digest}"
    return {"traffic": None, "traffic_source": stale or "no profiler capture for this workload"}


# ---------------------------------------------------------------------------------------------
# legs
# ---------------------------------------------------------------------------------------------
def time_allgather(job: Job, dC, rows: int, N: int, warmups: int = 3, reps: int = 20) -> dict:
    """The optional exchange, timed apart from the compute: NCCL all-gather of the bf16 C row
    shards into the full C on every rank (not part of `value`).  Each repetition is timed on the
    device; the figures are maxima over ranks of the per-rank minimum and median."""
    import torch

    from aster_b200 import _native as nat
    from aster_b200.sharding import allgather_rows

    shard = torch.empty((rows, N), dtype=torch.bfloat16, device="cuda")
    nat.call("b200_memcpy_d2d", C.c_void_p(shard.data_ptr()), dC.ptr, rows * N * 2)
    M_total = rows * job.world
    for _ in range(warmups):  # the first calls also build the communicator's channels
        full = allgather_rows(shard, M_total)
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        job.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        full = allgather_rows(shard, M_total)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms_min = job.max_over_ranks(float(np.min(times)))
    ms_med = job.max_over_ranks(float(np.median(times)))
    mine = full[job.rank * rows:(job.rank + 1) * rows]
    recv = (job.world - 1) * rows * N * 2
    return {"ms": ms_med, "ms_min": ms_min, "ms_max": job.max_over_ranks(float(np.max(times))), "warmups": warmups, "repetitions": reps,
            "recv_bytes_per_rank": recv, "recv_gbs_per_rank": recv / (ms_med * 1e-3) / 1e9, "recv_gbs_per_rank_best": recv / (ms_min * 1e-3) / 1e9,
            "own_shard_intact": job.all_ranks_true(bool(torch.equal(mine, shard))), "full_rows": int(full.shape[0])}


def run_e2e(args, job: Job, case: GemmCase, out_device: np.ndarray) -> dict:
    """End to end through the host-buffer API: pinned host -> device -> pinned host every step.
    (A direct-B workload runs this leg with a row-major twin of its plan: B arrives from the host
    every step.)  With several GPUs every rank uploads its rows of A and only its share of the
    replicated B; an all-gather over NVLink rebuilds B on every GPU."""
    from aster_b200.gemm import GemmPlan, HostGemmPipeline
    from aster_b200.sharding import ShardedHostGemmPipeline, bind_to_gpu_numa_node

    w, ops, plan = case.w, case.ops, case.plan
    numa = bind_to_gpu_numa_node(job.local_rank) if job.dist is not None else None
    if plan.direct_b or case.plan_kw.get("static_b"):  # B arrives from the host every step here: neither packed nor static
        plan = GemmPlan(case.rows, case.N, case.K, w["dtype_ab"], w["dtype_c"], **{k: v for k, v in case.plan_kw.items() if k not in ("b_layout", "static_b")})
    kw = dict(depth=2, bias=ops["bias"], scale_a=ops["scale_a"], scale_b=ops["scale_b"])
    sharded_b = job.dist is not None and job.world > 1 and case.N % job.world == 0
    pipe = ShardedHostGemmPipeline(plan, job.rank, job.world, **kw) if sharded_b else HostGemmPipeline(plan, **kw)
    hA, hB = pipe.pinned_operands()
    hA.array[...] = ops["A"]
    hB.array[...] = ops["B"][pipe.b_row_slice] if sharded_b else ops["B"]
    e2e_steps = max(2, min(args.steps, 200))
    for _ in range(3):
        pipe.submit(hA, hB)
    pipe.drain()
    job.barrier()
    te0 = time.perf_counter()
    for _ in range(e2e_steps):
        pipe.submit(hA, hB)
    pipe.drain()
    te_rank = time.perf_counter() - te0
    te = job.max_over_ranks(te_rank)
    ok = bool(np.array_equal(pipe.result(0), out_device)) if not w.get("hbm") else True
    h2d, d2h = pipe.h2d_bytes_per_problem, pipe.d2h_bytes_per_problem
    pipe.close()
    hA.free(), hB.free()
    total_flops = case.flops * job.world
    out = {"value": total_flops * e2e_steps / te / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "steps": e2e_steps, "matches_device_result": job.all_ranks_true(ok),
           "host_gbs_aggregate": (h2d + d2h) * job.world * e2e_steps / te / 1e9}
    if job.dist is not None:
        out["b_upload"] = (f"each rank uploads {case.N // job.world} of {case.N} rows of B, NCCL all-gather rebuilds B on the device" if sharded_b
                           else "every rank uploads all of B")
        out["per_rank_ms_per_step"] = [t * 1e3 / e2e_steps for t in job.gather_floats(te_rank)]
        out["numa_node_per_rank"] = job.gather_floats(-1.0 if numa is None else float(numa))
        out["limiter"] = "PCIe upload of A and B and download of C on every rank; aggregate limited by the host memory of the NUMA nodes the ranks' pinned buffers live on"
    return out


def run_gemm(args, job: Job, w: dict, name: str) -> tuple:
    """The headline leg: returns (JSON line, its GemmCase still resident)."""
    from aster_b200 import _native as nat

    world = job.world
    case = GemmCase(w, job.rank, world)
    res, plan, rows, N, K = case.res, case.plan, case.rows, case.N, case.K
    sampler = ClockSampler(job.local_rank)
    sampler.start()
    launches0 = nat.launch_count()
    timed = time_steps(job, case.run_step, args.steps, args.warmup, plan=plan)
    ms_total, ms_rank, t0, t1 = timed
    launches = (nat.launch_count() - launches0) - args.warmup * case.launches_per_step
    plan.status()
    mhz = timed.sm_mhz  # averaged over the K timed launches
    clocks = sampler.summary(t0, t1)

    out = case.result(args.warmup + args.steps - 1)
    check = case.verify(out)
    verified = job.all_ranks_true(check["ok"])
    e2e = run_e2e(args, job, case, out)
    sampler.stop()

    ms_per_step = ms_total / args.steps
    value = case.flops * world / (ms_per_step * 1e-3) / 1e12
    roof = roofline_of(case, ms_per_step, sustained=ms_total > 1000.0, sm_mhz=mhz or None)
    roof.update(dram_traffic(name))
    if w.get("hbm"):
        roof["frac_of_nominal"] = roof["achieved"] / 8000.0
    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if w.get("strong") else "weak",
        "vs_baseline": None, "dtype": w["dtype_ab"], "data": "synthetic", "impl": "ours",
        "config": common_config(w, name, world),
        "plan": {
            "tile": [res.tile_m, res.tile_n, res.tile_k], "stages": res.stages, "split_k": res.split_k, "grid_ctas": res.grid_ctas,
            "cta_group": res.cta_group, "tail_split": [res.tail_tiles, res.tail_parts],
            "tail_exchange": {0: "none", 1: "workspace", 2: "cluster shared memory"}[res.tail_exchange], "b_layout": plan.b_layout,
            "l2": f"rotating {case.n_sets} operand sets ({case.n_sets * case.set_bytes / 2**20:.0f} MiB) > {L2_BYTES / 1e6:.0f} MB L2",
        },
        "roofline": roof,
        "e2e": e2e,
        "gpu_launches": launches,
        "clocks": clocks,
        "verified": verified, "verify": check,
    }
    if job.dist is not None:
        line["per_rank"] = {"ms_per_step": [t / args.steps for t in job.gather_floats(ms_rank)], "sm_mhz_in_kernel": job.gather_floats(mhz),
                            "note": "value uses the slowest rank's time; in-kernel MHz = SM cycles / ns of CTA 0, summed over the timed launches"}
        if w["dtype_c"] == "bf16":
            line["allgather"] = time_allgather(job, case.sets[0][2], rows, N)
    if world == 1 and job.rank == 0 and not args.no_cpu_baseline:
        secs, reps, used = cpu_gemm_seconds(w, rows, 12.0, 5)
        line["cpu_baseline"] = {
            "value": 2.0 * used * N * K / secs / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
            "sample": f"{used} of {rows} rows, best of {reps} runs of numpy float32 matmul + epilogue ({secs:.3f} s)",
        }
    return line, case


def run_sustained(job: Job, case: GemmCase, ms_hint: float, target_ms: float = 400.0) -> dict:
    """The headline kernel over a region long enough for the power cap to settle and for NVML
    to be sampled many times: back-to-back launches for about `target_ms`, scored against the
    sustained cuBLAS figure."""
    steps = int(min(20000, max(50, target_ms / max(ms_hint, 1e-3))))
    sampler = ClockSampler(job.local_rank)
    sampler.start()
    timed = time_steps(job, case.run_step, steps, 3, plan=case.plan)
    ms_total, ms_rank, t0, t1 = timed
    case.plan.status()
    mhz = timed.sm_mhz
    clocks = sampler.summary(t0, t1)
    sampler.stop()
    inside = [s[1] for s in sampler.samples if t0 <= s[0] <= t1]
    ms = ms_total / steps
    roof = roofline_of(case, ms, sustained=True, sm_mhz=mhz or None)
    out = {"steps": steps, "timed_region_ms": ms_total, "ms_per_step": ms, "tflops_per_gpu": case.flops / (ms * 1e-3) / 1e12,
           "roofline": roof, "clocks": clocks}
    if inside:
        # Seen by NVML during the region: how the samples spread, and the same fraction against the
        # median sampled clock.
        med = float(np.median(inside))
        out["nvml_sm_mhz_quartiles"] = [float(np.percentile(inside, q)) for q in (0, 25, 50, 75, 100)]
        eight = case.w["dtype_ab"] in EIGHT_BIT
        out["frac_of_nvml_clock_peak"] = out["tflops_per_gpu"] / (SM_COUNT * FLOP_PER_CLK_PER_SM[1 if eight else 2] * med * 1e6 / 1e12)
    if job.dist is not None:
        out["per_rank_ms_per_step"] = [t / steps for t in job.gather_floats(ms_rank)]
    return out


def run_gemm_leg(job: Job, w: dict, name: str, launches: int = REF_LAUNCHES, drop: int = REF_DROP, back_to_back: int = 50) -> dict:
    """One configured GEMM by the reference's protocol (p50 of synchronised launches), plus a
    back-to-back figure, the in-kernel clock and the oracle check."""
    from aster_b200 import _native as nat

    t_setup = time.perf_counter()
    case = GemmCase(w, job.rank, job.world)
    res = case.res
    try:
        for i in range(3):
            case.run_step(i)
        nat.call("b200_device_synchronize")
        l0 = nat.launch_count()
        stats = time_reference_protocol(case.run_step, launches, drop, plan=case.plan)
        case.plan.status()
        mhz = stats["sm_mhz"]
        n_launched = nat.launch_count() - l0
        if stats["p50_ms"] < SHORT_KERNEL_MS:
            back_to_back = max(back_to_back, 300)  # a longer train for kernels of a few tens of microseconds
        timed = time_steps(job, case.run_step, back_to_back, 3, plan=case.plan)
        ms_b2b_all = timed[0]
        case.plan.status()
        mhz_b2b = timed.sm_mhz
        out = case.result(3 + back_to_back - 1)
        check = case.verify(out)
        p50 = job.max_over_ranks(stats["p50_ms"])
        ms_b2b = ms_b2b_all / back_to_back
        # A launch shorter than 100 us is mostly launch and synchronisation latency under the
        # reference's protocol (an event pair and a synchronise around every launch); its kernel time
        # is what back-to-back launches show, so that figure leads there and the other is kept beside it.
        short = p50 < SHORT_KERNEL_MS
        ms = ms_b2b if short else p50
        roof = roofline_of(case, ms, sustained=False, sm_mhz=(mhz_b2b if short else mhz) or None)
        roof.update(dram_traffic(name))
        leg = {
            "workload": w["text"], "per_gpu_shape": [case.rows, case.N, case.K], "dtype": w["dtype_ab"],
            "ms_per_step": ms,
            "timing": (f"{back_to_back} back-to-back launches between one event pair (the kernel is shorter than {SHORT_KERNEL_MS * 1e3:.0f} us, where the "
                       "reference protocol measures launch latency)" if short else
                       f"reference protocol: {launches} launches, each between its own event pair and synchronised, first {drop} dropped, median"),
            "reference_protocol": dict(stats, achieved=roofline_of(case, p50, False, mhz or None)["achieved"]),
            "achieved": roof["achieved"], "unit": roof["unit"],
            "tflops_total": case.flops * job.world / (ms * 1e-3) / 1e12,
            "roofline": roof,
            "back_to_back": {"steps": back_to_back, "ms_per_step": ms_b2b, "sm_mhz_in_kernel": mhz_b2b,
                             "achieved": roofline_of(case, ms_b2b, False, mhz_b2b or None)["achieved"]},
            "sm_mhz_in_kernel": mhz,
            "plan": {"tile": [res.tile_m, res.tile_n, res.tile_k], "stages": res.stages, "grid_ctas": res.grid_ctas, "cta_group": res.cta_group,
                     "tail_split": [res.tail_tiles, res.tail_parts], "tail_exchange": res.tail_exchange, "b_layout": case.plan.b_layout,
                     "operand_sets": case.n_sets},
            "gpu_launches": n_launched,
            "verified": job.all_ranks_true(check["ok"]), "verify": check,
        }
        if job.dist is not None:
            leg["per_rank_p50_ms"] = job.gather_floats(stats["p50_ms"])
            leg["per_rank_sm_mhz_in_kernel"] = job.gather_floats(mhz)
        return leg
    finally:
        case.free()
        log(f"  {name}: {time.perf_counter() - t_setup:.1f} s")


def run_strong(job: Job) -> dict:
    """M = 65536, N = K = 8192 split by rows over the ranks (B replicated, no collective in the
    timed region), and the all-gather of the bf16 C timed apart."""
    w = WORKLOADS["sharded_65536"]
    from aster_b200 import _native as nat

    t_setup = time.perf_counter()
    case = GemmCase(w, job.rank, job.world)
    try:
        for i in range(3):
            case.run_step(i)
        nat.call("b200_device_synchronize")
        job.barrier()
        sampler = ClockSampler(job.local_rank)
        sampler.start()
        t0 = time.perf_counter()
        stats = time_reference_protocol(case.run_step, 60, 10, plan=case.plan)
        t1 = time.perf_counter()
        clocks = sampler.summary(t0, t1)
        sampler.stop()
        inside = [s[1] for s in sampler.samples if t0 <= s[0] <= t1]
        case.plan.status()
        mhz = stats["sm_mhz"]
        ms_b2b, _, _, _ = time_steps(job, case.run_step, 20, 3)
        out = case.result(3 + 20 - 1)
        check = case.verify(out)
        p50 = job.max_over_ranks(stats["p50_ms"])
        total_flops = 2.0 * w["M"] * w["N"] * w["K"]
        res = case.res
        leg = {
            "workload": w["text"], "n_gpus": job.world, "per_gpu_shape": [case.rows, case.N, case.K],
            "protocol": "60 launches per rank, each between its own event pair and synchronised, first 10 dropped, median; max over ranks",
            "ms_per_step": p50, "tflops_total": total_flops / (p50 * 1e-3) / 1e12, "tflops_per_gpu": case.flops / (p50 * 1e-3) / 1e12,
            "back_to_back_ms_per_step": ms_b2b / 20, "back_to_back_tflops_total": total_flops / (ms_b2b / 20 * 1e-3) / 1e12,
            "roofline": roofline_of(case, p50, sustained=False, sm_mhz=mhz or None),
            "per_rank_p50_ms": job.gather_floats(stats["p50_ms"]), "per_rank_sm_mhz_in_kernel": job.gather_floats(mhz),
            "plan": {"tile": [res.tile_m, res.tile_n, res.tile_k], "stages": res.stages, "grid_ctas": res.grid_ctas, "cta_group": res.cta_group},
            "scaling_note": "efficiency at g GPUs = T_1 / (g * T_g) with T = ms_per_step of the runs at 1 and g GPUs",
            "verified": job.all_ranks_true(check["ok"]), "verify": check,
        }
        leg["clocks"] = clocks
        if inside:
            # The in-kernel clock is that of the one SM that runs CTA 0.  NVML's samples of the region
            # (rank 0's GPU) are printed beside it as they are: the launches are synchronised one by
            # one, so some samples fall between two launches, where the clock is back at its maximum.
            leg["nvml_sm_mhz_quartiles"] = [float(np.percentile(inside, q)) for q in (0, 25, 50, 75, 100)]
        if job.dist is not None and job.world > 1:
            leg["allgather"] = time_allgather(job, case.sets[0][2], case.rows, case.N)
        return leg
    finally:
        case.free()
        log(f"  strong_65536: {time.perf_counter() - t_setup:.1f} s")


def run_bandwidth(args, job: Job, w: dict, name: str, protocol_only: bool = False) -> dict:
    from aster_b200 import _native as nat
    from aster_b200 import bandwidth as bw
    from aster_b200.execution import GpuBuffer
    from aster_b200.gemm import PinnedArray

    peaks = measured_peaks()
    if "n" in w:
        n = w["n"]
        rng = np.random.default_rng(5 + job.rank)
        a = rng.integers(-(2**30), 2**30, n, dtype=np.int32)
        b = rng.integers(-(2**30), 2**30, n, dtype=np.int32)
        da, db, dc = GpuBuffer(a.nbytes), GpuBuffer(b.nbytes), GpuBuffer(a.nbytes)
        da.copy_from_host(a), db.copy_from_host(b)
        alg_bytes = 12 * n
        run_step = lambda i: bw.vector_add_device(da, db, dc, n)  # noqa: E731
        want = (a.view(np.uint32) + b.view(np.uint32)).view(np.int32)
        host_in, dev_in, out_shape, out_dtype = [a, b], [da, db], (n,), np.int32
        dev_out = dc
    else:
        M, N = w["M"], w["N"]
        src = np.random.default_rng(6 + job.rank).standard_normal((M, N), dtype=np.float32)  # drawn in float32: 268 M values
        da, dc = GpuBuffer(src.nbytes), GpuBuffer(src.nbytes)
        da.copy_from_host(src)
        alg_bytes = 8 * M * N
        run_step = lambda i: bw.copy_2d_padded_device(da, dc, M, N, depth=4)  # noqa: E731
        want = src
        host_in, dev_in, out_shape, out_dtype = [src], [da], (M, N), np.float32
        dev_out = dc
    l2_note = f"{alg_bytes / 2**20:.0f} MiB touched per step > {L2_BYTES / 1e6:.0f} MB L2"
    try:
        if protocol_only:
            for i in range(3):
                run_step(i)
            nat.call("b200_device_synchronize")
            l0 = nat.launch_count()
            stats = time_reference_protocol(run_step, 40, 10)
            n_launched = nat.launch_count() - l0
            ms_b2b, _, _, _ = time_steps(job, run_step, 20, 3)
            out = np.empty(out_shape, dtype=out_dtype)
            dev_out.copy_to_host(out)
            gbs = alg_bytes / (stats["p50_ms"] * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                    "peak_source": f"{peaks['_source']} (hbm copy)", "frac_of_nominal": gbs / 8000.0}
            roof.update(dram_traffic(name))
            return {"workload": w["text"], "dtype": "int32" if "n" in w else "f32",
                    "protocol": "40 launches, each between its own event pair and synchronised, first 10 dropped, median",
                    "ms_per_step": stats["p50_ms"], "stats_ms": stats, "achieved": gbs, "unit": "GB/s", "roofline": roof,
                    "back_to_back": {"steps": 20, "ms_per_step": ms_b2b / 20, "achieved": alg_bytes / (ms_b2b / 20 * 1e-3) / 1e9},
                    "l2": l2_note, "gpu_launches": n_launched, "verified": bool(np.array_equal(out, want)),
                    "verify": {"criterion": "bit-exact against the host result", "elements": int(np.prod(out_shape))}}
        sampler = ClockSampler(job.local_rank)
        sampler.start()
        l0 = nat.launch_count()
        ms_total, _, t0, t1 = time_steps(job, run_step, args.steps, args.warmup)
        launches = nat.launch_count() - l0 - args.warmup
        clocks = sampler.summary(t0, t1)
        out = np.empty(out_shape, dtype=out_dtype)
        dev_out.copy_to_host(out)
        verified = job.all_ranks_true(bool(np.array_equal(out, want)))

        # end to end: pinned host -> device, kernel, device -> pinned host, every step
        pins = [PinnedArray(h.shape, h.dtype) for h in host_in]
        for p, h in zip(pins, host_in):
            p.array[...] = h
        pout = PinnedArray(out_shape, out_dtype)
        e2e_steps = max(2, min(args.steps, 10))
        te0 = time.perf_counter()
        for i in range(e2e_steps):
            for p, d in zip(pins, dev_in):
                nat.call("b200_memcpy_h2d_async", d.ptr, p.ptr, p.nbytes, None)
            run_step(i)
            nat.call("b200_memcpy_d2h_async", pout.ptr, dev_out.ptr, pout.nbytes, None)
        nat.call("b200_device_synchronize")
        te = job.max_over_ranks(time.perf_counter() - te0)
        sampler.stop()
        ms_per_step = ms_total / args.steps
        gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                "peak_source": f"{peaks['_source']} (hbm copy)", "frac_of_nominal": gbs / 8000.0}
        roof.update(dram_traffic(name))
        line = {
            "metric": "bandwidth_gbs", "value": gbs * job.world, "unit": "GB/s", "n_gpus": job.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int32" if "n" in w else "f32", "data": "synthetic", "impl": "ours",
            "config": {"workload": w["text"], "name": name, "l2": l2_note},
            "roofline": roof,
            "e2e": {"value": alg_bytes * e2e_steps * job.world / te / 1e9, "unit": "GB/s", "h2d_bytes_per_step": sum(p.nbytes for p in pins),
                    "d2h_bytes_per_step": pout.nbytes, "steps": e2e_steps},
            "gpu_launches": launches, "clocks": clocks, "verified": verified,
        }
        if job.world == 1 and not args.no_cpu_baseline:
            from oracle import gemm_oracle as orc

            best = float("inf")
            for _ in range(3):
                c0 = time.perf_counter()
                _ = orc.vector_add(*host_in) if "n" in w else orc.copy_2d_padded(host_in[0], out)
                best = min(best, time.perf_counter() - c0)
            line["cpu_baseline"] = {"value": alg_bytes / best / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                    "sample": f"whole workload, best of 3 ({best:.3f} s), numpy"}
        return line
    finally:
        for d in dev_in + [dev_out]:
            d.free()


def all_verified(line: dict) -> bool:
    """Every `verified` flag in the line (headline, legs) and the end-to-end comparison."""
    flags = [line.get("verified", True), line.get("e2e", {}).get("matches_device_result", True)]
    flags += [leg.get("verified", True) for leg in line.get("workloads", {}).values() if isinstance(leg, dict)]
    if isinstance(line.get("strong_65536"), dict):
        flags.append(line["strong_65536"].get("verified", True))
    return all(bool(f) for f in flags)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="time this workload only; without it the headline (bf16_4096) is followed by every other configured workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip the sustained, per-workload and strong-scaling legs of the default run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    name = args.workload or DEFAULT_WORKLOAD
    w = WORKLOADS[name]
    full_run = args.workload is None and not args.headline_only

    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0
        print(json.dumps(run_reference_arm(args, w, name)), flush=True)
        return 0

    job = Job(args.gpus)
    from aster_b200 import _native as nat

    if nat.device_count() < 1:
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    nat.call("b200_init", job.local_rank)
    ok = True
    try:
        if "K" not in w:
            line = run_bandwidth(args, job, w, name)
        else:
            t_start = time.perf_counter()
            line, case = run_gemm(args, job, w, name)
            try:
                if full_run:
                    line["sustained"] = run_sustained(job, case, line["ms_per_step"])
            finally:
                case.free()
            if full_run:
                if job.world == 1:
                    legs = {}
                    for extra in EXTRA_WORKLOADS:
                        ew = WORKLOADS[extra]
                        legs[extra] = run_bandwidth(args, job, ew, extra, protocol_only=True) if "K" not in ew else run_gemm_leg(job, ew, extra)
                    line["workloads"] = legs
                line["strong_65536"] = run_strong(job)
                line["bench_seconds"] = time.perf_counter() - t_start
        ok = all_verified(line)
        line["all_verified"] = ok
        if job.rank == 0:
            print(json.dumps(line), flush=True)
    finally:
        job.close()
    if not ok:
        log("bench.py: a result did not verify against the oracle (see the `verified` fields)")
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
