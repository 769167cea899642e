"""Bench harness pieces the GEMM path is driven by: input initialisation, the timing
statistics, the peak table, the result record and the single-config runner.

Mirrors the corresponding parts of contrib/kittens/test/bench/bench_harness.py (init modes
:46-90, ``PerfStats`` / ``_compute_stats`` :100-198, peak table :31-41, ``run_single``
:1738-1850) and of tools/perf_bench_results_io.py (:113-144), so numbers produced here read
like the reference's: 100 launches, the first 20 dropped, p50 as the headline.
"""

from __future__ import annotations

import enum
import json
import os
import statistics
import tempfile
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from .dtypes import from_f32, quantize_e4m3
from .gemm_config import Operand

# Dense tensor peaks (TFLOP/s) per target and input type.  The reference keeps f16 peaks per
# AMD target (bench_harness.py:32-37); sm_100a uses the public dense B200 figures.
_PEAK_TFLOPS_F16_BY_MCPU = {"gfx940": 980.6, "gfx942": 1307.0, "gfx950": 2500.0, "gfx1201": 100.0, "sm_100a": 2250.0}
_PEAK_TFLOPS_FP8_BY_MCPU = {"sm_100a": 4500.0}
PEAK_HBM_GBS = {"sm_100a": 8000.0}


def peak_tflops_f16(mcpu: str) -> float:
    return _PEAK_TFLOPS_F16_BY_MCPU[mcpu]


def peak_tflops(mcpu: str, dtype_ab: str = "f16") -> float:
    return _PEAK_TFLOPS_FP8_BY_MCPU[mcpu] if dtype_ab in ("e4m3", "e5m2", "i8") else _PEAK_TFLOPS_F16_BY_MCPU[mcpu]


class InitMode(enum.StrEnum):
    """Input initialisation modes (bench_harness.py:46-63)."""

    HPL = "hpl"  # uniform [-0.5, 0.5)
    TRIG_FLOAT = "trig_float"  # A = sin(i), B = cos(i) over the flat index
    RAND_INT = "rand_int"  # integers in {-2..2}
    ZERO = "zero"
    SPECIAL = "special"  # fp16 extremes: A = 65280, B = 6.07967e-5
    NORM_DIST = "norm_dist"  # N(0, 1)


INIT_DEFAULT = InitMode.HPL
_SPECIAL = {"A": np.float16(65280.0), "B": np.float16(6.07967376708984375e-5)}

NUM_ITERATIONS = 100
WARMUP_ITERATIONS = 20
RESULT_SENTINEL = "BENCH_RESULT_JSON:"


def init_array(shape, mode: InitMode, role: str, dtype=np.float16, seed: int = 42) -> np.ndarray:
    """Deterministic operand values; role "B" draws from ``seed + 1`` (bench_harness.py:68-90)."""
    mode = InitMode(mode)
    count = int(np.prod(shape))
    if mode == InitMode.ZERO:
        return np.zeros(shape, dtype=dtype)
    if mode == InitMode.TRIG_FLOAT:
        wave = np.sin if role == "A" else np.cos
        return wave(np.arange(count, dtype=np.float64)).astype(dtype).reshape(shape)
    if mode == InitMode.SPECIAL:
        return np.full(shape, _SPECIAL["A" if role == "A" else "B"], dtype=dtype)
    rng = np.random.default_rng(seed + (role == "B"))
    if mode == InitMode.HPL:
        values = rng.uniform(-0.5, 0.5, size=count)
    elif mode == InitMode.RAND_INT:
        values = rng.integers(-2, 3, size=count)
    else:
        values = rng.standard_normal(size=count)
    return values.astype(dtype).reshape(shape)


def make_inputs(cfg, init_mode: InitMode = INIT_DEFAULT, seed: int = 42):
    """A and B for ``cfg`` in its storage type.  Returns ``(A, B)`` for 16-bit configs and
    ``(A, B, scale_a, scale_b)`` for e4m3 (per-tensor ``amax/448`` quantisation); int8 operands
    are scaled to the full integer range."""
    a = init_array(cfg.spec.operand_shape(Operand.A), init_mode, "A", dtype=np.float32, seed=seed)
    b = init_array(cfg.spec.operand_shape(Operand.B), init_mode, "B", dtype=np.float32, seed=seed)
    dt = getattr(cfg, "dtype_ab", "f16")
    if dt == "e4m3":
        qa, sa = quantize_e4m3(a)
        qb, sb = quantize_e4m3(b)
        return qa, qb, float(sa), float(sb)
    if dt == "i8":  # spread the values over the whole integer range
        a, b = (x * (127.0 / max(float(np.abs(x).max()), 1e-30)) for x in (a, b))
    return from_f32(a, dt), from_f32(b, dt)


@dataclass(frozen=True)
class PerfStats:
    p0_ns: float
    p10_ns: float
    p25_ns: float
    p50_ns: float
    p90_ns: float
    mean_ns: float
    stddev_ns: float
    stddev_tf: float
    total_flops: int
    peak_tflops: float

    def _ms(self, ns: float) -> float:
        return ns / 1e6

    def _tf(self, ns: float) -> float:
        return self.total_flops / ns * 1e-3

    def _pct(self, ns: float) -> float:
        return self._tf(ns) / self.peak_tflops * 100

    p0_ms = property(lambda s: s._ms(s.p0_ns))
    p10_ms = property(lambda s: s._ms(s.p10_ns))
    p25_ms = property(lambda s: s._ms(s.p25_ns))
    p50_ms = property(lambda s: s._ms(s.p50_ns))
    p90_ms = property(lambda s: s._ms(s.p90_ns))
    mean_ms = property(lambda s: s._ms(s.mean_ns))
    p0_tf = property(lambda s: s._tf(s.p0_ns))
    p10_tf = property(lambda s: s._tf(s.p10_ns))
    p25_tf = property(lambda s: s._tf(s.p25_ns))
    p50_tf = property(lambda s: s._tf(s.p50_ns))
    p90_tf = property(lambda s: s._tf(s.p90_ns))
    mean_tf = property(lambda s: s._tf(s.mean_ns))
    p0_pct = property(lambda s: s._pct(s.p0_ns))
    p50_pct = property(lambda s: s._pct(s.p50_ns))
    mean_pct = property(lambda s: s._pct(s.mean_ns))


def _percentile_ns(sorted_times: Sequence[float], pct: float) -> float:
    """Nearest-rank percentile of a sorted list (bench_harness.py:174-178)."""
    n = len(sorted_times)
    return float(sorted_times[max(0, min(n - 1, int(round(pct / 100.0 * (n - 1)))))])


def _compute_stats(post_warmup: Sequence[float], total_flops: int, peak_tflops: float) -> Optional[PerfStats]:
    """Post-warm-up timings (ns) -> percentiles, mean, standard deviations; ``None`` when a
    timing is missing or non-positive (bench_harness.py:181-198)."""
    if not post_warmup or min(post_warmup) <= 0:
        return None
    times = sorted(float(t) for t in post_warmup)
    rates = [int(total_flops) / t * 1e-3 for t in times]
    many = len(times) > 1
    return PerfStats(
        p0_ns=times[0],
        p10_ns=_percentile_ns(times, 10),
        p25_ns=_percentile_ns(times, 25),
        p50_ns=_percentile_ns(times, 50),
        p90_ns=_percentile_ns(times, 90),
        mean_ns=float(statistics.fmean(times)),
        stddev_ns=float(statistics.stdev(times)) if many else 0.0,
        stddev_tf=float(statistics.stdev(rates)) if many else 0.0,
        total_flops=int(total_flops),
        peak_tflops=peak_tflops,
    )


def result_record(bench: str, cfg, stats: PerfStats, **extra) -> dict:
    """The ``BENCH_RESULT_JSON`` record (tools/perf_bench_results_io.py:113-144), plus
    optional extra keys (roofline fraction, GPU count, CPU baseline)."""
    m, n, k = cfg.spec.gemm_size
    rec = {
        "mcpu": cfg.mapping.mcpu, "bench": bench, "M": m, "N": n, "K": k, "label": cfg.label,
        "tflops_median": stats.p50_tf, "tflops_p10": stats.p10_tf, "tflops_p90": stats.p90_tf,
        "tflops_mean": stats.mean_tf, "tflops_p0": stats.p0_tf, "tflops_p25": stats.p25_tf,
        "tflops_stddev": stats.stddev_tf, "pct_peak_p50": stats.p50_pct, "sample_n": 1,
    }
    rec.update(extra)
    return rec


def emit_one_result(stream, bench: str, cfg, stats: PerfStats, **extra) -> None:
    if stream is None:
        return
    print(RESULT_SENTINEL + json.dumps(result_record(bench, cfg, stats, **extra)), file=stream)
    stream.flush()


def verify_against_numpy(cfg, C_output: np.ndarray, A: np.ndarray, B: np.ndarray) -> Optional[str]:
    """The reference's gate for a result to count: numpy ``A.f32 @ B.f32.T`` with
    ``rtol = atol = 1e-2`` (bench_harness.py:819-861).  Returns ``None`` on success, else a
    one-line reason.  (Plain f16/bf16 configs only; other configs are verified by the tests.)"""
    from .dtypes import to_f32

    expected = (to_f32(A, cfg.dtype_ab) @ to_f32(B, cfg.dtype_ab).T).reshape(-1)
    got = to_f32(C_output, cfg.dtype_c).reshape(-1)
    rtol = atol = 1e-2
    if cfg.dtype_c == "bf16":
        rtol = 2 ** -7  # one bf16 ulp on top of the reference's gate
    bad = np.abs(got - expected) > atol + rtol * np.abs(expected)
    if bad.any():
        return f"max_abs_diff={float(np.max(np.abs(got - expected))):.6g} mismatched={int(bad.sum())}"
    return None


def run_single(cfg, compile_fn, execute_fn, *, iterations: int = NUM_ITERATIONS, init_mode: InitMode = INIT_DEFAULT,
               bench: str = "unknown", results_file: Optional[str] = None, hsaco: Optional[str] = None,
               stream=None) -> Optional[PerfStats]:
    """Compile, time and verify one config (bench_harness.py:1738-1850): ``iterations`` timed
    launches, the first ``WARMUP_ITERATIONS`` dropped, summary table, then a one-iteration
    correctness run against numpy.  Returns the statistics (``None`` when there is no GPU)."""
    import sys

    from .execution import system_has_gpu

    out = stream or sys.stdout
    tmp = None
    path = hsaco
    if not path:
        tmp = tempfile.NamedTemporaryFile(suffix=".b200plan.json", delete=False)
        tmp.close()
        path = tmp.name
    try:
        _, text = compile_fn(cfg, path)
        res = json.loads(text)["resources"]
        print(f"  {cfg.label}\n  tile {res['tile_m']}x{res['tile_n']}x{res['tile_k']} stages={res['stages']} "
              f"grid={res['grid_ctas']} smem={res['smem_bytes']} tmem_cols={res['tmem_columns']}", file=out)
        if not system_has_gpu(cfg.mapping.mcpu):
            print("No GPUs detected -- skipping execution.", file=out)
            return None
        inputs = make_inputs(cfg, init_mode=init_mode)
        A, B = inputs[0], inputs[1]
        kw = dict(scale_a=inputs[2], scale_b=inputs[3]) if len(inputs) == 4 else {}
        _, times_ns = execute_fn(cfg, path, iterations, A, B, skip_gpu_check=True, **kw)
        measured = times_ns[WARMUP_ITERATIONS:]
        if not measured:
            print(f"\nNo measurements after warmup ({iterations} iterations), use a number > {WARMUP_ITERATIONS}", file=out)
            return None
        s = _compute_stats(measured, cfg.total_flops, peak_tflops(cfg.mapping.mcpu, cfg.dtype_ab))
        if s is None:
            print(f"\nInvalid timings (min={min(measured)} ns)", file=out)
            return None
        if results_file:
            with open(results_file, "a") as rs:
                emit_one_result(rs, bench, cfg, s)
        print("\n--- Summary ---", file=out)
        print(f"  {'metric':<8s}  {'ms':>10s}  {'TFLOPS':>10s}  {'% peak':>8s}", file=out)
        for name, ms, tf, pct in (
            ("p0", s.p0_ms, s.p0_tf, s.p0_pct), ("p10", s.p10_ms, s.p10_tf, None), ("p25", s.p25_ms, s.p25_tf, None),
            ("p50", s.p50_ms, s.p50_tf, s.p50_pct), ("p90", s.p90_ms, s.p90_tf, None), ("mean", s.mean_ms, s.mean_tf, s.mean_pct),
        ):
            pct_s = f"{pct:>7.1f}%" if pct is not None else f"{'':>8s}"
            print(f"  {name:<8s}  {ms:>10.4f}  {tf:>10.1f}  {pct_s}", file=out)
        print(f"  {'stddev':<8s}  {'':>10s}  {s.stddev_tf:>10.1f}", file=out)
        if cfg.epilogue == "none" and cfg.dtype_ab != "e4m3":
            print("\n--- Correctness check ---", file=out)
            C_output, _ = execute_fn(cfg, path, 1, A, B, skip_gpu_check=True)
            why = verify_against_numpy(cfg, C_output, A, B)
            print("PASS" if why is None else f"FAIL: {why}", file=out)
        return s
    finally:
        if tmp is not None:
            try:
                os.unlink(tmp.name)
            except OSError:
                pass
