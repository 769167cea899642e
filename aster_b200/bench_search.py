"""Sweep search over GEMM plan knobs: enumerate, prune, sample, time, verify, record.

``SweepGrid`` has the interface of the reference's class (contrib/kittens/test/bench/
bench_search.py:59-258): chain ``.axis()`` / ``.filter()``, set ``.build_with()``, call
``.generate()``; filters are applied at the shallowest nesting level where all the axes they
read are bound.  The axes worth sweeping on B200 are few (tile width, CTA group, ring depth,
split), so a sweep is minutes, not the reference's hours of compile + run.

``run_sweep`` times every instance with the reference's protocol (N launches, first 20
dropped, p50 headline), checks the best ones against numpy before they may be recorded
(bench_search.py:596-643: only verified labels are emitted) and writes ``BENCH_RESULT_JSON``
lines that :mod:`aster_b200.perf_tools` folds into the registry.

    python -m aster_b200.bench_search --size 4096x4096x4096 --dtype bf16 --out-dtype bf16 \\
        --results-file sweep.jsonl [--iterations 60] [--sample 0]
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import tempfile
from typing import Any, Callable, Hashable, Iterable, Optional

from .bench_harness import NUM_ITERATIONS, WARMUP_ITERATIONS, _compute_stats, emit_one_result, make_inputs, peak_tflops, verify_against_numpy
from .gemm_config import make_b200_instance
from .multitile_gemm import BENCH_HOOKS, compile_multitile_gemm, execute_multitile_hsaco, fits_on_sm_post_compile


class SweepAxis:
    def __init__(self, name: str, values: Iterable[Any]) -> None:
        self.name = name
        self.values = list(values)


class SweepFilter:
    def __init__(self, deps: tuple, check: Callable[[dict], bool], name: Optional[str] = None) -> None:
        self.deps = deps
        self.check = check
        self.name = name


class SweepGrid:
    """Composable search space with hierarchical pruning."""

    def __init__(self) -> None:
        self._axes: list[SweepAxis] = []
        self._filters: list[SweepFilter] = []
        self._builder: Optional[Callable[[dict], Any]] = None

    def axis(self, name: str, values: Iterable[Any]) -> "SweepGrid":
        self._axes.append(SweepAxis(name, values))
        return self

    def filter(self, *deps: str, check: Callable[[dict], bool], name: Optional[str] = None) -> "SweepGrid":
        known = {a.name for a in self._axes}
        missing = [d for d in deps if d not in known]
        if missing:
            tag = f" (filter {name!r})" if name else ""
            raise ValueError(f"SweepGrid.filter: unknown axis dep(s) {missing}{tag}. Registered axes: {sorted(known)}")
        self._filters.append(SweepFilter(deps, check, name))
        return self

    def build_with(self, fn: Callable[[dict], Any]) -> "SweepGrid":
        self._builder = fn
        return self

    def filter_names(self) -> tuple:
        return tuple(f.name for f in self._filters if f.name is not None)

    def axis_values(self) -> dict:
        return {a.name: list(a.values) for a in self._axes}

    def restrict_axes(self, overrides: dict) -> None:
        for a in self._axes:
            if a.name in overrides:
                a.values = list(overrides[a.name])

    def retain_filters(self, allowed_names: set) -> None:
        self._filters = [f for f in self._filters if f.name is None or f.name in allowed_names]

    def _walk(self, depth: int, bound: dict, per_level: list, out: list) -> None:
        if depth == len(self._axes):
            out.append(dict(bound))
            return
        axis = self._axes[depth]
        for value in axis.values:
            bound[axis.name] = value
            if all(f.check(bound) for f in per_level[depth]):
                self._walk(depth + 1, bound, per_level, out)
            del bound[axis.name]

    def generate(self, sample_size: int = 3000, stratification_key: Optional[Callable[[dict], Hashable]] = None,
                 extra_eligible: Optional[list] = None, seed: int = 0) -> tuple:
        """Enumerate, sample, build.  Returns ``(instances, cfgs, total_eligible)``; ``cfgs[i]``
        is the axis dict behind ``instances[i]``.  ``extra_eligible`` configs skip enumeration
        and always survive sampling (if the filters accept them)."""
        empty = [a.name for a in self._axes if not a.values]
        if empty:
            raise ValueError(f"SweepGrid has axes with no values {empty!r}")
        assert self._builder is not None, "call build_with() before generate()"
        names = [a.name for a in self._axes]
        per_level = []
        for i in range(len(names)):
            now, before = set(names[: i + 1]), set(names[:i])
            per_level.append([f for f in self._filters if set(f.deps) <= now and not set(f.deps) <= before])
        eligible: list = []
        self._walk(0, {}, per_level, eligible)

        protected: list = []
        if extra_eligible:
            frozen = {tuple(sorted(c.items())) for c in eligible}
            seen = set()
            for extra in extra_eligible:
                key = tuple(sorted(extra.items()))
                if key in seen or any(not f.check(extra) for f in self._filters if all(d in extra for d in f.deps)):
                    continue
                seen.add(key)
                protected.append(extra)
                frozen.discard(key)
            eligible = [c for c in eligible if tuple(sorted(c.items())) in frozen]
        total = len(eligible) + len(protected)

        if sample_size > 0:
            budget = max(0, sample_size - len(protected))
            if len(eligible) > budget:
                rng = random.Random(seed)
                if stratification_key is None:
                    eligible = rng.sample(eligible, budget)
                else:
                    eligible = _stratified_sample(eligible, stratification_key, budget, rng)
        chosen = eligible + protected

        instances, cfgs, labels = [], [], set()
        for cfg in chosen:
            inst = self._builder(cfg)
            label = getattr(inst, "label", None)
            if label is not None:
                if label in labels:  # an axis that does not reach the builder
                    continue
                labels.add(label)
            instances.append(inst)
            cfgs.append(cfg)
        print(f"Total: {total:,} eligible, {len(instances):,} selected")
        return instances, cfgs, total


def _stratified_sample(configs: list, key: Callable[[dict], Hashable], budget: int, rng: random.Random) -> list:
    """Round-robin over the strata so that every stratum keeps representatives."""
    strata: dict = {}
    for c in configs:
        strata.setdefault(key(c), []).append(c)
    for bucket in strata.values():
        rng.shuffle(bucket)
    out: list = []
    while len(out) < budget and any(strata.values()):
        for k in list(strata):
            if strata[k] and len(out) < budget:
                out.append(strata[k].pop())
    return out


def parse_mnk(text: str) -> tuple:
    parts = text.lower().split("x")
    if len(parts) != 3:
        raise argparse.ArgumentTypeError(f"expected MxNxK, got {text!r}")
    return tuple(int(p) for p in parts)


def b200_gemm_grid(M: int, N: int, K: int, dtype_ab: str = "bf16", dtype_c: str = "bf16", epilogue: str = "none") -> SweepGrid:
    """The plan knobs worth sweeping on B200 for one problem size."""
    kb_elems = 128 if dtype_ab in ("e4m3", "e5m2", "i8") else 64
    k_blocks = -(-K // kb_elems)

    def stage_bytes(d):
        return (128 + d["tile_n"] // d["cta_group"]) * 128

    grid = (
        SweepGrid()
        .axis("tile_n", [64, 128, 256])
        .axis("cta_group", [1, 2])
        .axis("stages", [0, 3, 4, 5, 6])
        .axis("split_k", [0, 2, 4])
        .filter("tile_n", check=lambda d: d["tile_n"] <= max(64, N), name="tile_not_wider_than_n")
        .filter("cta_group", check=lambda d: d["cta_group"] == 1 or M >= 256, name="pair_needs_256_rows")
        .filter("tile_n", "cta_group", "stages", check=lambda d: d["stages"] * stage_bytes(d) + 1280 <= 232448, name="fits_shared_memory")
        .filter("split_k", check=lambda d: d["split_k"] == 0 or (k_blocks // d["split_k"] >= 4 and M * N * 4 * d["split_k"] <= 1 << 30),
                name="split_leaves_k_blocks")
    )
    return grid.build_with(lambda d: make_b200_instance(M, N, K, dtype_ab=dtype_ab, dtype_c=dtype_c, epilogue=epilogue, tile_n=d["tile_n"],
                                                        stages=d["stages"], split_k=d["split_k"], cta_group=d["cta_group"]))


def run_sweep(instances: list, *, iterations: int = NUM_ITERATIONS, results_stream=None, verify_top: int = 3,
              bench: str = BENCH_HOOKS["bench_label"], execute_fn=execute_multitile_hsaco, compile_fn=compile_multitile_gemm,
              log=print) -> list:
    """Time every instance, verify the ``verify_top`` fastest against numpy, emit their result
    records.  Returns ``[(label, stats or None, note)]`` sorted fastest first.  An instance that
    fails to compile, does not fit, or raises at run time is reported and skipped (the harness
    turns exceptions into one-line errors the same way, bench_harness.py:589-590)."""
    measured = []
    with tempfile.TemporaryDirectory() as tmp:
        for i, cfg in enumerate(instances):
            path = f"{tmp}/cfg{i}.b200plan.json"
            try:
                _, text = compile_fn(cfg, path)
                reason = fits_on_sm_post_compile(cfg, json.loads(text)["resources"])
                if reason is not None:
                    measured.append((cfg, path, None, f"filtered: {reason}"))
                    continue
                inputs = make_inputs(cfg)
                kw = dict(scale_a=inputs[2], scale_b=inputs[3]) if len(inputs) == 4 else {}
                _, times = execute_fn(cfg, path, iterations, inputs[0], inputs[1], skip_gpu_check=True, **kw)
                stats = _compute_stats(times[WARMUP_ITERATIONS:], cfg.total_flops, peak_tflops(cfg.mapping.mcpu, cfg.dtype_ab))
                measured.append((cfg, path, stats, "" if stats else "no valid timings"))
                if stats:
                    log(f"  {stats.p50_tf:8.1f} TFLOP/s p50  {cfg.label}")
            except Exception as e:  # one bad config must not end the sweep
                measured.append((cfg, path, None, str(e).splitlines()[0][:200] if str(e) else type(e).__name__))
        ranked = sorted(measured, key=lambda m: -(m[2].p50_tf if m[2] else -1.0))
        out = []
        for rank, (cfg, path, stats, note) in enumerate(ranked):
            if stats and rank < verify_top and cfg.epilogue == "none" and cfg.dtype_ab != "e4m3":
                inputs = make_inputs(cfg)
                C, _ = execute_fn(cfg, path, 1, inputs[0], inputs[1], skip_gpu_check=True)
                why = verify_against_numpy(cfg, C, inputs[0], inputs[1])
                if why is not None:
                    out.append((cfg.label, stats, f"FAILED verification: {why}"))
                    continue
                note = "verified"
                emit_one_result(results_stream, bench, cfg, stats)
            elif stats and rank < verify_top:
                note = "not verified here (epilogue / fp8 parity is covered by the tests)"
                emit_one_result(results_stream, bench, cfg, stats)
            out.append((cfg.label, stats, note))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--size", type=parse_mnk, required=True)
    ap.add_argument("--dtype", default="bf16", choices=["f16", "bf16", "e4m3", "e5m2", "i8"])
    ap.add_argument("--out-dtype", default="bf16", choices=["f32", "bf16", "i32"])
    ap.add_argument("--iterations", type=int, default=60)
    ap.add_argument("--sample", type=int, default=0, help="0 = every eligible config")
    ap.add_argument("--verify-top", type=int, default=3)
    ap.add_argument("--results-file")
    ap.add_argument("--list", action="store_true", help="print the labels and exit (needs no GPU)")
    args = ap.parse_args(argv)
    m, n, k = args.size
    instances, cfgs, total = b200_gemm_grid(m, n, k, args.dtype, args.out_dtype).generate(sample_size=args.sample)
    if args.list:
        for inst in instances:
            print(inst.label)
        return 0
    stream = open(args.results_file, "a") if args.results_file else sys.stdout
    try:
        # fp8 results get their own registry slot: the size key alone would make them compete
        # with the 16-bit configs of the same shape
        bench = BENCH_HOOKS["bench_label"] + {"e4m3": "_fp8", "e5m2": "_bf8", "i8": "_i8"}.get(args.dtype, "")
        ranked = run_sweep(instances, iterations=args.iterations, results_stream=stream, verify_top=args.verify_top, bench=bench)
    finally:
        if args.results_file:
            stream.close()
    print("\n--- ranking ---")
    for label, stats, note in ranked[:10]:
        print(f"  {stats.p50_tf if stats else float('nan'):8.1f}  {note:10s} {label}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
