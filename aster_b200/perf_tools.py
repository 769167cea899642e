"""Result records, the best-known registry and the regression dashboard for GEMM benches.

Same file formats and rules as the reference's tooling under
contrib/kittens/test/bench/tools/, so registries and result logs can be shared:

* result lines: ``BENCH_RESULT_JSON:{...}`` with ``mcpu, bench, M, N, K, label, tflops_median``
  (+ optional spread fields), noise between them ignored (perf_bench_results_io.py:15-110);
* registry ``{mcpu: {bench: {"MxNxK": [{label, expected_tflops}, ...]}}}``, top 5 per size,
  best first, written atomically via a temporary file (perf_best_known.py:1-67);
* dashboard: one row per stored entry, matched on ``(mcpu, bench, M, N, K, label)``;
  REGRESS below ``expected * (1 - 5 %)``, IMPROVE above ``expected * (1 + 3 %)``, OK otherwise,
  MISS without a measurement; exit code 1 on any REGRESS, else 2 on any MISS, else 0
  (perf_dashboard.py:21-131).

CLI::

    python -m aster_b200.perf_tools update --input results.jsonl --best-known-file reg.json [--apply]
    python -m aster_b200.perf_tools dashboard --measurements results.jsonl --best-known-file reg.json
    python -m aster_b200.perf_tools dashboard --dry-run --best-known-file reg.json
    python -m aster_b200.perf_tools evaluate --best-known-file reg.json --out results.jsonl
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Iterator, Optional

RESULT_SENTINEL = "BENCH_RESULT_JSON:"
TOP_N = 5
DEFAULT_IMPROVE_MARGIN = 0.03
DEFAULT_REGRESS_MARGIN = 0.05
DEFAULT_REGISTRY = Path(__file__).parent / "best_known.json"


# ---------------------------------------------------------------------------------------------
# result records
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class EntryKey:
    mcpu: str
    bench: str
    M: int
    N: int
    K: int


@dataclass(frozen=True)
class BenchResultRecord:
    key: EntryKey
    label: str
    tflops_median: float
    tflops_p10: Optional[float] = None
    tflops_p90: Optional[float] = None
    tflops_mean: Optional[float] = None
    sample_n: int = 1


def _opt_float(v) -> Optional[float]:
    try:
        return None if v is None else float(v)
    except (TypeError, ValueError):
        return None


def parse_jsonl_results(stream: Iterable[str]) -> Iterator[BenchResultRecord]:
    """One record per well-formed result line; anything else (logs, broken JSON, records that
    lack a required field) is skipped."""
    for raw in stream:
        at = raw.find(RESULT_SENTINEL)
        if at < 0:
            continue
        try:
            d = json.loads(raw[at + len(RESULT_SENTINEL):].strip())
            key = EntryKey(d["mcpu"], d["bench"], int(d["M"]), int(d["N"]), int(d["K"]))
            rec = BenchResultRecord(key, d["label"], float(d["tflops_median"]), _opt_float(d.get("tflops_p10")),
                                    _opt_float(d.get("tflops_p90")), _opt_float(d.get("tflops_mean")), int(d.get("sample_n", 1)))
        except (json.JSONDecodeError, KeyError, TypeError, ValueError):
            continue
        yield rec


def max_merge_by_key_label(records: Iterable[BenchResultRecord]) -> dict:
    """Best record per (key, label) across runs."""
    best: dict = {}
    for r in records:
        slot = (r.key, r.label)
        if slot not in best or r.tflops_median > best[slot].tflops_median:
            best[slot] = r
    return best


def max_merge_by_key(records: Iterable[BenchResultRecord]) -> dict:
    """Best record per key across runs and labels."""
    best: dict = {}
    for r in max_merge_by_key_label(records).values():
        if r.key not in best or r.tflops_median > best[r.key].tflops_median:
            best[r.key] = r
    return best


# ---------------------------------------------------------------------------------------------
# registry
# ---------------------------------------------------------------------------------------------
def size_key(M: int, N: int, K: int) -> str:
    return f"{M}x{N}x{K}"


def parse_size_key(key: str) -> tuple[int, int, int]:
    m, n, k = key.split("x")
    return int(m), int(n), int(k)


def load_registry(path=DEFAULT_REGISTRY) -> dict:
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        return json.load(f)


def save_registry(data: dict, path=DEFAULT_REGISTRY) -> None:
    tmp = f"{path}.tmp"
    with open(tmp, "w") as f:
        json.dump(data, f, indent=2, sort_keys=True)
        f.write("\n")
    os.replace(tmp, path)  # readers never see a half-written registry


def best_known_top_n(registry: dict, mcpu: str, bench: str, M: int, N: int, K: int) -> list:
    return list(registry.get(mcpu, {}).get(bench, {}).get(size_key(M, N, K)) or [])


def best_known(registry: dict, mcpu: str, bench: str, M: int, N: int, K: int) -> Optional[str]:
    slot = best_known_top_n(registry, mcpu, bench, M, N, K)
    return slot[0]["label"] if slot else None


def merge_results_into_registry(registry: dict, records: Iterable[BenchResultRecord], top_n: int = TOP_N) -> list[str]:
    """Fold measurements into the registry: per size slot keep the ``top_n`` labels by
    throughput (a label's stored value only ever rises).  Returns a line per changed slot."""
    changes = []
    for (key, label), rec in sorted(max_merge_by_key_label(records).items(), key=lambda kv: (kv[0][0].bench, kv[0][1])):
        slot = registry.setdefault(key.mcpu, {}).setdefault(key.bench, {}).setdefault(size_key(key.M, key.N, key.K), [])
        before = [(e["label"], e["expected_tflops"]) for e in slot]
        by_label = {e["label"]: e for e in slot}
        if label not in by_label:
            slot.append({"label": label, "expected_tflops": rec.tflops_median})
        elif rec.tflops_median > by_label[label]["expected_tflops"]:
            by_label[label]["expected_tflops"] = rec.tflops_median
        slot.sort(key=lambda e: -e["expected_tflops"])
        del slot[top_n:]
        if [(e["label"], e["expected_tflops"]) for e in slot] != before:
            changes.append(f"{key.mcpu}/{key.bench}/{size_key(key.M, key.N, key.K)}: {label} -> {rec.tflops_median:.1f}")
    return changes


# ---------------------------------------------------------------------------------------------
# dashboard
# ---------------------------------------------------------------------------------------------
_STATUS_ORDER = {"REGRESS": 0, "MISS": 1, "IMPROVE": 2, "OK": 3}


@dataclass
class Row:
    key: EntryKey
    rank: int
    label: str
    expected_tflops: float
    measured: Optional[float]


def status_of(measured: Optional[float], expected: float, regress_margin: float = DEFAULT_REGRESS_MARGIN,
              improve_margin: float = DEFAULT_IMPROVE_MARGIN) -> str:
    if measured is None:
        return "MISS"
    if measured < expected * (1.0 - regress_margin):
        return "REGRESS"
    if measured > expected * (1.0 + improve_margin):
        return "IMPROVE"
    return "OK"


def dashboard_rows(registry: dict, records: Iterable[BenchResultRecord]) -> list[Row]:
    measured = {slot: rec.tflops_median for slot, rec in max_merge_by_key_label(records).items()}
    rows = []
    for mcpu, benches in sorted(registry.items()):
        for bench, sizes in sorted(benches.items()):
            for skey, slot in sorted(sizes.items()):
                key = EntryKey(mcpu, bench, *parse_size_key(skey))
                for rank, entry in enumerate(slot, start=1):
                    rows.append(Row(key, rank, entry["label"], float(entry["expected_tflops"]), measured.get((key, entry["label"]))))
    return rows


def render_dashboard(rows: list[Row], dry_run: bool = False, regress_margin: float = DEFAULT_REGRESS_MARGIN,
                     improve_margin: float = DEFAULT_IMPROVE_MARGIN) -> tuple[str, int]:
    """Table + summary line, and the exit code (1 REGRESS, 2 MISS, 0 otherwise)."""
    judged = [(r, status_of(r.measured, r.expected_tflops, regress_margin, improve_margin)) for r in rows]
    judged.sort(key=lambda rs: (_STATUS_ORDER[rs[1]], rs[0].key.mcpu, rs[0].key.bench, rs[0].key.M, rs[0].key.N, rs[0].key.K, rs[0].rank))
    header = ["mcpu", "bench", "M", "N", "K", "rank", "expected", "measured", "delta_pct", "status", "label"]
    table = [header]
    for r, st in judged:
        delta = "---" if r.measured is None or r.expected_tflops == 0 else f"{(r.measured - r.expected_tflops) / r.expected_tflops * 100:+.2f}%"
        table.append([r.key.mcpu, r.key.bench, str(r.key.M), str(r.key.N), str(r.key.K), f"#{r.rank}", f"{r.expected_tflops:.1f}",
                      "---" if r.measured is None else f"{r.measured:.1f}", delta, "?" if dry_run else st,
                      r.label.split("_", 1)[1] if "_" in r.label else r.label])
    widths = [max(len(row[i]) for row in table) for i in range(len(header))]
    lines = ["  ".join(cell.ljust(w) for cell, w in zip(row, widths)).rstrip() for row in table]
    if dry_run:
        return "\n".join(lines + [f"{len(rows)} stored entries listed (dry-run; no measurements)."]), 0
    counts = {k: sum(1 for _, st in judged if st == k) for k in _STATUS_ORDER}
    slots = len({(r.key.mcpu, r.key.bench, r.key.M, r.key.N, r.key.K) for r in rows})
    summary = (f"{len(rows)} stored entries across {slots} (mcpu,bench,M,N,K) slot(s) checked.  "
               f"{counts['REGRESS']} REGRESS, {counts['IMPROVE']} IMPROVE, {counts['OK']} OK")
    summary += f", {counts['MISS']} MISS." if counts["MISS"] else "."
    code = 1 if counts["REGRESS"] else (2 if counts["MISS"] else 0)
    return "\n".join(lines + [summary]), code


# ---------------------------------------------------------------------------------------------
# CLI
# ---------------------------------------------------------------------------------------------
# ---------------------------------------------------------------------------------------------
# re-measuring the registry
# ---------------------------------------------------------------------------------------------
def iter_registry(data: dict, mcpu_filter: Optional[str] = None, bench_filter: Optional[str] = None):
    """``(mcpu, bench, size_key, slot)`` for every stored slot that passes the filters."""
    for mcpu, benches in sorted(data.items()):
        if mcpu_filter and mcpu != mcpu_filter:
            continue
        for bench, sizes in sorted(benches.items()):
            if bench_filter and bench != bench_filter:
                continue
            for key, slot in sorted(sizes.items()):
                yield mcpu, bench, key, slot


def collect_todo(data: dict, mcpu_filter: Optional[str] = None, bench_filter: Optional[str] = None) -> dict:
    """``{(mcpu, bench): [label, ...]}`` for every stored config (tools/perf_evaluate.py:42-51)."""
    todo: dict = {}
    for mcpu, bench, _key, slot in iter_registry(data, mcpu_filter, bench_filter):
        for entry in slot:
            todo.setdefault((mcpu, bench), []).append(entry["label"])
    return todo


def measure_all(data: dict, out_path: str, *, mcpu_filter: Optional[str] = None, bench_filter: Optional[str] = None,
                iterations: Optional[int] = None, compile_workers: Optional[int] = None, hsaco_dir: Optional[str] = None,
                num_gpus: Optional[int] = None, compile_only: bool = False, hooks_for=None, sweep_fn=None, verify_fn=None, log=None) -> str:
    """Re-measure every label of the registry, bench by bench, and write one result line per
    config that also passes verification (tools/perf_evaluate.py:54-149): truncate ``out_path``;
    per ``(mcpu, bench)`` rebuild the configs through the bench's ``from_label`` hook, run the
    pipelined sweep, verify every measured config on the GPUs, append only the verified ones.
    ``hooks_for(bench) -> BENCH_HOOKS dict or None``, ``sweep_fn`` and ``verify_fn`` default to
    the library's own (:func:`aster_b200.multitile_gemm.hooks_for_bench`,
    :func:`aster_b200.bench_workers.bench_perf_sweep_pipelined`, ``verify_top_configs``)."""
    from .bench_harness import emit_one_result

    if log is None:
        log = lambda *a: print(*a, file=sys.stderr)  # noqa: E731
    if hooks_for is None:
        from .multitile_gemm import hooks_for_bench as hooks_for
    if sweep_fn is None or verify_fn is None:
        from . import bench_workers as bw

        sweep_fn = sweep_fn or bw.bench_perf_sweep_pipelined
        verify_fn = verify_fn or bw.verify_top_configs
    open(out_path, "w").close()  # truncate
    todo = collect_todo(data, mcpu_filter, bench_filter)
    log(f"=== measure_all: {sum(len(v) for v in todo.values())} stored config(s) across {len(todo)} bench group(s) -> {out_path} ===")
    for i, ((mcpu, bench), labels) in enumerate(sorted(todo.items()), start=1):
        log(f"  [{i}/{len(todo)}] {bench} (mcpu={mcpu}, {len(labels)} label(s))")
        hooks = hooks_for(bench)
        if hooks is None:
            log(f"    SKIP -- no hooks known for bench {bench!r}")
            continue
        try:
            configs = [hooks["from_label"](lbl, mcpu) for lbl in labels]
        except Exception as e:
            log(f"    SKIP -- a stored label does not parse: {e}")
            continue
        per_bench_dir = os.path.join(hsaco_dir, bench) if hsaco_dir else None
        if per_bench_dir:
            os.makedirs(per_bench_dir, exist_ok=True)
        results, paths = sweep_fn(configs, hooks["compile_fn"], hooks["repro_cmd_fn"], mcpu=mcpu, bench=hooks["bench_label"],
                                  num_gpus=0 if compile_only else num_gpus, compile_workers=compile_workers,
                                  post_compile_filter=hooks["post_compile_filter"], iterations=iterations, hsaco_dir=per_bench_dir,
                                  results_file=None)  # lines are written after verification, not during the sweep
        verified: set = set()
        if results and not compile_only:
            ranked = sorted(results, key=lambda r: -(r[1].p50_tf if r[1] is not None else 0.0))
            verified = verify_fn(ranked, paths, top_n=len(ranked), num_gpus=num_gpus if num_gpus is not None else 1)
        if verified:
            with open(out_path, "a") as rs:
                for cfg, stats in results:
                    if stats is not None and cfg.label in verified:
                        emit_one_result(rs, hooks["bench_label"], cfg, stats)
            log(f"    Emitted {len(verified)}/{len(configs)} verified result(s)")
        elif not compile_only:
            log(f"    WARNING: 0/{len(configs)} configs passed correctness for {bench}")
    return out_path


def _read_records(paths: list[str]) -> list[BenchResultRecord]:
    out = []
    for p in paths:
        with open(p) as f:
            out.extend(parse_jsonl_results(f))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aster_b200.perf_tools")
    sub = ap.add_subparsers(dest="cmd", required=True)
    up = sub.add_parser("update", help="merge measured results into the registry")
    up.add_argument("--input", action="append", required=True)
    up.add_argument("--best-known-file", default=str(DEFAULT_REGISTRY))
    up.add_argument("--apply", action="store_true", help="write the registry (default: only report)")
    up.add_argument("--top-n", type=int, default=TOP_N)
    da = sub.add_parser("dashboard", help="compare measurements with the registry")
    da.add_argument("--measurements", action="append", default=[])
    da.add_argument("--best-known-file", default=str(DEFAULT_REGISTRY))
    da.add_argument("--dry-run", action="store_true")
    da.add_argument("--regress-margin", type=float, default=DEFAULT_REGRESS_MARGIN)
    da.add_argument("--improve-margin", type=float, default=DEFAULT_IMPROVE_MARGIN)
    ev = sub.add_parser("evaluate", help="re-measure every stored label on the GPUs; only verified results are written")
    ev.add_argument("--best-known-file", default=str(DEFAULT_REGISTRY))
    ev.add_argument("--out", required=True, help="result lines (BENCH_RESULT_JSON) are written here")
    ev.add_argument("--mcpu", default=None)
    ev.add_argument("--bench", default=None)
    ev.add_argument("--iterations", type=int, default=None)
    ev.add_argument("--compile-workers", type=int, default=None)
    ev.add_argument("--hsaco-dir", default=None)
    ev.add_argument("--num-gpus", type=int, default=None)
    ev.add_argument("--compile-only", action="store_true")
    args = ap.parse_args(argv)
    registry = load_registry(args.best_known_file)
    if args.cmd == "evaluate":
        measure_all(registry, args.out, mcpu_filter=args.mcpu, bench_filter=args.bench, iterations=args.iterations,
                    compile_workers=args.compile_workers, hsaco_dir=args.hsaco_dir, num_gpus=args.num_gpus, compile_only=args.compile_only)
        return 0
    if args.cmd == "update":
        changes = merge_results_into_registry(registry, _read_records(args.input), args.top_n)
        for c in changes:
            print(("updated " if args.apply else "would update ") + c)
        if args.apply:
            save_registry(registry, args.best_known_file)
        print(f"{len(changes)} slot update(s){'' if args.apply else ' (not written; pass --apply)'}.")
        return 0
    rows = dashboard_rows(registry, [] if args.dry_run else _read_records(args.measurements))
    text, code = render_dashboard(rows, args.dry_run, args.regress_margin, args.improve_margin)
    print(text)
    return code


if __name__ == "__main__":
    sys.exit(main())
