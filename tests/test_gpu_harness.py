"""The sweep tooling on a GPU: the single-process sweep and the persistent-worker pipeline time
real plans and only count results that pass the numpy check."""

import io
import json

import pytest

from aster_b200 import bench_workers as bw
from aster_b200.bench_search import run_sweep
from aster_b200.gemm_config import make_b200_instance
from aster_b200.multitile_gemm import BENCH_HOOKS

pytestmark = pytest.mark.gpu


def small_instances():
    return [make_b200_instance(256, 256, 512, dtype_ab="bf16", dtype_c="f32", tile_n=tn, cta_group=cg, stages=st)
            for tn, cg, st in ((64, 1, 0), (128, 1, 3), (128, 2, 0), (256, 1, 2))]


def test_run_sweep_times_and_verifies_real_plans(gpu):
    out = io.StringIO()
    ranked = run_sweep(small_instances(), iterations=30, results_stream=out, verify_top=4, log=lambda *_: None)
    assert len(ranked) == 4
    for label, stats, note in ranked:
        assert stats is not None and stats.p50_tf > 0 and note == "verified", (label, note)
    lines = [l for l in out.getvalue().splitlines() if l.startswith("BENCH_RESULT_JSON:")]
    assert len(lines) == 4 and {json.loads(l.split(":", 1)[1])["label"] for l in lines} == {r[0] for r in ranked}


def test_pipelined_sweep_and_verification_with_real_workers(gpu, tmp_path):
    """One persistent worker process on GPU 0 (its own CUDA context), lock file in a private
    directory; then the verification pass over the same artifacts."""
    cfgs = small_instances()
    logs = []
    results, paths = bw.bench_perf_sweep_pipelined(
        cfgs, BENCH_HOOKS["compile_fn"], BENCH_HOOKS["repro_cmd_fn"], mcpu="sm_100a", bench=BENCH_HOOKS["bench_label"], num_gpus=1,
        post_compile_filter=BENCH_HOOKS["post_compile_filter"], iterations=30, hsaco_dir=str(tmp_path / "plans"),
        results_file=str(tmp_path / "results.jsonl"), lock_dir=str(tmp_path / "locks"), log=logs.append)
    assert len(results) == 4 and set(paths) == {c.label for c in cfgs}, logs
    assert all(stats.p50_tf > 0 for _, stats in results)
    passed, errors = bw.verify_on_gpus(cfgs, paths, 1, lock_dir=str(tmp_path / "locks"))
    assert (passed, errors) == (4, [])
    assert bw.verify_top_configs(results, paths, top_n=2, num_gpus=1, lock_dir=str(tmp_path / "locks")) == {c.label for c, _ in results[:2]}
    assert bw.detect_num_gpus("sm_100a") >= 1
