"""The harness process model on CPU: persistent workers that survive crashes and hangs of their
children, per-GPU locks, verification fan-out, the pipelined sweep, the tier schedule and the
registry re-measurement.  Every failure here is made on the host (a child that exits, kills
itself or never answers; an artifact cut short); no GPU is involved."""

import argparse
import io
import json
import os
import queue
import threading
import time

import pytest

import fake_gpu_workers as fake
from aster_b200 import bench_tier as bt
from aster_b200 import bench_workers as bw
from aster_b200 import perf_tools as pt
from aster_b200.bench_harness import PerfStats, _compute_stats
from aster_b200.bench_search import SweepGrid
from aster_b200.gemm_config import make_b200_instance
from aster_b200.multitile_gemm import BENCH_HOOKS, compile_multitile_gemm, hooks_for_bench


class FakeMapping:
    mcpu = "sm_100a"
    direct_b = False


class FakeSpec:
    gemm_size = (256, 256, 256)


class FakeCfg:
    """What the harness needs of a config: label, sizes, kernel name, flops."""

    kernel_name = "gemm_multitile"
    num_workgroups = 4
    num_threads = 256
    gemm_size = (256, 256, 256)
    total_flops = 2 * 256 ** 3
    dtype_ab = "f16"
    mapping = FakeMapping()
    spec = FakeSpec()

    def __init__(self, label):
        self.label = label


def item(label, iters=3):
    return bw.work_item(FakeCfg(label), f"/nonexistent/{label}.json", iters)


def test_visible_devices_and_lock_paths(tmp_path):
    assert bw.visible_device_ids({}) is None and bw.visible_device_ids({"CUDA_VISIBLE_DEVICES": " "}) is None
    assert bw.visible_device_ids({"CUDA_VISIBLE_DEVICES": "3,5, 6"}) == [3, 5, 6]
    assert bw.visible_device_ids({"CUDA_VISIBLE_DEVICES": "GPU-abcdef"}) is None  # UUIDs carry no index
    assert bw.physical_gpu_id(1, [3, 5, 6]) == 5 and bw.physical_gpu_id(4, [3, 5, 6]) == 5 and bw.physical_gpu_id(2, None) == 2 or bw._VISIBLE_GPU_IDS
    path = bw.gpu_lock_path(1, str(tmp_path / "locks"), visible=[3, 5, 6])
    assert path.endswith("gpu_5.lock") and os.path.isdir(tmp_path / "locks")
    assert bw.GPU_LOCK_DIR.endswith("aster-gpu-locks")  # the reference's directory: both harnesses take turns


def test_gpu_lock_excludes_a_second_holder(tmp_path):
    path = str(tmp_path / "gpu_0.lock")
    order = []

    def second():
        with bw.gpu_lock(path):
            order.append("second")

    with bw.gpu_lock(path):
        t = threading.Thread(target=second)
        t.start()
        time.sleep(0.2)
        order.append("first still holds")
    t.join(timeout=5)
    assert order == ["first still holds", "second"]
    with bw.gpu_lock(None):  # no path: no lock
        pass


def test_worker_survives_crash_kill_and_hang():
    w = bw.PersistentGpuWorker(0, loop_fn=fake.timing_loop)
    try:
        assert w.execute(item("a_ns500")) == ("a_ns500", [500, 500, 500], None)
        assert w.spawns == 1
        assert w.execute(item("b_ns700", 2)) == ("b_ns700", [700, 700], None) and w.spawns == 1  # same child
        label, times, err = w.execute(item("crash_here"))
        assert (label, times) == ("crash_here", None) and err == "worker crash (exit 7)"
        assert w.execute(item("c_ns900", 1)) == ("c_ns900", [900], None) and w.spawns == 2  # fresh child
        label, times, err = w.execute(item("kill_here"))
        assert times is None and err == "worker crash (signal 9)"
        t0 = time.monotonic()
        label, times, err = w.execute(item("hang_here"), timeout=1.0)
        assert times is None and "timed out after 1s" in err and time.monotonic() - t0 < 20
        assert w.execute(item("d_ns100", 1)) == ("d_ns100", [100], None) and w.spawns == 4
        label, times, err = w.execute(item("raise_here"))
        assert times is None and err.startswith("CUDA error at") and w.spawns == 4  # an error is not a crash
    finally:
        w.shutdown()
    w.shutdown()  # idempotent


def test_run_gpu_queue_list_and_live_queue():
    out = queue.Queue()
    bw.run_gpu_queue(0, [item("x_ns10", 1), item("crash"), item("y_ns20", 1)], out, loop_fn=fake.timing_loop)
    got = [out.get_nowait() for _ in range(3)]
    assert [g[0] for g in got] == ["x_ns10", "crash", "y_ns20"] and got[1][1] is None and got[2][1] == [20]
    live, out2 = queue.Queue(), queue.Queue()
    t = threading.Thread(target=bw.run_gpu_queue, args=(1, live, out2), kwargs=dict(loop_fn=fake.timing_loop))
    t.start()
    live.put(item("p_ns30", 1))
    assert out2.get(timeout=30) == ("p_ns30", [31], None)  # worker index 1 adds 1 ns
    live.put(None)
    t.join(timeout=30)
    assert not t.is_alive()


def test_run_on_gpus_round_robin_results_and_failures(tmp_path):
    cfgs = [FakeCfg(f"cfg{i}_ns{1000 * (i + 1)}") for i in range(5)] + [FakeCfg("crash_cfg"), FakeCfg("not_compiled_ns5")]
    paths = {c.label: "unused" for c in cfgs[:-1]}
    results_file = tmp_path / "results.jsonl"
    results, failed = bw.run_on_gpus(cfgs, paths, 25, 2, bench="fake_bench", results_file=str(results_file), loop_fn=fake.timing_loop,
                                     lock_dir=str(tmp_path / "locks"))
    assert sorted(c.label for c, _ in results) == sorted(c.label for c in cfgs[:5])
    assert [(c.label, why) for c, why in failed] == [("crash_cfg", "worker crash (exit 7)")]
    by = {c.label: s for c, s in results}
    assert isinstance(by["cfg0_ns1000"], PerfStats) and by["cfg0_ns1000"].p50_ns in (1000.0, 1001.0)
    lines = [l for l in results_file.read_text().splitlines() if l.startswith("BENCH_RESULT_JSON:")]
    assert len(lines) == 5 and json.loads(lines[0].split(":", 1)[1])["bench"] == "fake_bench"
    # too few iterations: nothing is left after the warm-up launches are dropped
    res2, failed2 = bw.run_on_gpus(cfgs[:1], paths, 5, 1, loop_fn=fake.timing_loop, use_locks=False)
    assert res2 == [] and failed2[0][1] == "no valid measurements"


def test_verify_on_gpus_and_top_configs(tmp_path):
    cfgs = [FakeCfg("good1"), FakeCfg("wrong2"), FakeCfg("good3"), FakeCfg("crash4"), FakeCfg("good5")]
    paths = {c.label: "unused" for c in cfgs}
    passed, errors = bw.verify_on_gpus(cfgs, paths, 2, loop_fn=fake.verify_loop, lock_dir=str(tmp_path))
    assert passed == 3 and sorted(errors) == ["crash4: worker crash (exit 9)", "wrong2: numeric: max_abs_diff=1.5 mismatched=3"]
    stats = _compute_stats([1000.0], 10, 1.0)
    ok = bw.verify_top_configs([(c, stats) for c in cfgs], paths, top_n=3, num_gpus=1, loop_fn=fake.verify_loop, lock_dir=str(tmp_path))
    assert ok == {"good1", "good3"}


def test_workers_of_one_physical_gpu_take_turns(tmp_path):
    """Two workers mapped to the same physical GPU (here: the same lock file) never hold it at once."""
    lock = str(tmp_path / "gpu_0.lock")
    outs = [queue.Queue(), queue.Queue()]
    threads = [threading.Thread(target=bw.run_gpu_queue, args=(i, [item(f"w{i}a"), item(f"w{i}b")], outs[i]),
                                kwargs=dict(loop_fn=fake.lock_probe_loop, lock_path=lock)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    spans = sorted(tuple(o.get_nowait()[1]) for o in outs for _ in range(2))
    assert len(spans) == 4
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 <= b0, "two holders overlapped"


def test_pipelined_sweep_with_fake_workers(tmp_path):
    cfgs = [FakeCfg(f"ok{i}_ns{2000 - 100 * i}") for i in range(4)] + [FakeCfg("bad_compile_ns1"), FakeCfg("too_big_ns1"), FakeCfg("hang_ns1")]

    def compile_fn(cfg, path):
        if "bad_compile" in cfg.label:
            raise RuntimeError("B200_ERR_INVALID: tile_n=48 unsupported\nsecond line")
        text = json.dumps({"resources": {"smem_bytes": 300000 if "too_big" in cfg.label else 1000}})
        with open(path, "w") as f:
            f.write(text)
        return path, text

    logs = []
    results, paths = bw.bench_perf_sweep_pipelined(
        cfgs, compile_fn, lambda c: f"repro {c.label}", bench="fake", num_gpus=2, iterations=30, hsaco_dir=str(tmp_path / "art"),
        post_compile_filter=lambda cfg, res: "smem: too much -- details" if res["smem_bytes"] > 232448 else None,
        results_file=str(tmp_path / "r.jsonl"), exec_timeout=1.0, loop_fn=fake.timing_loop, lock_dir=str(tmp_path / "locks"), log=logs.append)
    assert [c.label for c, _ in results] == ["ok3_ns1700", "ok2_ns1800", "ok1_ns1900", "ok0_ns2000"]  # fastest first
    assert set(paths) == {c.label for c in cfgs} - {"bad_compile_ns1"}
    text = "\n".join(logs)
    assert "compile: B200_ERR_INVALID: tile_n=48 unsupported: bad_compile_ns1 | repro: repro bad_compile_ns1" in text
    assert "compile: smem: too much: too_big_ns1" in text and "execution timed out after 1s: hang_ns1" in text
    assert len((tmp_path / "r.jsonl").read_text().splitlines()) == 4
    # compile only: artifacts, no execution
    res0, paths0 = bw.bench_perf_sweep_pipelined(cfgs[:2], compile_fn, None, num_gpus=0, hsaco_dir=str(tmp_path / "art"), log=logs.append)
    assert res0 == [] and len(paths0) == 2


def test_real_worker_loop_reports_a_truncated_artifact(tmp_path, native_lib):
    """The library's own worker loop, on the host only: the plan artifact was cut short on disk,
    so loading it fails before anything reaches a device, and the failure comes back as a result."""
    cfg = make_b200_instance(256, 256, 256)
    path, text = compile_multitile_gemm(cfg, str(tmp_path / "cut.b200plan.json"))
    with open(path, "w") as f:
        f.write(text[: len(text) // 2])
    w = bw.PersistentGpuWorker(0)  # persistent_worker_loop
    try:
        label, times, err = w.execute(bw.work_item(cfg, path, 3), timeout=120)
    finally:
        w.shutdown()
    assert label == cfg.label and times is None and err


def test_cli_builders():
    ap = argparse.ArgumentParser()
    bw.add_sweep_cli_args(ap)
    a = ap.parse_args(["--mcpu", "sm_100a", "--compile-only", "--num-gpus", "2", "--init", "zero", "--no-direct-b", "--tier-time-budget", "5"])
    assert (a.mcpu, a.compile_only, a.num_gpus, a.init.value, a.direct_b, a.iterations, a.compile_sample) == ("sm_100a", True, 2, "zero", False, 100, 512)
    with pytest.raises(SystemExit):
        ap.parse_args([])  # --mcpu is required
    ap1 = argparse.ArgumentParser()
    bw.add_single_cli_args(ap1)
    s = ap1.parse_args(["--mcpu", "sm_100a", "--hsaco", "x.json", "--print-asm"])
    assert s.hsaco == "x.json" and s.print_asm and s.num_wg_per_cu == 1
    bw.require_gpu_or_compile_only(argparse.Namespace(compile_only=True, mcpu="sm_100a"))  # returns


# ---------------------------------------------------------------------------------------------
# tiers
# ---------------------------------------------------------------------------------------------
class AxisItem:
    total_flops = 2 * 256 ** 3
    mapping = FakeMapping()
    spec = FakeSpec()

    def __init__(self, d):
        self.d = dict(d)
        self.label = "_".join(f"{k}{v}" for k, v in sorted(d.items()))


def tier_grid():
    return (SweepGrid().axis("tile", [32, 64, 128, 256]).axis("stages", [2, 3, 4, 5, 6]).axis("split", [1, 2, 4])
            .filter("tile", "stages", check=lambda d: d["tile"] * d["stages"] <= 1024, name="fits")
            .build_with(AxisItem))


def fake_speed(d):  # best at tile 128, stages 5, split 1
    return 1000.0 - abs(d["tile"] - 128) - 40 * abs(d["stages"] - 5) - 25 * (d["split"] - 1)


def test_tier_overrides_and_neighbors():
    assert bt.ordinal_neighbors(64, [32, 64, 128, 256], 1) == [32, 64, 128]
    assert bt.ordinal_neighbors(256, [32, 64, 128, 256], 2) == [64, 128, 256] and bt.ordinal_neighbors(7, [1, 2], 1) == [7]
    t2 = bt.TierSpec(2, 10, 0, ("fits",), free_axes=["stages"], neighbor_radius={"tile": 1}, fixed_axes={"split": 1})
    universe = tier_grid().axis_values()
    over = bt.tier_axis_overrides(universe, t2, [{"tile": 64, "stages": 3, "split": 2, "_tflops": 5.0}], {"split": 4})
    assert over == {"tile": [128, 32, 64], "stages": [2, 3, 4, 5, 6], "split": [4]}  # ambient pin beats the tier's own pin
    g = tier_grid()
    bt.apply_tier_overrides(g, bt.TierSpec(1, 10, 0, (), fixed_axes={"stages": 6}), [])
    assert g.axis_values()["stages"] == [6] and g.filter_names() == ()  # the named filter was dropped
    with pytest.raises(ValueError, match="no values"):
        bt.apply_tier_overrides(tier_grid(), bt.TierSpec(1, 10, 0, (), axis_grid={"tile": []}), [])
    assert bt.keep_count(1000) == 100 and bt.keep_count(200) == 50 and bt.keep_count(7) == 7
    assert bt.make_constraints(tier_grid()) == ("fits",)


def test_tier_mode_converges_and_emits_only_verified():
    calls = []

    def sweep(instances):
        calls.append([i.label for i in instances])
        res = [(inst, _compute_stats([inst.total_flops / fake_speed(inst.d) * 1e-3], inst.total_flops, 2250.0)) for inst in instances]
        return res, {inst.label: "p" for inst in instances}

    schedule = [
        bt.TierSpec(1, 8, 1, ("fits",), fixed_axes={"stages": 3, "split": 1}, discriminator="tile", per_stratum_diversity=True),
        bt.TierSpec(2, 12, 2, ("fits",), free_axes=["stages"], neighbor_radius={"tile": 0}),
    ]
    out = io.StringIO()
    ranked = bt.run_tier_mode(grid_factory=tier_grid, tier_schedule=schedule, sweep_fn=sweep, bench_label="tier_test", results_stream=out,
                              verify_fn=lambda results, paths: {results[0][0].label, results[2][0].label}, log=lambda *_: None)
    assert len(calls) == 2 and len(calls[0]) == 4  # one per tile in tier 1
    assert ranked[0][0].d == {"tile": 128, "stages": 5, "split": 1}
    lines = [l for l in out.getvalue().splitlines() if l.startswith("BENCH_RESULT_JSON:")]
    assert len(lines) == 2 and json.loads(lines[0].split(":", 1)[1])["label"] == ranked[0][0].label
    # dry run: the first tier's labels, nothing executed
    seen = []
    assert bt.run_tier_mode(grid_factory=tier_grid, tier_schedule=schedule, sweep_fn=sweep, dry_run=True, log=seen.append) == []
    assert len(calls) == 2 and sum("stages3" in s for s in seen) == 4


def test_b200_schedule_runs_on_the_plan_grid():
    from aster_b200.bench_search import b200_gemm_grid

    sched = bt.b200_tier_schedule(seed=1, cap=6)
    g = b200_gemm_grid(4096, 4096, 4096)
    bt.apply_tier_overrides(g, sched[0], [])
    inst, cfgs, total = g.generate(sample_size=sched[0].max_configs, stratification_key=lambda d: (d["tile_n"], d["cta_group"]))
    assert total == 6 and all(c["stages"] == 0 and c["split_k"] == 0 for c in cfgs)
    g2 = b200_gemm_grid(4096, 4096, 4096)
    bt.apply_tier_overrides(g2, sched[1], [dict(cfgs[-1], _tflops=1.0)], universe=b200_gemm_grid(4096, 4096, 4096).axis_values())
    vals = g2.axis_values()
    assert vals["stages"] == [0, 3, 4, 5, 6] and vals["cta_group"] == [cfgs[-1]["cta_group"]]


# ---------------------------------------------------------------------------------------------
# re-measuring the registry
# ---------------------------------------------------------------------------------------------
def test_measure_all_writes_only_verified_results(tmp_path):
    reg = pt.load_registry()
    assert hooks_for_bench(BENCH_HOOKS["bench_label"])["from_label"] is BENCH_HOOKS["from_label"]
    assert hooks_for_bench(BENCH_HOOKS["bench_label"] + "_fp8")["bench_label"].endswith("_fp8") and hooks_for_bench("something_else") is None
    todo = pt.collect_todo(reg, mcpu_filter="sm_100a")
    assert todo and all(labels for labels in todo.values())
    swept = []

    def sweep(configs, compile_fn, repro_cmd_fn, **kw):
        swept.append((kw["bench"], [c.label for c in configs], kw["num_gpus"]))
        res = [(c, _compute_stats([1e6 * (i + 1)], c.total_flops, 2250.0)) for i, c in enumerate(configs)]
        return res, {c.label: "p" for c in configs}

    def verify(ranked, paths, *, top_n, num_gpus):
        assert top_n == len(ranked)
        return {c.label for c, _ in ranked[:-1]}  # the slowest one fails verification

    out = tmp_path / "eval.jsonl"
    out.write_text("stale line\n")
    pt.measure_all(reg, str(out), mcpu_filter="sm_100a", num_gpus=1, sweep_fn=sweep, verify_fn=verify, log=lambda *_: None)
    recs = list(pt.parse_jsonl_results(out.read_text().splitlines()))
    stored = sum(len(v) for v in todo.values())
    assert len(swept) == len(todo) and len(recs) == stored - len(todo) and "stale" not in out.read_text()
    assert {r.key.bench for r in recs} == {bench for (_, bench) in todo}
    # every stored label parses back into a config through the bench's from_label hook
    assert all(lbl in {l for _, labels, _ in swept for l in labels} for labels in todo.values() for lbl in labels)
    # compile only: nothing is emitted
    pt.measure_all(reg, str(out), compile_only=True, sweep_fn=lambda *a, **k: ([], {}), verify_fn=verify, log=lambda *_: None)
    assert out.read_text() == ""
