"""Sweep search without a GPU: grid enumeration / pruning / sampling semantics (the reference's
tier tests use a fake axis universe the same way, contrib/kittens/test/bench/test_tiered_sweep.py:23-129)
and the sweep runner driven by a fake execute function."""

import io
import json

import numpy as np
import pytest

from aster_b200 import perf_tools as pt
from aster_b200.bench_search import SweepGrid, b200_gemm_grid, run_sweep
from aster_b200.dtypes import to_f32


class Item:
    def __init__(self, d):
        self.d = dict(d)
        self.label = "_".join(f"{k}{v}" for k, v in sorted(d.items()))


def small_grid():
    return (SweepGrid().axis("a", [1, 2, 3, 4]).axis("b", [1, 2, 3]).axis("c", ["x", "y"])
            .filter("a", check=lambda d: d["a"] != 4, name="no_four")
            .filter("a", "b", check=lambda d: d["a"] % d["b"] == 0, name="b_divides_a")
            .build_with(Item))


def test_enumeration_applies_filters_at_the_shallowest_level():
    calls = []
    grid = (SweepGrid().axis("a", [1, 2]).axis("b", [1, 2, 3])
            .filter("a", check=lambda d: calls.append(dict(d)) or d["a"] == 1).build_with(Item))
    inst, cfgs, total = grid.generate(sample_size=0)
    assert total == 3 and [c["b"] for c in cfgs] == [1, 2, 3]
    assert calls == [{"a": 1}, {"a": 2}]  # checked once per value of `a`, before `b` is bound


def test_filters_sampling_and_names():
    grid = small_grid()
    inst, cfgs, total = grid.generate(sample_size=0)
    expect = [(a, b, c) for a in (1, 2, 3) for b in (1, 2, 3) if a % b == 0 for c in "xy"]
    assert total == len(expect) == 10 and [(c["a"], c["b"], c["c"]) for c in cfgs] == expect
    assert grid.filter_names() == ("no_four", "b_divides_a")
    sampled, _, total2 = grid.generate(sample_size=4, seed=1)
    assert total2 == 10 and len(sampled) == 4
    again, _, _ = grid.generate(sample_size=4, seed=1)
    assert [i.label for i in again] == [i.label for i in sampled]  # reproducible
    strat, cfgs_s, _ = grid.generate(sample_size=3, stratification_key=lambda d: d["a"], seed=0)
    assert sorted(c["a"] for c in cfgs_s) == [1, 2, 3]  # one per stratum


def test_restrict_retain_extras_and_errors():
    grid = small_grid()
    grid.restrict_axes({"a": [2, 4], "c": ["x"]})
    grid.retain_filters({"b_divides_a"})
    _, cfgs, total = grid.generate(sample_size=0)
    assert [(c["a"], c["b"]) for c in cfgs] == [(2, 1), (2, 2), (4, 1), (4, 2)] and total == 4
    extras = [{"a": 2, "b": 2, "c": "x"}, {"a": 2, "b": 3, "c": "x"}, {"a": 2, "b": 2, "c": "x"}]  # 2nd rejected, 3rd duplicate
    _, cfgs, total = grid.generate(sample_size=1, extra_eligible=extras)
    assert total == 4 and cfgs == [{"a": 2, "b": 2, "c": "x"}]  # the extra uses up the whole budget
    with pytest.raises(ValueError, match="unknown axis"):
        SweepGrid().axis("a", [1]).filter("zz", check=lambda d: True)
    with pytest.raises(ValueError, match="no values"):
        SweepGrid().axis("a", []).build_with(Item).generate()
    dup = SweepGrid().axis("a", [1, 2]).build_with(lambda d: Item({"fixed": 0}))
    inst, _, _ = dup.generate(sample_size=0)
    assert len(inst) == 1  # duplicate labels collapse


def test_b200_grid_is_legal_everywhere(native_lib):
    from aster_b200.gemm import GemmPlan

    inst, cfgs, total = b200_gemm_grid(4096, 4096, 4096).generate(sample_size=0)
    assert total == len(inst) > 20 and len({i.label for i in inst}) == len(inst)
    for i, c in zip(inst, cfgs):
        r = GemmPlan(**i.plan_kwargs()).resources()  # every generated config passes plan validation
        assert r.tile_n == c["tile_n"] and r.cta_group == c["cta_group"] and r.smem_bytes <= 232448
        assert (c["stages"] == 0 or r.stages == c["stages"]) and r.split_k == max(1, c["split_k"])
    skinny, cfgs_s, _ = b200_gemm_grid(16, 8192, 8192).generate(sample_size=0)
    assert skinny and all(c["cta_group"] == 1 for c in cfgs_s)


def test_run_sweep_ranks_verifies_and_emits(native_lib):
    inst, cfgs, _ = b200_gemm_grid(256, 256, 512, "bf16", "f32").generate(sample_size=0)
    inst = inst[:5]
    speed = {c.label: 100.0 + 10 * i for i, c in enumerate(inst)}
    wrong = inst[4].label  # the fastest config computes garbage: it must not be recorded

    def fake_execute(cfg, path, iters, A, B, skip_gpu_check=False, **kw):
        assert json.load(open(path))["label"] == cfg.label
        if cfg is inst[1]:
            raise RuntimeError("CUDA error at x.cu:1 - boom\nsecond line")
        C = to_f32(A, "bf16") @ to_f32(B, "bf16").T
        if cfg.label == wrong:
            C = C + 1.0
        t_ns = cfg.total_flops / speed[cfg.label] * 1e-3
        return C.reshape(-1).astype(np.float32), [t_ns] * iters

    out = io.StringIO()
    ranked = run_sweep(inst, iterations=30, results_stream=out, verify_top=3, execute_fn=fake_execute, log=lambda *_: None)
    labels = [r[0] for r in ranked]
    assert labels[0] == wrong and "FAILED verification" in ranked[0][2]
    assert ranked[1][2] == "verified" and ranked[2][2] == "verified" and ranked[3][2] == ""
    assert ranked[-1][1] is None and ranked[-1][2] == "CUDA error at x.cu:1 - boom"
    recs = list(pt.parse_jsonl_results(out.getvalue().splitlines()))
    assert [r.label for r in recs] == labels[1:3] and recs[0].tflops_median == pytest.approx(speed[labels[1]], rel=1e-6)
    assert recs[0].key == pt.EntryKey("sm_100a", "bench_perf_102_gemm_multitile_lds_sm100", 256, 256, 512)
