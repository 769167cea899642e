"""bench.py's host-side pieces without a GPU: the workload table, the shared config object, the
roofline arithmetic, the DRAM-traffic records that are only quoted for unchanged kernel sources,
and the verification roll-up that decides the exit code."""

import importlib.util
import os
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_workload_table_covers_the_configured_problems(bench):
    for name in ("bf16_4096", "fp16_512", "bf16_8192", "fused_8192x8192x2048", "fp8_8192", "decode_16", "decode_128", "vector_add",
                 "copy_2d_padded", "sharded_65536"):
        assert name in bench.WORKLOADS
    assert bench.DEFAULT_WORKLOAD == "bf16_4096" and set(bench.EXTRA_WORKLOADS) <= set(bench.WORKLOADS)
    w = bench.WORKLOADS["sharded_65536"]
    assert (w["M"], w["N"], w["K"], w["seed"], w.get("strong")) == (65536, 8192, 8192, 4, True)
    assert bench.WORKLOADS["fused_8192x8192x2048"]["epilogue"] == "bias_relu"
    assert (bench.REF_LAUNCHES, bench.REF_DROP) == (100, 20)  # the reference's protocol


def test_config_object_is_the_same_for_both_arms(bench):
    w = bench.WORKLOADS["bf16_4096"]
    c1, c8 = bench.common_config(w, "bf16_4096", 1), bench.common_config(w, "bf16_4096", 8)
    assert c1["per_gpu_shape"] == [4096, 4096, 4096] and c1["global_rows"] == 4096 and c8["global_rows"] == 8 * 4096
    s = bench.common_config(bench.WORKLOADS["sharded_65536"], "sharded_65536", 8)
    assert s["per_gpu_shape"] == [8192, 8192, 8192] and s["global_rows"] == 65536
    assert set(c1) == {"workload", "name", "per_gpu_shape", "global_rows", "parallelism"}


def test_roofline_arithmetic(bench, monkeypatch):
    monkeypatch.setattr(bench, "measured_peaks", lambda: {"hbm_gbs": 6000.0, "bf16_tflops": 1600.0, "bf16_tflops_sustained": 1300.0, "_source": "test"})
    case = types.SimpleNamespace(w={"dtype_ab": "bf16"}, flops=2.0 * 4096 ** 3, algorithmic_bytes=0.0)
    r = bench.roofline_of(case, 0.1, sustained=False, sm_mhz=1500.0)
    assert r["bound"] == "tensor" and r["achieved"] == pytest.approx(1374.39, rel=1e-4) and r["frac"] == pytest.approx(1374.39 / 1600, rel=1e-4)
    assert r["frac_of_nominal"] == pytest.approx(1374.39 / 2250, rel=1e-4)
    assert r["frac_of_clock_peak"] == pytest.approx(1374.39 / (148 * 8192 * 1500e6 / 1e12), rel=1e-4)
    assert bench.roofline_of(case, 0.1, sustained=True, sm_mhz=None)["peak"] == 1300.0
    fp8 = types.SimpleNamespace(w={"dtype_ab": "e4m3"}, flops=2.0 * 8192 ** 3, algorithmic_bytes=0.0)
    r8 = bench.roofline_of(fp8, 0.36, sustained=False, sm_mhz=1300.0)
    assert r8["peak"] == 3200.0 and r8["frac_of_nominal"] == pytest.approx(r8["achieved"] / 4500.0)
    assert r8["frac_of_clock_peak"] == pytest.approx(r8["achieved"] / (148 * 16384 * 1300e6 / 1e12))
    skinny = types.SimpleNamespace(w={"dtype_ab": "bf16", "hbm": True}, flops=1.0, algorithmic_bytes=134.5e6)
    rs = bench.roofline_of(skinny, 0.027, sustained=False, sm_mhz=1800.0)
    assert rs["bound"] == "hbm" and rs["unit"] == "GB/s" and rs["achieved"] == pytest.approx(134.5e6 / 0.027e-3 / 1e9)


def test_traffic_records_are_quoted_only_for_unchanged_kernel_sources(bench, tmp_path, monkeypatch):
    digest = bench.kernel_source_digest()
    assert len(digest) == 16
    prof = tmp_path / "profiles"
    prof.mkdir()
    (prof / "a.md").write_text(f"text\ntraffic-record: workload=w_now dram_bytes_per_launch=89.65e6 kernel_sources={digest}\n"
                               "traffic-record: workload=w_old dram_bytes_per_launch=1e6 kernel_sources=0123456789abcdef\n")
    (prof / "ignored.json").write_text("traffic-record: workload=w_json dram_bytes_per_launch=5 kernel_sources=" + digest)
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    monkeypatch.setattr(bench, "kernel_source_digest", lambda: digest)
    now = bench.dram_traffic("w_now")
    assert now["traffic"] == 89.65e6 and "profiles/a.md" in now["traffic_source"]
    old = bench.dram_traffic("w_old")
    assert old["traffic"] is None and "0123456789abcdef" in old["traffic_source"]
    assert bench.dram_traffic("w_json")["traffic"] is None and bench.dram_traffic("nothing")["traffic"] is None


def test_committed_traffic_records_parse(bench):
    """Every record under profiles/ is well formed; those of the current kernel sources are quoted."""
    import re

    found = 0
    for fn in os.listdir(os.path.join(ROOT, "profiles")):
        for line in open(os.path.join(ROOT, "profiles", fn)):
            if line.startswith("traffic-record:"):
                m = re.match(r"traffic-record:\s+workload=(\S+)\s+dram_bytes_per_launch=(\S+)\s+kernel_sources=([0-9a-f]{16})$", line.strip())
                assert m, line
                assert m.group(1) in bench.WORKLOADS and float(m.group(2)) > 0
                found += 1
    assert found >= 5


def test_verification_roll_up(bench):
    line = {"verified": True, "e2e": {"matches_device_result": True}, "workloads": {"a": {"verified": True}, "b": {"verified": True}},
            "strong_65536": {"verified": True}}
    assert bench.all_verified(line)
    for breaker in (lambda d: d.update(verified=False), lambda d: d["e2e"].update(matches_device_result=False),
                    lambda d: d["workloads"]["b"].update(verified=False), lambda d: d["strong_65536"].update(verified=False)):
        import copy

        bad = copy.deepcopy(line)
        breaker(bad)
        assert not bench.all_verified(bad)
    assert bench.all_verified({"verified": True})  # a single-workload line
