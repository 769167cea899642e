"""Registry and dashboard tooling on synthetic result logs, following the reference's
contrib/kittens/test/bench/tools/smoke_check.sh (:35-102): merge new labels into a one-entry
slot, list the registry, all-OK dashboard, and a regression that must exit with code 1."""

import io
import json

import pytest

from aster_b200 import perf_tools as pt

BENCH = "bench_perf_102_gemm_multitile_lds_sm100"


def line(label, tf, mcpu="sm_100a", bench=BENCH, size=(4096, 4096, 4096), **extra):
    rec = {"mcpu": mcpu, "bench": bench, "M": size[0], "N": size[1], "K": size[2], "label": label, "tflops_median": tf}
    rec.update(extra)
    return pt.RESULT_SENTINEL + json.dumps(rec)


@pytest.fixture
def registry_file(tmp_path):
    path = tmp_path / "best_known.json"
    path.write_text(json.dumps({"sm_100a": {BENCH: {"4096x4096x4096": [{"label": "m4096xn4096xk4096_old_winner", "expected_tflops": 900.0}]}}}))
    return path


def test_parse_skips_noise_and_broken_records():
    text = "\n".join([
        "compiling 3 configs ...",
        line("a", 950.0, tflops_p10=940, tflops_p90="n/a"),
        "prefix " + line("b", 920.0),
        pt.RESULT_SENTINEL + "{broken json",
        pt.RESULT_SENTINEL + json.dumps({"mcpu": "sm_100a", "label": "no size"}),
    ])
    recs = list(pt.parse_jsonl_results(io.StringIO(text)))
    assert [r.label for r in recs] == ["a", "b"]
    assert recs[0].tflops_p10 == 940.0 and recs[0].tflops_p90 is None and recs[0].sample_n == 1
    assert recs[0].key == pt.EntryKey("sm_100a", BENCH, 4096, 4096, 4096)


def test_max_merge():
    recs = list(pt.parse_jsonl_results([line("a", 900.0), line("a", 950.0), line("b", 920.0), line("c", 10.0, size=(512, 512, 512))]))
    by_label = pt.max_merge_by_key_label(recs)
    assert by_label[(recs[0].key, "a")].tflops_median == 950.0 and len(by_label) == 3
    by_key = pt.max_merge_by_key(recs)
    assert by_key[recs[0].key].label == "a" and by_key[recs[3].key].label == "c"


def test_update_merges_into_slot_and_writes_atomically(registry_file, tmp_path, capsys):
    sweep = tmp_path / "sweep.jsonl"
    sweep.write_text("\n".join([line("m4096xn4096xk4096_new_top", 950.0), line("m4096xn4096xk4096_runner", 920.0)]) + "\n")
    before = registry_file.read_text()
    assert pt.main(["update", "--input", str(sweep), "--best-known-file", str(registry_file)]) == 0
    assert registry_file.read_text() == before and "not written" in capsys.readouterr().out  # report only
    assert pt.main(["update", "--input", str(sweep), "--best-known-file", str(registry_file), "--apply"]) == 0
    slot = json.loads(registry_file.read_text())["sm_100a"][BENCH]["4096x4096x4096"]
    assert [(e["label"], e["expected_tflops"]) for e in slot] == [
        ("m4096xn4096xk4096_new_top", 950.0), ("m4096xn4096xk4096_runner", 920.0), ("m4096xn4096xk4096_old_winner", 900.0)]
    assert not (tmp_path / "best_known.json.tmp").exists()
    reg = pt.load_registry(registry_file)
    assert pt.best_known(reg, "sm_100a", BENCH, 4096, 4096, 4096) == "m4096xn4096xk4096_new_top"
    assert pt.best_known(reg, "sm_100a", BENCH, 1, 2, 3) is None


def test_slot_keeps_top_n_and_values_only_rise():
    reg = {}
    recs = list(pt.parse_jsonl_results([line(f"l{i}", 100.0 + i) for i in range(8)]))
    pt.merge_results_into_registry(reg, recs)
    slot = reg["sm_100a"][BENCH]["4096x4096x4096"]
    assert [e["label"] for e in slot] == ["l7", "l6", "l5", "l4", "l3"]
    assert pt.merge_results_into_registry(reg, list(pt.parse_jsonl_results([line("l7", 50.0)]))) == []
    assert slot[0]["expected_tflops"] == 107.0
    assert pt.size_key(1, 2, 3) == "1x2x3" and pt.parse_size_key("4x5x6") == (4, 5, 6)


def test_dashboard_statuses_and_exit_codes(registry_file, tmp_path, capsys):
    sweep = tmp_path / "sweep.jsonl"
    sweep.write_text("\n".join([line("m4096xn4096xk4096_new_top", 950.0), line("m4096xn4096xk4096_runner", 920.0)]) + "\n")
    pt.main(["update", "--input", str(sweep), "--best-known-file", str(registry_file), "--apply"])
    capsys.readouterr()

    assert pt.main(["dashboard", "--dry-run", "--best-known-file", str(registry_file)]) == 0
    assert "3 stored entries listed" in capsys.readouterr().out

    reg = pt.load_registry(registry_file)
    same = tmp_path / "dash.jsonl"
    same.write_text("\n".join(line(e["label"], e["expected_tflops"]) for e in reg["sm_100a"][BENCH]["4096x4096x4096"]) + "\n")
    assert pt.main(["dashboard", "--measurements", str(same), "--best-known-file", str(registry_file)]) == 0
    out = capsys.readouterr().out
    assert "3 OK" in out and "0 REGRESS" in out

    regress = tmp_path / "regress.jsonl"
    regress.write_text(same.read_text().replace("950.0", "700.0"))
    assert pt.main(["dashboard", "--measurements", str(regress), "--best-known-file", str(registry_file)]) == 1
    assert "REGRESS" in capsys.readouterr().out.splitlines()[1]  # worst status sorts first

    missing = tmp_path / "missing.jsonl"
    missing.write_text("\n".join(same.read_text().splitlines()[:2]) + "\n")
    assert pt.main(["dashboard", "--measurements", str(missing), "--best-known-file", str(registry_file)]) == 2
    assert "1 MISS" in capsys.readouterr().out


def test_margins():
    assert pt.status_of(None, 100.0) == "MISS"
    assert pt.status_of(94.9, 100.0) == "REGRESS" and pt.status_of(95.0, 100.0) == "OK"
    assert pt.status_of(103.0, 100.0) == "OK" and pt.status_of(103.1, 100.0) == "IMPROVE"
    assert pt.status_of(96.0, 100.0, regress_margin=0.01) == "REGRESS"
