"""The operator surface against fixtures produced by the reference's own pure-Python layer
(tests/golden/make_golden.py): labels, derived quantities, resource estimates, init modes,
statistics, pipeline table, cooperative split."""

import hashlib
import pickle

import numpy as np
import pytest

from aster_b200 import bench_harness as bh
from aster_b200 import kittens_helpers as kh
from aster_b200.gemm_config import (
    B200GemmInstance, GemmMappingSpec, GemmSpec, LoadType, Operand, OperandPath, WeakScaledMappedGemmInstance,
    make_b200_instance, mfma_shape_for_mcpu,
)


def build_case(case):
    var = dict(case["variant"])
    if "load_type" in var:
        var["load_type"] = LoadType(var["load_type"])
    if "operand_path" in var:
        var["operand_path"] = OperandPath(var["operand_path"])
    spec = GemmSpec.from_sizes(case["M"], case["N"], case["K"])
    mapping = GemmMappingSpec(case["wg"], case["waves"], case["tpw"], pipeline_strategy=case["pipeline_strategy"], **var)
    return WeakScaledMappedGemmInstance(spec, mapping)


def test_labels_and_estimates_match_reference(golden):
    assert len(golden["label_cases"]) >= 200
    for case in golden["label_cases"]:
        cfg = build_case(case)
        assert cfg.label == case["label"]
        for key in ("total_flops", "num_threads", "num_workgroups", "num_tiles_per_workgroup", "k_scaling_factor",
                    "lds_bytes", "estimated_vgprs", "estimated_agprs", "simd_occupancy", "kernel_name"):
            assert getattr(cfg, key) == case[key], (key, case["label"])
        assert list(cfg.spec.operand_layout(Operand.A).strides) == case["strides_a"]
        assert list(cfg.spec.operand_layout(Operand.C).strides) == case["strides_c"]


def test_label_roundtrip(golden):
    fields = ["gemm_size", "pipeline_strategy", "load_type", "num_wg_per_cu", "lcm_unroll", "unroll_factor_multiplier",
              "epilogue_peeling", "ll_sched", "hoist_wait", "rotate_compute_stage", "use_conservative_barriers",
              "num_workgroups_per_kernel", "num_waves_per_workgroup", "num_tiles_per_workgroup", "num_threads"]
    for case in golden["label_cases"]:
        if case["variant"].get("operand_path"):
            continue  # the label does not carry the operand path (same in the reference)
        cfg = build_case(case)
        back = WeakScaledMappedGemmInstance.from_label(case["label"])
        assert back.label == case["label"]
        for f in fields:
            assert getattr(back, f) == getattr(cfg, f), f


def test_from_label_rejects_garbage_and_truncated(golden):
    with pytest.raises(ValueError, match="Cannot parse label"):
        WeakScaledMappedGemmInstance.from_label("not_a_valid_label")
    with pytest.raises(ValueError):
        WeakScaledMappedGemmInstance.from_label(golden["label_cases"][0]["label"][:-5])


def test_weak_scale_violation_message(golden):
    with pytest.raises(AssertionError) as e:
        WeakScaledMappedGemmInstance(GemmSpec.from_sizes(100, 64, 64), GemmMappingSpec([1, 1, 1], [1, 1, 1], [4, 4, 1]))
    assert str(e.value) == golden["weak_scale_error"]


def test_registry_labels(golden):
    """Labels stored in the reference's best_known.json predate the mandatory ``_consbar``
    token: the strict parser rejects them (as the reference's does), the lenient one reads them."""
    assert golden["best_known_labels"]
    for label in golden["best_known_labels"]:
        with pytest.raises(AssertionError, match="Round-trip failed"):
            B200GemmInstance.from_label(label)
        cfg = B200GemmInstance.from_label(label, strict=False)
        m, n, k = cfg.gemm_size
        assert label.startswith(f"m{m}xn{n}xk{k}_")
        assert cfg.mapping.use_conservative_barriers is False
        assert cfg.tile_n in (128, 256) and cfg.plan_kwargs()["M"] == m


def test_pickle_and_delegation(golden):
    cfg = build_case(golden["label_cases"][3])
    clone = pickle.loads(pickle.dumps(cfg))
    assert clone.label == cfg.label and clone.pipeline_strategy == cfg.mapping.pipeline_strategy
    with pytest.raises(AttributeError):
        cfg.no_such_attribute


def test_pipeline_strategies_table(golden):
    assert {str(k): v for k, v in kh.PIPELINE_STRATEGIES.items()} == golden["pipeline_strategies"]
    for k, want in golden["pipeline_strategy_stages"].items():
        assert list(kh.pipeline_strategy_stages(int(k))) == want


def test_coop_2d_split(golden):
    for row in golden["coop_2d_split"]:
        assert list(kh.coop_2d_split(*row["args"])) == row["result"], row["args"]


def test_init_array_modes(golden):
    assert {m.value for m in bh.InitMode} == {k.split("/")[0] for k in golden["init_array"]}
    for key, want in golden["init_array"].items():
        mode, role = key.split("/")
        arr = bh.init_array((24, 40), mode, role, dtype=np.float16, seed=42)
        assert arr.reshape(-1)[:8].astype(np.float64).tolist() == want["first8"], key
        assert hashlib.sha256(arr.tobytes()).hexdigest() == want["sha256"], key


def test_compute_stats(golden):
    g = golden["compute_stats"]
    s = bh._compute_stats(g["times_ns"], g["total_flops"], g["peak"])
    for k, v in g["fields"].items():
        assert getattr(s, k) == pytest.approx(v, rel=1e-12), k
    for k, v in g["derived"].items():
        assert getattr(s, k) == pytest.approx(v, rel=1e-12), k
    assert golden["compute_stats_none"] is True
    assert bh._compute_stats([], 1, 1.0) is None and bh._compute_stats([1.0, 0.0], 1, 1.0) is None


def test_peak_table_is_a_superset(golden):
    for mcpu, peak in golden["peak_table"].items():
        assert bh.peak_tflops_f16(mcpu) == peak
    assert bh.peak_tflops("sm_100a", "bf16") == 2250.0 and bh.peak_tflops("sm_100a", "e4m3") == 4500.0
    assert mfma_shape_for_mcpu("gfx950") == [16, 16, 32] and mfma_shape_for_mcpu("sm_100a") == [16, 16, 16]


class TestB200Instance:
    def test_plain_label_is_reference_label(self):
        cfg = make_b200_instance(4096, 4096, 4096, stages=None)
        assert "_b200_" not in cfg.label
        assert WeakScaledMappedGemmInstance.from_label(cfg.label).label == cfg.label
        assert cfg.tile_n == 256 and cfg.stages == 3 and cfg.requested_cta_tile == [128, 256, 32]

    @pytest.mark.parametrize("kw", [
        dict(dtype_ab="bf16", dtype_c="bf16"),
        dict(dtype_ab="e4m3", dtype_c="bf16"),
        dict(dtype_ab="bf16", dtype_c="bf16", epilogue="bias_relu"),
        dict(dtype_ab="bf16", dtype_c="bf16", epilogue="bias", bias_axis="m"),
        dict(dtype_ab="f16", dtype_c="f32", stages=4, split_k=-1),
        dict(dtype_ab="f16", dtype_c="f32", stages=None),
        dict(dtype_ab="f16", dtype_c="f32", stages=0),
        dict(dtype_ab="bf16", dtype_c="f32", epilogue="relu", tile_n=64, split_k=8, cta_group=1),
    ])
    def test_suffix_roundtrip(self, kw):
        cfg = make_b200_instance(1024, 2048, 512, **kw)
        back = B200GemmInstance.from_label(cfg.label)
        assert back.label == cfg.label
        assert back.plan_kwargs() == cfg.plan_kwargs()

    def test_ring_depth_mapping(self):
        assert make_b200_instance(256, 256, 256, stages=None, pipeline_strategy=9).stages == 6  # max(stage) + 1
        auto = make_b200_instance(256, 256, 256)
        assert auto.stages == 0 and auto.label.endswith("_st0") and auto.plan_kwargs()["stages"] == 0
        assert make_b200_instance(256, 256, 256, stages=5).label.endswith("_st5")

    def test_tile_snapping(self):
        # twg_n * 16 = 32 -> 32; 112 -> 64; 400 -> 256
        for tiles, want in ((2, 32), (7, 64), (25, 256)):
            spec = GemmSpec.from_sizes(48, tiles * 16, 128)
            cfg = B200GemmInstance(spec, GemmMappingSpec([1, 1, 1], [1, 1, 1], [3, tiles, 1]))
            assert cfg.tile_n == want

    def test_direct_b_maps_to_preshuffled_layout(self):
        cfg = make_b200_instance(256, 256, 256, operand_path=OperandPath.DIRECT_B)
        assert cfg.plan_kwargs()["b_layout"] == "ref_preshuffled" and cfg.mapping.direct_b

    def test_transfer_tile_geometry(self):
        # test_102_gemm_python_multitile_lds_cdna3.py:372-388: 32 K elements, 64-byte rows, 1024 bytes.
        cfg = make_b200_instance(256, 256, 256)
        assert (cfg.transfer_tile_k_elems, cfg.transfer_tile_row_bytes, cfg.transfer_tile_bytes) == (32, 64, 1024)

    def test_type_mismatch_is_rejected(self):
        spec = GemmSpec.from_sizes(128, 128, 128)
        mapping = GemmMappingSpec([1, 1, 1], [1, 1, 1], [8, 8, 1])
        with pytest.raises(ValueError):
            B200GemmInstance(spec, mapping, dtype_ab="e4m3")
        with pytest.raises(ValueError):
            B200GemmInstance(spec, mapping, dtype_c="bf16")
