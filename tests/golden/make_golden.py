"""Generates ``reference_golden.json`` from the reference's own pure-Python layer.

Run in a container that has the reference checkout (it cannot run where the reference is
absent; the committed JSON is what the tests read):

    python tests/golden/make_golden.py <path to the iree-org/aster checkout>

It imports, read-only, ``kittens.gemm_config``, ``kittens_helpers``, ``bench_harness`` from the
reference tree, evaluates them on fixed inputs and records the outputs: labels and resource
estimates for a grid of (spec, mapping) pairs, ``shuffle_weight`` images, ``init_array``
digests, ``_compute_stats`` results, the pipeline-strategy table, ``coop_2d_split`` results
and the labels stored in the reference's ``best_known.json``.
"""

from __future__ import annotations

import ast
import hashlib
import itertools
import json
import math
import os
import sys

import numpy as np


def digest(arr: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(arr).tobytes()).hexdigest()


def main(ref: str) -> None:
    sys.dont_write_bytecode = True
    for sub in ("", "python", "contrib", "contrib/kittens/test", "contrib/kittens/test/bench", "contrib/kittens/test/bench/tools"):
        sys.path.insert(0, os.path.join(ref, sub))
    from kittens.gemm_config import GemmMappingSpec, GemmSpec, LoadType, OperandPath, WeakScaledMappedGemmInstance
    import kittens_helpers as kh
    import bench_harness as bh

    out: dict = {"source": "iree-org/aster pure-Python layer", "numpy": np.__version__}

    # 1. labels + derived quantities + resource estimates
    cases = []
    grids = [
        dict(M=4096, N=4096, K=4096, wg=[32, 16, 1], waves=[1, 4, 1], tpw=[8, 4, 1]),
        dict(M=2432, N=4096, K=4096, wg=[19, 16, 1], waves=[1, 4, 1], tpw=[8, 4, 1]),
        dict(M=2048, N=4096, K=4096, wg=[16, 32, 1], waves=[1, 4, 1], tpw=[8, 2, 2]),
        dict(M=2432, N=2048, K=8192, wg=[19, 16, 1], waves=[2, 2, 1], tpw=[4, 4, 2]),
        dict(M=48, N=32, K=128, wg=[1, 1, 1], waves=[1, 1, 1], tpw=[3, 2, 1]),
        dict(M=192, N=96, K=256, wg=[1, 1, 1], waves=[4, 2, 1], tpw=[3, 3, 1]),
        dict(M=512, N=512, K=512, wg=[4, 2, 1], waves=[1, 4, 1], tpw=[8, 4, 1]),
    ]
    variants = [
        dict(),
        dict(load_type=LoadType.BUFFER),
        dict(operand_path=OperandPath.DIRECT_B),
        dict(num_wg_per_cu=2, lcm_unroll=False, unroll_factor_multiplier=3, epilogue_peeling=False, ll_sched=2,
             hoist_wait=True, rotate_compute_stage=True, use_conservative_barriers=True),
    ]
    for g, ps, var in itertools.product(grids, [0, 1, 2, 3, 5, 6, 7, 9, 11, 13], variants):
        spec = GemmSpec.from_sizes(g["M"], g["N"], g["K"])
        mapping = GemmMappingSpec(g["wg"], g["waves"], g["tpw"], pipeline_strategy=ps, **var)
        cfg = WeakScaledMappedGemmInstance(spec, mapping)
        assert WeakScaledMappedGemmInstance.from_label(cfg.label).label == cfg.label
        cases.append({
            "M": g["M"], "N": g["N"], "K": g["K"], "wg": g["wg"], "waves": g["waves"], "tpw": g["tpw"],
            "pipeline_strategy": ps,
            "variant": {k: (v.value if hasattr(v, "value") else v) for k, v in var.items()},
            "label": cfg.label,
            "total_flops": cfg.total_flops,
            "num_threads": cfg.num_threads,
            "num_workgroups": cfg.num_workgroups,
            "num_tiles_per_workgroup": cfg.num_tiles_per_workgroup,
            "k_scaling_factor": cfg.k_scaling_factor,
            "lds_bytes": cfg.lds_bytes,
            "estimated_vgprs": cfg.estimated_vgprs,
            "estimated_agprs": cfg.estimated_agprs,
            "simd_occupancy": cfg.simd_occupancy,
            "kernel_name": cfg.kernel_name,
            "strides_a": list(spec.operand_layout(type(list(spec._operand_layouts)[0]).A).strides),
            "strides_c": list(spec.operand_layout(type(list(spec._operand_layouts)[0]).C).strides),
        })
    out["label_cases"] = cases

    # 2. weak-scale violation message
    try:
        WeakScaledMappedGemmInstance(GemmSpec.from_sizes(100, 64, 64), GemmMappingSpec([1, 1, 1], [1, 1, 1], [4, 4, 1]))
        out["weak_scale_error"] = None
    except AssertionError as e:
        out["weak_scale_error"] = str(e)

    # 3. shuffle_weight
    small = np.arange(16 * 32, dtype=np.int16).reshape(16, 32)
    big = (np.arange(64 * 128, dtype=np.int64) * 7 % 65521).astype(np.uint16).reshape(64, 128)
    out["shuffle_weight"] = {
        "small_16x32": kh.shuffle_weight(small).reshape(-1).tolist(),
        "big_64x128_sha256": digest(kh.shuffle_weight(big)),
    }

    # 4. pipeline strategies
    out["pipeline_strategies"] = {str(k): v for k, v in kh.PIPELINE_STRATEGIES.items()}
    out["pipeline_strategy_stages"] = {str(k): list(kh.pipeline_strategy_stages(k)) for k in kh.PIPELINE_STRATEGIES}

    # 5. init_array digests
    init = {}
    for mode in bh.InitMode:
        for role in ("A", "B"):
            arr = bh.init_array((24, 40), mode, role, dtype=np.float16, seed=42)
            init[f"{mode.value}/{role}"] = {"first8": arr.reshape(-1)[:8].astype(np.float64).tolist(), "sha256": digest(arr)}
    out["init_array"] = init

    # 6. _compute_stats
    times = [float(t) for t in (np.random.default_rng(7).integers(90_000, 130_000, size=80))]
    s = bh._compute_stats(times, 2 * 4096**3, 1307.0)
    out["compute_stats"] = {
        "times_ns": times,
        "total_flops": 2 * 4096**3,
        "peak": 1307.0,
        "fields": {k: getattr(s, k) for k in ("p0_ns", "p10_ns", "p25_ns", "p50_ns", "p90_ns", "mean_ns", "stddev_ns", "stddev_tf")},
        "derived": {k: getattr(s, k) for k in ("p0_tf", "p50_tf", "p90_tf", "mean_tf", "p50_pct", "p50_ms")},
    }
    out["compute_stats_none"] = bh._compute_stats([], 1, 1.0) is None and bh._compute_stats([1.0, 0.0], 1, 1.0) is None
    out["peak_table"] = dict(bh._PEAK_TFLOPS_F16_BY_MCPU)

    # 7. coop_2d_split: coop.py imports the MLIR bindings at module level, so only the pure
    # function is taken from its source.
    src = open(os.path.join(ref, "contrib/kittens/test/coop.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "coop_2d_split")
    ns: dict = {"math": math}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "coop.py", "exec"), ns)
    out["coop_2d_split"] = [
        {"args": [t, w, k], "result": list(ns["coop_2d_split"](t, w, k))}
        for t, w, k in itertools.product([1, 2, 3, 6, 8, 12, 16], [1, 2, 4, 8], [1, 2, 3])
    ]

    # 8. labels stored in the reference's registry
    labels = []
    reg = json.load(open(os.path.join(ref, "contrib/kittens/test/bench/tools/best_known.json")))

    def walk(node):
        if isinstance(node, dict):
            for k, v in node.items():
                if k == "label" and isinstance(v, str):
                    labels.append(v)
                walk(v)
        elif isinstance(node, list):
            for v in node:
                walk(v)

    walk(reg)
    out["best_known_labels"] = sorted(set(labels))

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(f"wrote {dst}: {len(cases)} label cases, {len(out['best_known_labels'])} registry labels")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the iree-org/aster checkout>")
    main(sys.argv[1])
