"""Single-config GEMM bench, the B200 twin of running one label through the reference's
``bench_perf_102_gemm_python_multitile_*`` scripts (``run_single``, bench_harness.py:1738-1850).

    python -m aster_b200.bench_gemm <label> [--iterations N] [--results-file F] [--direct-b]
    python -m aster_b200.bench_gemm --size MxNxK [--dtype bf16] [--out-dtype bf16] [--epilogue bias_relu]

Prints the tile the plan selected, the timing table (p0/p10/p25/p50/p90/mean, TFLOP/s, % of the
dense tensor peak) over ``iterations`` launches with the first 20 dropped, and PASS/FAIL of the
numpy check.
"""

from __future__ import annotations

import argparse
import sys

from .bench_harness import INIT_DEFAULT, NUM_ITERATIONS, InitMode, run_single
from .gemm_config import OperandPath, make_b200_instance
from .multitile_gemm import BENCH_HOOKS, BENCH_HOOKS_DIRECT_B, compile_multitile_gemm, execute_multitile_hsaco


def parse_mnk(text: str) -> tuple[int, int, int]:
    parts = text.lower().split("x")
    if len(parts) != 3:
        raise argparse.ArgumentTypeError(f"expected MxNxK, got {text!r}")
    return tuple(int(p) for p in parts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("label", nargs="?", help="config label (reference grammar, optional _b200_ suffix)")
    ap.add_argument("--size", type=parse_mnk, help="MxNxK when no label is given")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16", "e4m3", "e5m2", "i8"])
    ap.add_argument("--out-dtype", default="f32", choices=["f32", "bf16", "i32"])
    ap.add_argument("--epilogue", default="none", choices=["none", "bias_relu", "bias", "relu"])
    ap.add_argument("--direct-b", action="store_true", help="B preshuffled as in the reference's direct-B path")
    ap.add_argument("--iterations", type=int, default=NUM_ITERATIONS)
    ap.add_argument("--init", default=INIT_DEFAULT.value, choices=[m.value for m in InitMode])
    ap.add_argument("--results-file")
    ap.add_argument("--hsaco", help="where to keep the plan artifact")
    args = ap.parse_args(argv)

    hooks = BENCH_HOOKS_DIRECT_B if args.direct_b else BENCH_HOOKS
    if args.label:
        cfg = hooks["from_label"](args.label, "sm_100a")
    elif args.size:
        m, n, k = args.size
        cfg = make_b200_instance(m, n, k, dtype_ab=args.dtype, dtype_c=args.out_dtype, epilogue=args.epilogue,
                                 operand_path=OperandPath.DIRECT_B if args.direct_b else OperandPath.LDS)
    else:
        ap.error("give a label or --size")
    if cfg.epilogue in ("bias_relu", "bias"):
        print("note: epilogue configs are timed without the numpy check (run the tests for parity)", file=sys.stderr)

        def execute(cfg_, path, iters, A, B, skip_gpu_check=False, **kw):
            import numpy as np

            bias = (np.random.default_rng(44).standard_normal(cfg_.gemm_size[1]) * 0.1).astype(np.float32)
            return execute_multitile_hsaco(cfg_, path, iters, A, B, skip_gpu_check, bias=bias, **kw)
    else:
        execute = execute_multitile_hsaco
    stats = run_single(cfg, compile_multitile_gemm, execute, iterations=args.iterations, init_mode=InitMode(args.init),
                       bench=hooks["bench_label"], results_file=args.results_file, hsaco=args.hsaco)
    return 0 if stats is not None else 1


if __name__ == "__main__":
    sys.exit(main())
