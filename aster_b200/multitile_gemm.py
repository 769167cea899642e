"""The GEMM "generator" interface of the reference, served by the B200 plan.

``compile_multitile_gemm(cfg, output_path, **kw) -> (path, text)`` and
``execute_multitile_hsaco(cfg, path, num_iterations, A, B, skip_gpu_check=False) -> (C, times_ns)``
keep the signatures of contrib/kittens/test/test_102_gemm_python_multitile_lds_cdna3.py:391-436
(and of the direct-B twin, test_102_..._directb_cdna3.py:380-428).  Where the reference
compiles MLIR to an HSACO file, "compiling" here validates the config against the native
library, selects the kernel instance and writes a small JSON artifact describing it; executing
loads that artifact, uploads A and B, runs the timed launch loop and returns the flattened C.
"""

from __future__ import annotations

import json
import math
from typing import Optional

import numpy as np

from . import _native as nat
from .dtypes import STORAGE
from .execution import GpuBuffer, InputArray, OutputArray, execute_launch, system_has_gpu
from .gemm import GemmPlan
from .gemm_config import B200GemmInstance, GemmMappingSpec, Operand, OperandPath, WeakScaledMappedGemmInstance
from .kittens_helpers import shuffle_weight

KERNEL_NAME = "gemm_multitile"
MCPU = "sm_100a"
ARTIFACT_SUFFIX = ".b200plan.json"


class MultitileGemmInstance(B200GemmInstance):
    """Name used by the reference's tests and bench drivers for the executable config."""


def _resources_dict(plan: GemmPlan) -> dict:
    r = plan.resources()
    return {name: getattr(r, name) for name, _ in r._fields_}


def compile_multitile_gemm(cfg: B200GemmInstance, output_path: str, **kw):
    """Validate ``cfg``, select its kernel and write the plan artifact.

    Returns ``(path, text)`` like the reference returns ``(hsaco_path, asm)``; ``text`` is the
    artifact's JSON, whose ``resources`` block is what a post-compile filter inspects.
    The register-budget / print keywords of the reference are accepted and ignored.
    """
    plan = GemmPlan(**cfg.plan_kwargs())
    try:
        artifact = {
            "kernel_name": KERNEL_NAME,
            "mcpu": MCPU,
            "label": cfg.label,
            "operand_path": cfg.mapping.operand_path.value,
            "plan": {k: v for k, v in cfg.plan_kwargs().items()},
            "resources": _resources_dict(plan),
        }
    finally:
        plan.destroy()
    text = json.dumps(artifact, indent=1, sort_keys=True)
    with open(output_path, "w") as f:
        f.write(text)
    return output_path, text


def load_artifact(path: str) -> dict:
    with open(path) as f:
        art = json.load(f)
    if art.get("kernel_name") != KERNEL_NAME or "plan" not in art:
        raise RuntimeError(f"{path} is not a {KERNEL_NAME} plan artifact")
    return art


def fits_on_sm_post_compile(cfg, resources: Optional[dict]) -> Optional[str]:
    """Post-compile filter: ``None`` if the instance fits one SM, else the reason
    (role of ``fits_on_cu_post_compile``, contrib/kittens/test/bench/bench_search.py:454-476)."""
    if not resources:
        return "no resources reported"
    if resources["smem_bytes"] > 232448:
        return f"shared memory {resources['smem_bytes']} > 232448"
    if resources["tmem_columns"] > 512:
        return f"tensor memory columns {resources['tmem_columns']} > 512"
    if 0 < resources.get("regs_per_thread", 0) * resources["block_threads"] > 65536:
        return "register file exceeded"
    return None


def execute_multitile_hsaco(cfg: B200GemmInstance, hsaco_path: str, num_iterations: int, A: np.ndarray, B: np.ndarray,
                            skip_gpu_check: bool = False, *, bias: Optional[np.ndarray] = None,
                            scale_a: Optional[float] = None, scale_b: Optional[float] = None, flush_llc=None):
    """Run a compiled config ``num_iterations`` times; returns ``(C_flat, times_ns)``.

    A is ``[M,K]`` and B ``[N,K]`` in the storage type of ``cfg.dtype_ab`` (float16, uint16 /
    uint8 bit patterns, or int8).  For a direct-B config B is preshuffled on the host exactly as the
    reference does before upload (test_102_..._directb_cdna3.py:418) and packed on the device
    before the timed loop.  C is float32, bf16 bit patterns when ``cfg.dtype_c == "bf16"``, or
    int32 when ``cfg.dtype_c == "i32"``.
    """
    if not skip_gpu_check and not system_has_gpu(MCPU):
        import pytest

        pytest.skip(f"GPU {MCPU} not available, skip execution")
    art = load_artifact(hsaco_path)
    if art["label"] != cfg.label:
        raise RuntimeError(f"artifact {hsaco_path} was compiled for {art['label']}, not {cfg.label}")
    plan = GemmPlan(**art["plan"])
    res = plan.resources()
    m, n, k = cfg.gemm_size
    want = STORAGE[cfg.dtype_ab]
    A = np.ascontiguousarray(A).reshape(m, k)
    B = np.ascontiguousarray(B).reshape(n, k)
    if A.dtype != want or B.dtype != want:
        raise TypeError(f"A/B must be stored as {np.dtype(want)} for {cfg.dtype_ab}, got {A.dtype}/{B.dtype}")
    C_output = np.zeros(math.prod(cfg.spec.operand_shape(Operand.C)), dtype=STORAGE[cfg.dtype_c])
    nat.init_current()
    extra = []
    try:
        if cfg.mapping.direct_b:
            b_host = shuffle_weight(B)
            staging = GpuBuffer(b_host.nbytes)
            extra.append(staging)
            staging.copy_from_host(b_host)
            b_dev = GpuBuffer(res.packed_b_bytes)
            extra.append(b_dev)
            plan.pack_b(staging, b_dev)
            b_arg = b_dev
        else:
            b_arg = InputArray(B.reshape(-1))
        scalars = {}
        for name, val in (("scale_a", scale_a), ("scale_b", scale_b)):
            if val is not None:
                buf = GpuBuffer(4)
                buf.copy_from_host(np.array([val], dtype=np.float32))
                extra.append(buf)
                scalars[name] = buf
        bias_dev = None
        if bias is not None:
            bias_dev = GpuBuffer(4 * bias.size)
            bias_dev.copy_from_host(np.ascontiguousarray(bias, dtype=np.float32))
            extra.append(bias_dev)
        ws = None
        ws_bytes = res.workspace_bytes or res.optional_workspace_bytes
        if ws_bytes:
            ws = GpuBuffer(ws_bytes)
            extra.append(ws)

        def launch(a_buf, b_buf, c_buf):
            plan.run(a_buf, b_buf, c_buf, bias_dev, scalars.get("scale_a"), scalars.get("scale_b"), ws)

        times_ns = execute_launch(
            launch, [InputArray(A.reshape(-1)), b_arg, OutputArray(C_output)], num_iterations=num_iterations, flush_llc=flush_llc
        )
        plan.status()
    finally:
        for buf in extra:
            buf.free()
        plan.destroy()
    return C_output, times_ns


def _as_b200_instance(cfg) -> B200GemmInstance:
    """A plain ``WeakScaledMappedGemmInstance`` (the older template family's config type) as the
    executable instance of the same label and operand path."""
    if isinstance(cfg, B200GemmInstance):
        return cfg
    return MultitileGemmInstance.from_label(cfg.label, operand_path=cfg.mapping.operand_path)


def compile_gemm(cfg, output_hsaco_path: str, **kw):
    """``compile_gemm`` of the weak-scaled template family
    (contrib/kittens/test/test_perf_001_gemm_fp16_weak_scaled.py:181-231): same call, same
    ``(path, text)`` return; the config may be a plain ``WeakScaledMappedGemmInstance``."""
    return compile_multitile_gemm(_as_b200_instance(cfg), output_hsaco_path, **kw)


def execute_gemm_hsaco(cfg, hsaco_path: str, num_iterations: int, A: np.ndarray, B: np.ndarray, skip_gpu_check: bool = False):
    """``execute_gemm_hsaco`` of the same family (test_perf_001_...:234-272): row-major A and B in,
    ``(C_output, times_ns)`` out; a direct-B config has its B preshuffled here."""
    return execute_multitile_hsaco(_as_b200_instance(cfg), hsaco_path, num_iterations, A, B, skip_gpu_check)


def _repro_cmd(cfg) -> str:
    return f"python -m aster_b200.bench_gemm {cfg.label}"


def _from_label(label: str, mcpu: str = MCPU, operand_path: OperandPath = OperandPath.LDS) -> MultitileGemmInstance:
    cfg = MultitileGemmInstance.from_label(label, operand_path=operand_path)
    cfg.mapping.mcpu = mcpu
    return cfg


def _from_label_direct_b(label: str, mcpu: str = MCPU) -> MultitileGemmInstance:
    return _from_label(label, mcpu, OperandPath.DIRECT_B)


def _post_compile_filter(cfg, resources):
    return fits_on_sm_post_compile(cfg, resources)


# Hooks a sweep / regression driver consumes, same keys as the reference's
# (bench_perf_102_gemm_python_multitile_lds_cdna3.py:303-309).
BENCH_HOOKS = {
    "bench_label": "bench_perf_102_gemm_multitile_lds_sm100",
    "from_label": _from_label,
    "compile_fn": compile_multitile_gemm,
    "repro_cmd_fn": _repro_cmd,
    "post_compile_filter": _post_compile_filter,
}
BENCH_HOOKS_DIRECT_B = dict(BENCH_HOOKS, bench_label="bench_perf_102_gemm_multitile_directb_sm100", from_label=_from_label_direct_b)


def hooks_for_bench(bench: str):
    """The hooks dict behind a registry's bench name, or ``None``.  Benches of other element
    types share the hooks of their family under a suffixed name (``..._fp8``, ``..._bf8``,
    ``..._i8``): a label carries its own element types."""
    for hooks in (BENCH_HOOKS, BENCH_HOOKS_DIRECT_B):
        base = hooks["bench_label"]
        if bench == base or (bench.startswith(base + "_") and bench[len(base) + 1:] in ("fp8", "bf8", "i8")):
            return dict(hooks, bench_label=bench)
    return None
