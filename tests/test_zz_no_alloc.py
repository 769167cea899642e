"""The allocation-free split-K entry point against the regular one.

``b200_gemm_splitk_noalloc`` keeps its fp32 partial sums in a scratch array that is part of
the library image, for hosts that cannot call cudaMalloc when they need the GEMM.  It must
produce exactly what ``b200_gemm_run`` produces with a caller workspace and the same tile and
split, on repeated calls (the scratch keeps the previous call's contents, so the second call
runs over stale partial sums).  This file sorts last so that a run stopping at the first
failure has already gone through every other test.
"""

import ctypes as C

import numpy as np
import pytest

from aster_b200 import _native as nat
from aster_b200.execution import GpuBuffer
from aster_b200.gemm import DTYPE_CODES, GemmPlan, gemm_splitk_noalloc, gemm_splitk_noalloc_status
from oracle import gemm_oracle as orc

pytestmark = pytest.mark.gpu


def _device_operands(inp, M, N, dtype_c):
    a, b = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes)
    a.copy_from_host(inp["A"])
    b.copy_from_host(inp["B"])
    c_bytes = M * N * (4 if dtype_c == "f32" else 2)
    return a, b, GpuBuffer(c_bytes), GpuBuffer(c_bytes)


@pytest.mark.parametrize("M,N,K,split_k,dtype_ab,dtype_c", [
    (16, 1024, 4096, 4, "bf16", "bf16"),
    (128, 2048, 2048, 8, "bf16", "f32"),
    (48, 200, 1000, 3, "f16", "f32"),
    (64, 512, 2048, 2, "e4m3", "bf16"),
    (100, 384, 512, 1, "bf16", "bf16"),
])
def test_matches_regular_split_k_on_two_calls_in_a_row(gpu, M, N, K, split_k, dtype_ab, dtype_c):
    inp = orc.make_inputs(M, N, K, dtype_ab, "uniform" if dtype_ab != "e4m3" else "normal", 4)
    dA, dB, dC_ref, dC_new = _device_operands(inp, M, N, dtype_c)
    storage = np.float32 if dtype_c == "f32" else np.uint16

    # Regular entry point: same tile (64 columns, one CTA) and split, caller-provided workspace.
    plan = GemmPlan(M, N, K, dtype_ab, dtype_c, tile_n=64, cta_group=1, stages=8, split_k=split_k)
    res = plan.resources()
    ws = GpuBuffer(res.workspace_bytes) if res.workspace_bytes else None
    plan.run(dA, dB, dC_ref, workspace=ws)
    plan.status()
    want = np.empty((M, N), storage)
    dC_ref.copy_to_host(want)

    before = nat.launch_count()
    for call in range(2):
        dC_new.zero()
        status = nat.lib().b200_gemm_splitk_noalloc(dA.ptr, dB.ptr, dC_new.ptr, M, N, K, DTYPE_CODES[dtype_ab],
                                                     DTYPE_CODES[dtype_c], split_k, None)
        assert status == nat.OK, nat.last_error()
        assert gemm_splitk_noalloc_status() == [0, 0, 0, 0]  # synchronises; no bounded wait gave up
        got = np.empty((M, N), storage)
        dC_new.copy_to_host(got)
        # Same kernels, same tile order, same summation order: the outputs are identical, which
        # is tighter than the GEMM tolerances used elsewhere (checked against the oracle below).
        assert np.array_equal(got, want), f"call {call}: differs from b200_gemm_run"
    assert nat.launch_count() - before == 2 * (2 if res.split_k > 1 else 1)

    # And both agree with the CPU oracle within the usual tolerance.
    ref = orc.gemm_f32(inp["A"], inp["B"], dtype_ab)
    if dtype_ab == "e4m3":
        alpha = 1.0  # no scales on this entry point: compare raw quantised products
        assert orc.rel_frobenius(orc.decode(got, dtype_c), orc.decode(orc.encode(ref * alpha, dtype_c), dtype_c)) <= 0.02
    elif dtype_c == "f32":
        assert float(np.max(np.abs(got - ref))) <= orc.abs_bound(inp["A"], inp["B"], dtype_ab)
    else:
        assert orc.bf16_output_error(got, ref, orc.accumulation_slack(inp["A"], inp["B"], dtype_ab)) <= 0.0
    for buf in (dA, dB, dC_ref, dC_new, ws):
        if buf is not None:
            buf.free()


def test_python_wrapper_and_limits(gpu):
    M, N, K = 16, 512, 1024
    inp = orc.make_inputs(M, N, K, "bf16", "uniform", 4)
    dA, dB, dC, _ = _device_operands(inp, M, N, "bf16")
    gemm_splitk_noalloc(dA, dB, dC, M, N, K, "bf16", "bf16", split_k=4)
    assert gemm_splitk_noalloc_status() == [0, 0, 0, 0]
    got = np.empty((M, N), np.uint16)
    dC.copy_to_host(got)
    ref = orc.gemm_f32(inp["A"], inp["B"], "bf16")
    assert orc.bf16_output_error(got, ref, orc.accumulation_slack(inp["A"], inp["B"], "bf16")) <= 0.0

    lib = nat.lib()
    # 8 * 1024 * 1024 * 4 bytes = 32 MiB of partial sums: beyond the built-in 16 MiB.
    assert lib.b200_gemm_splitk_noalloc(dA.ptr, dB.ptr, dC.ptr, 1024, 1024, 8192, nat.BF16, nat.BF16, 8, None) == nat.ERR_WORKSPACE
    assert "16777216-byte scratch" in nat.last_error()
    assert lib.b200_gemm_splitk_noalloc(None, dB.ptr, dC.ptr, M, N, K, nat.BF16, nat.BF16, 4, None) == nat.ERR_INVALID
    assert lib.b200_gemm_splitk_noalloc(dA.ptr, dB.ptr, dC.ptr, M, N, 7, nat.BF16, nat.BF16, 4, None) == nat.ERR_INVALID
    assert lib.b200_gemm_splitk_noalloc(dA.ptr, dB.ptr, dC.ptr, M, N, K, nat.BF16, nat.BF16, 65, None) == nat.ERR_INVALID
    assert lib.b200_gemm_splitk_noalloc(dA.ptr, dB.ptr, dC.ptr, M, N, K, 9, nat.BF16, 4, None) == nat.ERR_INVALID
    for buf in (dA, dB, dC):
        buf.free()
