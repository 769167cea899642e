"""GEMM parity on a B200: the CUDA path (through the C ABI) against the CPU oracle on the same
seeded inputs.  The matrix follows the reference's own test classes
(contrib/kittens/test/test_102_gemm_python_multitile_lds_cdna3.py:515-702 and the direct-B
twin): geometry, pipeline depth x K length, multi-workgroup, plus the element types, the
fused epilogue, the scaled fp8 path, split-K and the configured full-size problems.

Tolerances (stated once here, used below):
* f16 / bf16 inputs, f32 output: max |err| <= 2e-3 * sqrt(K) * max|a| * max|b|, and the
  reference's own gate rtol = atol = 1e-2 where the reference uses it.
* bf16 output: |out - oracle f32| <= one bf16 spacing at the oracle's magnitude, plus
  1e-6 * K * max|a| * max|b| for the different fp32 summation orders of GPU and BLAS.
* e4m3: relative Frobenius error <= 2 % against the oracle built from the same quantised inputs.
"""

import math
import tempfile

import numpy as np
import pytest

from aster_b200.gemm import GemmPlan, gemm
from aster_b200.gemm_config import B200GemmInstance, GemmMappingSpec, GemmSpec, OperandPath, make_b200_instance
from aster_b200.kittens_helpers import PIPELINE_STRATEGIES
from aster_b200.multitile_gemm import compile_multitile_gemm, execute_multitile_hsaco
from oracle import gemm_oracle as orc

pytestmark = pytest.mark.gpu


def check(got, inp, dtype_ab, dtype_c, *, bias=None, relu=False, bias_axis="n"):
    alpha = 1.0
    if inp["scale_a"] is not None:
        alpha = float(np.float32(inp["scale_a"]) * np.float32(inp["scale_b"]))
    want = orc.gemm_epilogue(orc.gemm_f32(inp["A"], inp["B"], dtype_ab), bias, relu, bias_axis, alpha)
    got_f32 = orc.decode(got, dtype_c).reshape(want.shape)
    if dtype_ab == "e4m3":
        want_c = orc.decode(orc.encode(want, dtype_c), dtype_c)
        rel = orc.rel_frobenius(got_f32, want_c)
        assert rel <= 0.02, f"relative Frobenius error {rel}"
        # accumulation is exact enough that the error is far below the budget
        assert rel <= 1e-3
    elif dtype_c == "f32":
        bound = orc.abs_bound(inp["A"], inp["B"], dtype_ab) * (abs(alpha) if alpha != 1.0 else 1.0)
        err = float(np.max(np.abs(got_f32 - want)))
        assert err <= bound, f"max |err| {err} > {bound}"
    else:
        excess = orc.bf16_output_error(got, want, orc.accumulation_slack(inp["A"], inp["B"], dtype_ab, alpha))
        assert excess <= 0.0, f"bf16 output exceeds one bf16 spacing + accumulation slack by {excess}"


def run(M, N, K, dtype_ab="f16", dtype_c="f32", dist="normal", seed=0, bias=False, relu=False, bias_axis="n", **kw):
    inp = orc.make_inputs(M, N, K, dtype_ab, dist, seed, with_bias=False)
    b = None
    if bias:
        b = (np.random.default_rng(seed + 2).standard_normal(N if bias_axis == "n" else M) * 0.1).astype(np.float32)
    got = gemm(inp["A"], inp["B"], dtype_ab=dtype_ab, dtype_c=dtype_c, bias=b, relu=relu, bias_axis=bias_axis,
               scale_a=inp["scale_a"], scale_b=inp["scale_b"], **kw)
    check(got, inp, dtype_ab, dtype_c, bias=b, relu=relu, bias_axis=bias_axis)
    return got


class TestKnownAnswers:
    """The reference's single-instruction known answers, through the full kernel."""

    def test_f16_ones_times_twos(self, gpu):
        a = np.ones((16, 16), np.float16)
        b = np.full((16, 16), 2.0, np.float16)
        assert np.all(gemm(a, b) == 32.0)

    @pytest.mark.parametrize("dtype", ["f16", "bf16"])
    def test_ones_k32(self, gpu, dtype):
        ones = orc.encode(np.ones((16, 32), np.float32), dtype)
        assert np.all(gemm(ones, ones, dtype_ab=dtype) == 32.0)

    def test_fp8_ones_and_initial_accumulator(self, gpu):
        ones = orc.encode(np.ones((16, 32), np.float32), "e4m3")
        assert np.all(gemm(ones, ones, dtype_ab="e4m3") == 32.0)
        a = orc.encode(np.full((16, 32), 1.5, np.float32), "e4m3")
        b = orc.encode(np.full((16, 32), 2.0, np.float32), "e4m3")
        assert np.all(gemm(a, b, dtype_ab="e4m3", bias=np.full(16, 10.0, np.float32)) == 106.0)

    def test_scaled_fp8(self, gpu):
        a = orc.encode(np.full((16, 128), 1.75, np.float32), "e4m3")
        b = orc.encode(np.full((16, 128), 1.25, np.float32), "e4m3")
        assert np.all(gemm(a, b, dtype_ab="e4m3", scale_a=4.0, scale_b=2.0) == 2240.0)

    def test_bf16_tile_64(self, gpu):
        a = orc.encode(np.ones((16, 32), np.float32), "bf16")
        b = orc.encode(np.full((16, 32), 2.0, np.float32), "bf16")
        assert np.all(gemm(a, b, dtype_ab="bf16") == 64.0)


def reference_style_instance(num_workgroups, num_waves_per_wg, num_tiles_per_wg, k_mult, pipeline_strategy=1,
                             operand_path=OperandPath.LDS, **mapping_kw):
    """``_make_instance`` of the reference tests: sizes follow from the mapping."""
    tiles_per_wave = [t // w for t, w in zip(num_tiles_per_wg, num_waves_per_wg)]
    M = num_workgroups[0] * num_tiles_per_wg[0] * 16
    N = num_workgroups[1] * num_tiles_per_wg[1] * 16
    K = k_mult * num_tiles_per_wg[2] * 32
    mapping = GemmMappingSpec(num_workgroups, num_waves_per_wg, tiles_per_wave, pipeline_strategy=pipeline_strategy,
                              operand_path=operand_path, **mapping_kw)
    return B200GemmInstance(GemmSpec.from_sizes(M, N, K), mapping)


def run_reference_style(cfg):
    """``_run_multitile`` of the reference tests: seed 42+M+N+K, randn * 0.1 in f16, compile to
    a temporary artifact, execute once, numpy oracle with rtol = atol = 1e-2."""
    M, N, K = cfg.gemm_size
    np.random.seed(42 + M + N + K)
    A = (np.random.randn(M, K) * 0.1).astype(np.float16)
    B = (np.random.randn(N, K) * 0.1).astype(np.float16)
    with tempfile.NamedTemporaryFile(suffix=".b200plan.json") as tmp:
        compile_multitile_gemm(cfg, tmp.name)
        C, times = execute_multitile_hsaco(cfg, tmp.name, 1, A, B)
    assert len(times) == 1 and times[0] > 0
    orc.assert_reference_close(C, orc.gemm_f32(A, B).reshape(-1))


GEOMETRIES = [
    ([1, 1, 1], [3, 2, 1]), ([1, 1, 1], [2, 2, 3]), ([2, 1, 1], [6, 2, 1]), ([2, 2, 1], [8, 4, 1]),
    ([2, 2, 1], [6, 4, 1]), ([2, 2, 1], [6, 6, 1]), ([4, 1, 1], [8, 7, 1]), ([4, 1, 1], [12, 5, 1]),
    ([1, 4, 1], [10, 8, 1]), ([4, 2, 1], [12, 6, 1]), ([2, 4, 1], [8, 8, 1]), ([2, 4, 1], [12, 8, 1]),
]


class TestGeometry:
    """Wave-geometry sweep of the reference (test_102_..._lds_cdna3.py:515-562)."""

    @pytest.mark.parametrize("waves,tiles", GEOMETRIES)
    def test_correctness(self, gpu, waves, tiles):
        run_reference_style(reference_style_instance([1, 1, 1], waves, tiles, k_mult=4, pipeline_strategy=3))


class TestPipeline:
    """Pipeline strategy x K length (test_102_..._lds_cdna3.py:565-595): the strategy's depth is
    the shared-memory ring depth here, so short K against deep rings is the interesting corner."""

    @pytest.mark.parametrize("waves,tiles", [([2, 2, 1], [6, 4, 1]), ([4, 2, 1], [12, 6, 1])])
    @pytest.mark.parametrize("k_mult", [2, 4, 8])
    @pytest.mark.parametrize("pipeline_strategy", [1, 2, 3, 4, 5, 6, 9])
    def test_correctness(self, gpu, waves, tiles, k_mult, pipeline_strategy):
        if k_mult < max(PIPELINE_STRATEGIES[pipeline_strategy].values()) + 1:
            pytest.skip("fewer K iterations than pipeline stages (the reference skips these too)")
        run_reference_style(reference_style_instance([1, 1, 1], waves, tiles, k_mult, pipeline_strategy))


class TestMultiWG:
    @pytest.mark.parametrize("wg", [[2, 2, 1], [3, 1, 1], [1, 5, 1], [4, 3, 1], [19, 2, 1]])
    def test_correctness(self, gpu, wg):
        run_reference_style(reference_style_instance(wg, [2, 2, 1], [8, 8, 1], k_mult=8, pipeline_strategy=3))

    def test_label_knobs_do_not_change_results(self, gpu):
        run_reference_style(reference_style_instance([2, 2, 1], [2, 2, 1], [8, 8, 1], 8, 5, ll_sched=1, hoist_wait=True,
                                                     rotate_compute_stage=True, use_conservative_barriers=True))


class TestDirectB:
    """B handed over in the reference's preshuffled order (test_102_..._directb_cdna3.py)."""

    @pytest.mark.parametrize("wg,waves,tiles,k_mult", [
        ([1, 1, 1], [1, 1, 1], [3, 2, 1], 4), ([1, 1, 1], [2, 2, 1], [8, 4, 1], 4),
        ([2, 3, 1], [1, 4, 1], [8, 16, 1], 8), ([2, 2, 1], [2, 2, 1], [6, 6, 2], 4),
    ])
    def test_correctness(self, gpu, wg, waves, tiles, k_mult):
        run_reference_style(reference_style_instance(wg, waves, tiles, k_mult, 3, operand_path=OperandPath.DIRECT_B))

    def test_packed_row_major_input(self, gpu):
        run(384, 640, 512, b_layout="packed")
        run(200, 136, 264, b_layout="packed", tile_n=64)

    def test_direct_b_equals_staged_b_bitwise(self, gpu):
        inp = orc.make_inputs(256, 512, 1024, "bf16", "uniform", 9)
        staged = gemm(inp["A"], inp["B"], dtype_ab="bf16", tile_n=128)
        direct = gemm(inp["A"], inp["B"], dtype_ab="bf16", tile_n=128, b_layout="packed")
        assert np.array_equal(staged, direct)


class TestShapesAndTypes:
    @pytest.mark.parametrize("tile_n", [32, 64, 128, 256])
    def test_tile_widths(self, gpu, tile_n):
        run(256, 512, 384, tile_n=tile_n)

    @pytest.mark.parametrize("shape", [(1, 8, 8), (16, 16, 16), (48, 32, 128), (130, 70, 72), (127, 255, 1000),
                                       (129, 257, 1032), (300, 36, 200), (5, 1000, 64)])
    @pytest.mark.parametrize("dtype_c", ["f32", "bf16"])
    def test_ragged(self, gpu, shape, dtype_c):
        run(*shape, "bf16", dtype_c, "uniform", seed=sum(shape))

    @pytest.mark.parametrize("stages", [1, 2, 3, 5, 8])
    def test_ring_depths(self, gpu, stages):
        run(256, 256, 2048, "bf16", "f32", "uniform", 1, tile_n=64, stages=stages)

    @pytest.mark.parametrize("max_ctas", [1, 7, 148])
    def test_persistent_grid_sizes(self, gpu, max_ctas):
        run(1024, 1536, 256, "bf16", "bf16", "uniform", 1, max_ctas=max_ctas, tile_n=128)

    @pytest.mark.parametrize("raster_group", [1, 3, 8, 64])
    def test_rasterisation(self, gpu, raster_group):
        run(1280, 1024, 128, "f16", "f32", raster_group=raster_group, tile_n=128)

    def test_empty_k_tail_and_zero_inputs(self, gpu):
        a = np.zeros((128, 64), np.float16)
        assert not gemm(a, a).any()


class TestCtaPair:
    """One CTA per tile (cta_group 1) against a CTA pair per 256-row tile (cta_group 2)."""

    @pytest.mark.parametrize("cta_group", [1, 2])
    @pytest.mark.parametrize("tile_n", [64, 128, 256])
    @pytest.mark.parametrize("shape", [(256, 256, 256), (640, 768, 320), (300, 200, 264), (1024, 512, 2048)])
    def test_tile_shapes(self, gpu, cta_group, tile_n, shape):
        run(*shape, "bf16", "f32", "uniform", 1, cta_group=cta_group, tile_n=tile_n)

    @pytest.mark.parametrize("dtype_ab,dtype_c", [("f16", "f32"), ("bf16", "bf16"), ("e4m3", "bf16")])
    def test_pair_equals_single_bitwise(self, gpu, dtype_ab, dtype_c):
        inp = orc.make_inputs(768, 512, 1024, dtype_ab, "normal", 5)
        kw = dict(dtype_ab=dtype_ab, dtype_c=dtype_c, scale_a=inp["scale_a"], scale_b=inp["scale_b"], tile_n=128)
        assert np.array_equal(gemm(inp["A"], inp["B"], cta_group=1, **kw), gemm(inp["A"], inp["B"], cta_group=2, **kw))

    @pytest.mark.parametrize("stages", [1, 2, 4, 7])
    def test_pair_ring_depths(self, gpu, stages):
        run(512, 512, 2048, "bf16", "f32", "uniform", 1, cta_group=2, tile_n=256, stages=stages)

    @pytest.mark.parametrize("max_ctas", [2, 6, 148])
    def test_pair_persistent_grid(self, gpu, max_ctas):
        run(2048, 1024, 256, "bf16", "bf16", "uniform", 1, cta_group=2, tile_n=128, max_ctas=max_ctas)

    def test_pair_epilogue_and_split_k(self, gpu):
        run(512, 1024, 256, "bf16", "bf16", "normal", 2, bias=True, relu=True, cta_group=2)
        run(512, 1024, 256, "bf16", "bf16", "normal", 2, bias=True, relu=True, bias_axis="m", cta_group=2)
        run(256, 1024, 4096, "bf16", "bf16", "uniform", 4, split_k=4, tile_n=64, cta_group=2)

    def test_odd_row_count_in_pair(self, gpu):
        # 129..255 rows: the second CTA of the pair owns a partly or wholly empty half.
        for m in (129, 200, 255, 257, 385):
            run(m, 192, 128, "bf16", "bf16", "uniform", m, cta_group=2, tile_n=64)


class TestTailSplit:
    """The last, partly filled round of tiles cut along K when the caller lends the workspace."""

    @pytest.mark.parametrize("shape,kw", [
        ((4096, 4096, 2048), {}),                                   # 256 tiles on 74 pairs: 34 tail tiles x 2 parts
        ((1024, 1024, 4096), dict(tile_n=256)),                     # 16 tiles, all tail: 4 parts
        ((512, 512, 2048), {}),                                     # 8 small tiles x 2 parts
        ((1280, 512, 4096), dict(tile_n=128, max_ctas=16)),         # 20 tiles on 8 pairs: 4 tail tiles x 2 parts
        ((640, 512, 4096), dict(cta_group=1, tile_n=128, max_ctas=16)),  # single CTAs: 20 tiles on 16 CTAs -> 4 tail x 4 parts
        ((300, 200, 2056), dict(tile_n=64)),                        # ragged edges in the exchanged tiles
    ])
    @pytest.mark.parametrize("dtype_c", ["f32", "bf16"])
    def test_against_oracle(self, gpu, shape, kw, dtype_c):
        M, N, K = shape
        plan = GemmPlan(M, N, K, "bf16", dtype_c, **kw)
        assert plan.resources().tail_parts >= 2, "case does not exercise the tail split"
        run(M, N, K, "bf16", dtype_c, "uniform", 1, tail_split=True, **kw)

    def test_epilogue_and_fp8(self, gpu):
        run(1024, 1024, 2048, "bf16", "bf16", "normal", 2, bias=True, relu=True, tail_split=True, tile_n=256)
        run(1024, 1024, 4096, "e4m3", "bf16", "normal", 3, tail_split=True, tile_n=256)

    def test_two_plans_take_turns_with_one_workspace(self, gpu):
        """Launch epochs are unique across plans: a flag left by one plan is never taken for the
        other plan's (both plans below are at the same launch count when they meet)."""
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        shapes = [(1024, 1024, 4096), (1024, 1024, 2048)]
        plans, inputs, bufs, outs = [], [], [], []
        for M, N, K in shapes:
            inp = orc.make_inputs(M, N, K, "bf16", "uniform", K)
            plan = GemmPlan(M, N, K, "bf16", "f32", tile_n=256)
            assert plan.resources().tail_parts >= 2
            dA, dB, dC = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes), GpuBuffer(M * N * 4)
            dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
            plans.append(plan), inputs.append(inp), bufs.append((dA, dB, dC))
        ws = GpuBuffer(max(p.resources().optional_workspace_bytes for p in plans))
        for rnd in range(3):
            for plan, (dA, dB, dC) in zip(plans, bufs):
                plan.run(dA, dB, dC, workspace=ws)  # back to back, same stream, same workspace
        nat.call("b200_device_synchronize")
        for plan, inp, (dA, dB, dC), (M, N, K) in zip(plans, inputs, bufs, shapes):
            plan.status()
            out = np.empty((M, N), np.float32)
            dC.copy_to_host(out)
            check(out, inp, "bf16", "f32")

    def test_short_k_is_not_split(self, gpu):
        # the exchange costs more than a few K blocks save: such plans keep whole tiles
        assert GemmPlan(512, 512, 512, "bf16", "bf16").resources().tail_parts == 0
        assert GemmPlan(512, 512, 2048, "bf16", "bf16").resources().tail_parts == 2

    def test_repeated_launches_reuse_the_workspace(self, gpu):
        from aster_b200.execution import GpuBuffer

        M = N = 1024
        K = 2048
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 7)
        plan = GemmPlan(M, N, K, "bf16", "f32", tile_n=256)
        res = plan.resources()
        dA, dB, dC = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes), GpuBuffer(M * N * 4)
        dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
        ws = GpuBuffer(res.optional_workspace_bytes)
        outs = []
        for _ in range(4):
            dC.zero()
            plan.run(dA, dB, dC, workspace=ws)
            plan.status()
            out = np.empty((M, N), np.float32)
            dC.copy_to_host(out)
            outs.append(out)
        assert all(np.array_equal(outs[0], o) for o in outs[1:])  # fixed summation order
        assert float(np.max(np.abs(outs[0] - orc.gemm_f32(inp["A"], inp["B"], "bf16")))) <= orc.abs_bound(inp["A"], inp["B"], "bf16")
        # without the workspace the same plan computes whole tiles
        plan.run(dA, dB, dC)
        plan.status()
        whole = np.empty((M, N), np.float32)
        dC.copy_to_host(whole)
        assert np.allclose(whole, outs[0], rtol=1e-5, atol=1e-3)
        for b in (dA, dB, dC, ws):
            b.free()


class TestEpilogue:
    @pytest.mark.parametrize("dtype_c", ["f32", "bf16"])
    @pytest.mark.parametrize("bias,relu", [(True, True), (True, False), (False, True)])
    def test_bias_relu(self, gpu, dtype_c, bias, relu):
        run(384, 512, 256, "bf16", dtype_c, "normal", 2, bias=bias, relu=relu)

    def test_bias_per_row(self, gpu):
        run(384, 512, 256, "bf16", "bf16", "normal", 2, bias=True, relu=True, bias_axis="m")

    def test_relu_actually_clamps(self, gpu):
        got = run(256, 256, 256, "bf16", "f32", "normal", 2, bias=True, relu=True)
        assert got.min() == 0.0 and (got == 0.0).mean() > 0.3

    def test_ragged_with_bias(self, gpu):
        run(130, 70, 72, "bf16", "bf16", "normal", 2, bias=True, relu=True)


class TestFp8:
    @pytest.mark.parametrize("shape", [(128, 128, 128), (512, 512, 512), (200, 136, 272), (256, 1024, 4096)])
    @pytest.mark.parametrize("dtype_c", ["bf16", "f32"])
    def test_scaled(self, gpu, shape, dtype_c):
        run(*shape, "e4m3", dtype_c, "normal", 3)

    def test_against_unquantised_inputs_is_quantisation_noise(self, gpu):
        rng = np.random.default_rng(3)
        a = rng.standard_normal((256, 1024)).astype(np.float32)
        b = rng.standard_normal((256, 1024)).astype(np.float32)
        (qa, sa), (qb, sb) = orc.quantize_e4m3(a), orc.quantize_e4m3(b)
        got = gemm(qa, qb, dtype_ab="e4m3", dtype_c="f32", scale_a=float(sa), scale_b=float(sb))
        assert 0.02 < orc.rel_frobenius(got, a @ b.T) < 0.06


class TestSplitK:
    @pytest.mark.parametrize("M", [16, 128])
    @pytest.mark.parametrize("split_k", [2, 4, 8, -1])
    def test_skinny(self, gpu, M, split_k):
        run(M, 1024, 4096, "bf16", "bf16", "uniform", 4, split_k=split_k, tile_n=64)

    def test_uneven_split_and_epilogue(self, gpu):
        run(48, 200, 1000, "bf16", "f32", "uniform", 4, split_k=3, tile_n=64, bias=True, relu=True)
        run(48, 203, 1000 + 8, "bf16", "f32", "uniform", 4, split_k=5, tile_n=32)

    def test_split_k_is_deterministic(self, gpu):
        inp = orc.make_inputs(16, 512, 8192, "bf16", "uniform", 4)
        outs = [gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", split_k=8, tile_n=64) for _ in range(3)]
        assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


class TestConfiguredProblems:
    """The configured workloads at full size (seeds as configured)."""

    def test_fp16_512(self, gpu):
        inp = orc.make_inputs(512, 512, 512, "f16", "normal", 0)
        got = gemm(inp["A"], inp["B"])
        check(got, inp, "f16", "f32")
        orc.assert_reference_close(got, orc.gemm_f32(inp["A"], inp["B"]))

    def test_bf16_4096(self, gpu):
        inp = orc.make_inputs(4096, 4096, 4096, "bf16", "uniform", 1)
        check(gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="f32"), inp, "bf16", "f32")
        check(gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16"), inp, "bf16", "bf16")

    def test_fused_epilogue_8192x8192x2048(self, gpu):
        inp = orc.make_inputs(8192, 8192, 2048, "bf16", "normal", 2, with_bias=True)
        got = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", bias=inp["bias"], relu=True)
        check(got, inp, "bf16", "bf16", bias=inp["bias"], relu=True)

    def test_fp8_8192_rows_sample(self, gpu):
        # The full 8192^3 product on the GPU; the oracle checks a fixed random sample of 512 rows
        # (each row of C depends on one row of A and all of B).
        inp = orc.make_inputs(8192, 8192, 8192, "e4m3", "normal", 3)
        got = gemm(inp["A"], inp["B"], dtype_ab="e4m3", dtype_c="bf16", scale_a=inp["scale_a"], scale_b=inp["scale_b"])
        rows = np.sort(np.random.default_rng(0).choice(8192, 512, replace=False))
        sub = dict(inp, A=inp["A"][rows])
        check(got[rows], sub, "e4m3", "bf16")

    @pytest.mark.parametrize("M", [16, 128])
    def test_decode_shapes(self, gpu, M):
        inp = orc.make_inputs(M, 8192, 8192, "bf16", "uniform", 4)
        got = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", split_k=-1, tile_n=64)
        check(got, inp, "bf16", "bf16")

    # The plans the benchmark times, at the benchmark's sizes (bench.py WORKLOADS).

    @pytest.mark.parametrize("M", [16, 128])
    def test_decode_shapes_as_benchmarked(self, gpu, M):
        """Direct-B (weights packed once), static B, 128-column tiles cut in two K halves that meet
        in the shared memory of a CTA cluster."""
        kw = dict(tile_n=128, b_layout="packed", static_b=True)
        res = GemmPlan(M, 8192, 8192, "bf16", "bf16", **kw).resources()
        assert (res.tile_n, res.tail_tiles, res.tail_parts, res.tail_exchange, res.grid_ctas) == (128, 64, 2, 2, 128)
        inp = orc.make_inputs(M, 8192, 8192, "bf16", "uniform", 4)
        got = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", **kw)
        check(got, inp, "bf16", "bf16")
        # the same sums in the same order as the exchange through a lent workspace
        assert np.array_equal(got, gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", tail_split=True, workspace_exchange=True, **kw))

    def test_bf16_4096_as_benchmarked(self, gpu):
        """With the optional workspace lent: 34 of the 256 tiles are cut in two K halves."""
        res = GemmPlan(4096, 4096, 4096, "bf16", "bf16").resources()
        assert (res.tile_m, res.tile_n, res.cta_group, res.tail_tiles, res.tail_parts, res.tail_exchange) == (256, 256, 2, 34, 2, 1)
        inp = orc.make_inputs(4096, 4096, 4096, "bf16", "uniform", 1)
        check(gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", tail_split=True), inp, "bf16", "bf16")
        check(gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="f32", tail_split=True), inp, "bf16", "f32")

    def test_bf16_8192_rows_sample(self, gpu):
        inp = orc.make_inputs(8192, 8192, 8192, "bf16", "uniform", 1)
        got = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", tail_split=True)
        rows = np.sort(np.random.default_rng(0).choice(8192, 512, replace=False))
        check(got[rows], dict(inp, A=inp["A"][rows]), "bf16", "bf16")

    def test_one_shard_of_the_65536_row_problem(self, gpu):
        """Rank 3 of 8 of the M = 65536, N = K = 8192 problem: rows 24576..32767 of the global A
        (drawn block-wise so that every world size sees the same matrix), all of B."""
        from aster_b200.sharding import shard_rows, sharded_uniform_rows

        first, rows = shard_rows(65536, 8, 3)
        assert (first, rows) == (24576, 8192)
        a = orc.encode(sharded_uniform_rows(4, first, rows, 8192, threads=4), "bf16")
        b = orc.encode(np.random.default_rng(5).uniform(-1.0, 1.0, size=(8192, 8192)).astype(np.float32), "bf16")
        got = gemm(a, b, dtype_ab="bf16", dtype_c="bf16", tail_split=True)
        pick = np.sort(np.random.default_rng(0).choice(rows, 512, replace=False))
        check(got[pick], dict(A=a[pick], B=b, scale_a=None, scale_b=None), "bf16", "bf16")


class TestProperties:
    """Size-independent properties, usable where a full oracle pass would be slow."""

    def test_linearity_in_a(self, gpu):
        rng = np.random.default_rng(12)
        a1 = rng.integers(-4, 5, (512, 1024)).astype(np.float16)
        a2 = rng.integers(-4, 5, (512, 1024)).astype(np.float16)
        b = rng.integers(-4, 5, (768, 1024)).astype(np.float16)
        # small integers: every product and partial sum is exact in fp32, so linearity is exact
        assert np.array_equal(gemm(a1 + a2, b), gemm(a1, b) + gemm(a2, b))

    def test_row_shards_are_slices_of_the_whole(self, gpu):
        inp = orc.make_inputs(1024, 512, 512, "bf16", "uniform", 4)
        whole = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", tile_n=128)
        for g in (2, 4, 8):
            rows = 1024 // g
            parts = [gemm(inp["A"][r * rows:(r + 1) * rows], inp["B"], dtype_ab="bf16", dtype_c="bf16", tile_n=128) for r in range(g)]
            assert np.array_equal(np.concatenate(parts), whole)

    def test_identity_b_returns_a(self, gpu):
        a = orc.make_inputs(300, 256, 256, "bf16", "uniform", 8)["A"]
        eye = orc.encode(np.eye(256, dtype=np.float32), "bf16")
        assert np.array_equal(gemm(a, eye, dtype_ab="bf16", dtype_c="bf16"), a)


class TestBoundedWaits:
    """Failure detection without faulting the GPU: a wait that nothing will ever satisfy runs
    into its time limit, the kernel records which wait gave up and returns normally, the host
    reads B200_ERR_TIMEOUT, and the context (and the plan) stay usable."""

    @pytest.mark.parametrize("cta_group,shape", [(1, (512, 256, 512)), (2, (512, 256, 512)),
                                                 (1, (16, 1024, 4096))])  # the last: clusters of four that exchange partial sums
    def test_expired_wait_is_reported_not_hung(self, gpu, cta_group, shape):
        import time

        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        M, N, K = shape
        if M == 16:
            assert GemmPlan(M, N, K, "bf16", "f32", cta_group=cta_group, tile_n=128).resources().tail_exchange == 2
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 3)
        dA, dB, dC = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes), GpuBuffer(M * N * 4)
        dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
        stuck = GemmPlan(M, N, K, "bf16", "f32", cta_group=cta_group, tile_n=128, debug_mode=8, wait_limit_ms=50)
        t0 = time.perf_counter()
        stuck.run(dA, dB, dC)
        with pytest.raises(nat.B200Error) as e:
            stuck.status()
        elapsed = time.perf_counter() - t0
        # whichever role's wait expired first is named: 0x10 producer, 0x20 MMA issuer, 0x30 epilogue, 0x32 cluster exchange
        assert e.value.status == nat.ERR_TIMEOUT and any(f"code 0x{c:x}" in e.value.message for c in (0x10, 0x20, 0x30, 0x32))
        assert 0.04 < elapsed < 2.0
        assert stuck.status() == [0, 0, 0, 0]  # reading clears the words
        # The device and the library are still healthy: the same operands through a normal plan.
        good = GemmPlan(M, N, K, "bf16", "f32", cta_group=cta_group, tile_n=128)
        good.run(dA, dB, dC)
        good.status()
        out = np.empty((M, N), np.float32)
        dC.copy_to_host(out)
        assert float(np.max(np.abs(out - orc.gemm_f32(inp["A"], inp["B"], "bf16")))) <= orc.abs_bound(inp["A"], inp["B"], "bf16")
        for b in (dA, dB, dC):
            b.free()


class TestPlanObject:
    def test_timing_loops_and_status(self, gpu):
        from aster_b200.execution import GpuBuffer

        plan = GemmPlan(1024, 1024, 1024, "bf16", "bf16")
        bufs = [GpuBuffer(1024 * 1024 * 2) for _ in range(3)]
        for b in bufs:
            b.zero()
        t = plan.time(*bufs, iters=5)
        assert t.shape == (5,) and (t > 0).all()
        tf = plan.time(*bufs, iters=3, flush_l2=True)
        assert (tf > 0).all()
        assert plan.time_batch(*bufs, iters=4) > 0
        assert plan.status() == [0, 0, 0, 0]
        # cycle / nanosecond totals of the launches in between: their average SM clock
        from aster_b200.gemm import mean_sm_mhz

        before = plan.clock_totals()
        for _ in range(5):
            plan.run(*bufs)
        after = plan.clock_totals()
        assert after[2] - before[2] == 5 and 300.0 < mean_sm_mhz(before, after) < 2200.0
        assert 300.0 < plan.last_sm_mhz() < 2200.0
        assert plan.resources().regs_per_thread > 0
        for b in bufs:
            b.free()

    def test_milestone_timeline(self, gpu):
        """The bring-up timeline: every CTA's stamps are in causal order and within the launch."""
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        if not nat.is_bringup_build():
            pytest.skip("the per-CTA timeline exists only in a library built with -DB200_BRINGUP")
        plan = GemmPlan(1024, 1024, 2048, "bf16", "bf16", no_tail_split=True)
        grid = plan.resources().grid_ctas
        bufs = [GpuBuffer(n) for n in (1024 * 2048 * 2, 1024 * 2048 * 2, 1024 * 1024 * 2)]
        for b in bufs:
            b.zero()
        tl = GpuBuffer(grid * 16 * 8)
        tl.zero()
        nat.call("b200_gemm_debug_timeline", plan.handle, tl.ptr)
        plan.run(*bufs)
        nat.call("b200_device_synchronize")
        nat.call("b200_gemm_debug_timeline", plan.handle, None)
        t = np.zeros((grid, 16), np.uint64)
        tl.copy_to_host(t)
        t = t.astype(np.int64)
        leaders = t[::plan.resources().cta_group]
        for a, b in ((0, 1), (1, 2), (2, 3), (3, 4), (4, 5), (5, 6), (6, 7), (7, 8)):
            assert (leaders[:, a] <= leaders[:, b]).all(), (a, b)
        assert (t[:, 0] > 0).all() and (t[:, 8] - t[:, 0]).max() < 5_000_000  # ns
        plan.run(*bufs)  # detached: launches no longer write the buffer
        nat.call("b200_device_synchronize")
        again = np.zeros((grid, 16), np.uint64)
        tl.copy_to_host(again)
        assert np.array_equal(again.astype(np.int64), t)

    def test_bound_launch_equals_run(self, gpu):
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        inp = orc.make_inputs(256, 384, 512, "bf16", "uniform", 9)
        plan = GemmPlan(256, 384, 512, "bf16", "f32")
        dA, dB = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes)
        dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
        outs = []
        for use_bind in (False, True):
            dC = GpuBuffer(256 * 384 * 4)
            dC.zero()
            if use_bind:
                launch = plan.bind(dA, dB, dC)
                launch()
                launch()  # reusable
            else:
                plan.run(dA, dB, dC)
            nat.call("b200_device_synchronize")
            out = np.empty((256, 384), np.float32)
            dC.copy_to_host(out)
            outs.append(out)
        assert np.array_equal(outs[0], outs[1])
        check(outs[1], inp, "bf16", "f32")


class TestDependentLaunch:
    """Launches use programmatic stream serialisation: a kernel may set itself up, and with
    ``static_b`` request its first B tiles, while the previous kernel of the stream finishes.
    Whatever one launch reads from the previous one must still be complete."""

    def test_second_gemm_reads_the_first_ones_output(self, gpu):
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        M, K1, N1, N2 = 256, 4096, 2048, 512  # C1 [M, N1] is the A operand of the second product
        rng = np.random.default_rng(3)
        a1 = orc.encode(rng.uniform(-1, 1, (M, K1)).astype(np.float32), "bf16")
        b1 = orc.encode(rng.uniform(-1, 1, (N1, K1)).astype(np.float32) / 64, "bf16")
        b2 = orc.encode(rng.uniform(-1, 1, (N2, N1)).astype(np.float32), "bf16")
        p1 = GemmPlan(M, N1, K1, "bf16", "bf16")
        p2 = GemmPlan(M, N2, N1, "bf16", "f32", static_b=True)
        bufs = [GpuBuffer(x.nbytes) for x in (a1, b1, b2)]
        for buf, x in zip(bufs, (a1, b1, b2)):
            buf.copy_from_host(x)
        c1, c2 = GpuBuffer(M * N1 * 2), GpuBuffer(M * N2 * 4)
        results = []
        for _ in range(3):  # back to back, no synchronisation between the two launches
            c1.zero()
            c2.zero()
            p1.run(bufs[0], bufs[1], c1)
            p2.run(c1, bufs[2], c2)
            nat.call("b200_device_synchronize")
            h1, h2 = np.empty((M, N1), np.uint16), np.empty((M, N2), np.float32)
            c1.copy_to_host(h1)
            c2.copy_to_host(h2)
            results.append((h1, h2))
        h1, h2 = results[0]
        check(h1, dict(A=a1, B=b1, scale_a=None, scale_b=None), "bf16", "bf16")
        check(h2, dict(A=h1, B=b2, scale_a=None, scale_b=None), "bf16", "f32")  # from the bits the first launch wrote
        assert all(np.array_equal(h1, r[0]) and np.array_equal(h2, r[1]) for r in results[1:])

    @pytest.mark.parametrize("shape,kw", [((16, 1024, 4096), dict(tile_n=128, tail_split=True)), ((512, 512, 1024), {}),
                                           ((300, 200, 520), dict(cta_group=1, b_layout="packed")),
                                           ((48, 200, 1000), dict(split_k=3, tile_n=64)), ((2048, 1024, 512), dict(stages=3))])
    def test_static_b_does_not_change_results(self, gpu, shape, kw):
        inp = orc.make_inputs(*shape, "bf16", "uniform", 6)
        plain = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", **kw)
        early = [gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", static_b=True, **kw) for _ in range(2)]
        assert np.array_equal(plain, early[0]) and np.array_equal(plain, early[1])
        no_pdl = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", debug_mode=16, **kw)
        assert np.array_equal(plain, no_pdl)


class TestSharedKernelInstances:
    def test_plans_with_different_rings_take_turns(self, gpu):
        """Plans of one tile shape share a kernel instance whatever their ring depth: a plan with a
        shallow ring set up after a deep one must not leave the deep one unable to launch."""
        M, N, K = 256, 256, 2048
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 11)
        kw = dict(dtype_ab="bf16", dtype_c="f32")
        deep = GemmPlan(M, N, K, "bf16", "f32", tile_n=128, cta_group=1, stages=6)
        shallow = GemmPlan(M, N, K, "bf16", "f32", tile_n=128, cta_group=1, stages=2)
        assert deep.resources().smem_bytes > shallow.resources().smem_bytes
        first = gemm(inp["A"], inp["B"], plan=deep, **kw)
        second = gemm(inp["A"], inp["B"], plan=shallow, **kw)
        third = gemm(inp["A"], inp["B"], plan=deep, **kw)
        assert np.array_equal(first, second) and np.array_equal(first, third)
        check(first, inp, "bf16", "f32")


    def test_plan_rotating_over_more_buffers_than_it_caches_maps_for(self, gpu):
        """A plan keeps the tensor maps of its last few operand addresses; six operand sets taking
        turns (twice around) must each produce their own product."""
        from aster_b200.execution import GpuBuffer

        M, N, K = 256, 256, 512
        plan = GemmPlan(M, N, K, "bf16", "f32", tile_n=128)
        sets = []
        for i in range(6):
            inp = orc.make_inputs(M, N, K, "bf16", "uniform", 20 + i)
            dA, dB, dC = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes), GpuBuffer(M * N * 4)
            dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
            sets.append((inp, dA, dB, dC))
        for _ in range(2):
            for inp, dA, dB, dC in sets:
                dC.zero()
                plan.run(dA, dB, dC)
        plan.status()
        for inp, dA, dB, dC in sets:
            out = np.empty((M, N), np.float32)
            dC.copy_to_host(out)
            check(out, inp, "bf16", "f32")
            for b in (dA, dB, dC):
                b.free()


class TestSkinnyM:
    """M <= 64: stages hold only 32 or 64 rows of A (more ring slots for B).  Same MMAs in the
    same order as with full A stages, so the results are bit-identical to ``tile_m=128``."""

    @pytest.mark.parametrize("M", [1, 8, 16, 32, 33, 48, 64])
    @pytest.mark.parametrize("kw", [dict(tile_n=64), dict(tile_n=128), dict(tile_n=128, tail_split=True), dict(tile_n=64, split_k=2),
                                    dict(tile_n=64, b_layout="packed")])
    def test_equals_full_a_stages_bitwise(self, gpu, M, kw):
        N, K = 1024, 4096
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 4)
        short = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", **kw)
        full = gemm(inp["A"], inp["B"], dtype_ab="bf16", dtype_c="bf16", tile_m=128, **kw)
        assert np.array_equal(short, full)
        check(short, inp, "bf16", "bf16")

    @pytest.mark.parametrize("M,N,K,kw,parts", [
        (16, 1024, 4096, dict(tile_n=64), 2),                   # 16 tiles x 2 parts: clusters of two
        (16, 1024, 4096, dict(tile_n=128), 4),                  # 8 tiles x 4 parts: clusters of four
        (128, 8192, 4096, dict(tile_n=128), 2),                 # full A stages, all four epilogue warps exchange
        (100, 1000, 8192, dict(tile_n=128), 4),                 # ragged rows and columns in the exchanged tiles
        (64, 512, 8192, dict(tile_n=256), 8),                   # 2 tiles x 8 parts: clusters of eight
        (16, 8192, 4096, dict(tile_n=128, b_layout="packed", static_b=True), 2),  # direct-B, as the decode workloads run
    ])
    @pytest.mark.parametrize("dtype_c", ["bf16", "f32"])
    def test_cluster_exchange_equals_workspace_exchange_bitwise(self, gpu, M, N, K, kw, parts, dtype_c):
        """One round of tiles, each cut along K: the parts of a tile are the CTAs of a cluster and
        meet in its shared memory.  Same partial sums added in the same order as when they meet
        in the lent workspace, so the two forms agree bit for bit, and with the oracle."""
        res = GemmPlan(M, N, K, "bf16", dtype_c, **kw).resources()
        assert (res.tail_parts, res.tail_exchange, res.optional_workspace_bytes) == (parts, 2, 0)
        assert res.grid_ctas == res.num_tiles * parts
        via_ws = GemmPlan(M, N, K, "bf16", dtype_c, workspace_exchange=True, **kw).resources()
        assert (via_ws.tail_parts, via_ws.tail_exchange) == (parts, 1) and via_ws.optional_workspace_bytes > 0
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 4, with_bias=True)
        common = dict(dtype_ab="bf16", dtype_c=dtype_c, bias=inp["bias"], relu=True)
        cluster = gemm(inp["A"], inp["B"], **common, **kw)
        workspace = gemm(inp["A"], inp["B"], **common, tail_split=True, workspace_exchange=True, **kw)
        assert np.array_equal(cluster, workspace)
        check(cluster, inp, "bf16", dtype_c, bias=inp["bias"], relu=True)

    def test_cluster_exchange_back_to_back_launches(self, gpu):
        """The parking area is the stage ring: a launch must not disturb the next one (dependent
        launches overlap the next launch's prologue with this one's end)."""
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer

        M, N, K = 16, 4096, 4096
        inp = orc.make_inputs(M, N, K, "bf16", "uniform", 9)
        plan = GemmPlan(M, N, K, "bf16", "bf16", tile_n=128)
        assert plan.resources().tail_exchange == 2
        dA, dB = GpuBuffer(inp["A"].nbytes), GpuBuffer(inp["B"].nbytes)
        dA.copy_from_host(inp["A"]), dB.copy_from_host(inp["B"])
        outs = [GpuBuffer(M * N * 2) for _ in range(6)]
        for o in outs:
            plan.run(dA, dB, o)
        nat.call("b200_device_synchronize")
        plan.status()
        first = np.empty((M, N), np.uint16)
        outs[0].copy_to_host(first)
        check(first, inp, "bf16", "bf16")
        for o in outs[1:]:
            got = np.empty((M, N), np.uint16)
            o.copy_to_host(got)
            assert np.array_equal(got, first)
        for b in (dA, dB, *outs):
            b.free()

    def test_deep_rings_and_other_types(self, gpu):
        # short A stages: as many slots as put 112 KB of B tiles on request (14 of 8 KB, 7 of 16 KB), 16 on demand
        plan = GemmPlan(16, 8192, 8192, "bf16", "bf16", tile_n=64)
        assert plan.resources().stages == 14 and GemmPlan(16, 8192, 8192, "bf16", "bf16", tile_n=64, tile_m=128).resources().stages <= 8
        assert GemmPlan(16, 8192, 8192, "bf16", "bf16", tile_n=128).resources().stages == 7
        assert GemmPlan(16, 8192, 8192, "bf16", "bf16", tile_n=64, stages=16).resources().stages == 16
        run(16, 2048, 8192, "bf16", "f32", "uniform", 4, tile_n=64, bias=True, relu=True)
        run(16, 2048, 8192, "bf16", "f32", "uniform", 4, tile_n=64, stages=16)
        run(16, 1024, 8192, "bf16", "bf16", "uniform", 4, tile_n=128, stages=11)  # the deepest ring of 20 KB stages
        run(24, 1000, 2064, "f16", "f32", "normal", 5, tile_n=64)            # ragged N, K not a multiple of the stage
        run(40, 512, 4096, "e4m3", "bf16", "normal", 3, tile_n=128)
        ia = np.random.default_rng(1).integers(-128, 128, (16, 2048), dtype=np.int8)
        ib = np.random.default_rng(2).integers(-128, 128, (512, 2048), dtype=np.int8)
        assert np.array_equal(gemm(ia, ib, dtype_ab="i8", dtype_c="i32", tile_n=64), orc.gemm_i32(ia, ib))
