"""Further operand types on the tensor cores, each against the CPU oracle on the same inputs:
8-bit integers with 32-bit integer sums (the reference's v_mfma_i32_16x16x32_i8,
include/aster/Dialect/AMDGCN/IR/Instructions/MMA.td:636-651) -- bit-exact -- and fp8 e5m2 alone
or mixed with e4m3 (v_mfma_f32_16x16x32_bf8_bf8 / _bf8_fp8 / _fp8_bf8, MMA.td:138-210).

Tolerances: integer sums are compared with ``array_equal``; dequantised integer output and the
8-bit float types use the rules of the other GEMM tests (relative Frobenius error <= 1e-3 against
the oracle on the same stored inputs: only the fp32 summation order differs)."""

import numpy as np
import pytest

from aster_b200 import _native as nat
from aster_b200.dtypes import from_f32
from aster_b200.gemm import GemmPlan, gemm
from oracle import gemm_oracle as orc

pytestmark = pytest.mark.gpu


def int8_inputs(M, N, K, seed, lo=-128, hi=128):
    rng = np.random.default_rng(seed)
    return rng.integers(lo, hi, (M, K), dtype=np.int8), rng.integers(lo, hi, (N, K), dtype=np.int8)


class TestInt8:
    def test_known_answers(self, gpu):
        # ones x ones over K = 32 -> 32 (the K-32 MFMA known answer), and the extreme products
        a, b = np.ones((16, 32), np.int8), np.ones((16, 32), np.int8)
        assert np.array_equal(gemm(a, b, dtype_ab="i8", dtype_c="i32"), np.full((16, 16), 32, np.int32))
        a, b = np.full((128, 64), -128, np.int8), np.full((64, 64), -128, np.int8)
        assert np.array_equal(gemm(a, b, dtype_ab="i8", dtype_c="i32"), np.full((128, 64), 64 * 16384, np.int32))
        b = np.full((64, 64), 127, np.int8)
        assert np.array_equal(gemm(a, b, dtype_ab="i8", dtype_c="i32"), np.full((128, 64), -64 * 128 * 127, np.int32))

    @pytest.mark.parametrize("shape", [(128, 128, 128), (256, 256, 512), (100, 72, 272), (512, 1000, 1040), (1024, 512, 8192)])
    @pytest.mark.parametrize("kw", [{}, {"cta_group": 1, "tile_n": 64}, {"cta_group": 1, "tile_n": 256, "stages": 3}])
    def test_sums_are_exact(self, gpu, shape, kw):
        a, b = int8_inputs(*shape, seed=sum(shape))
        got = gemm(a, b, dtype_ab="i8", dtype_c="i32", **kw)
        assert got.dtype == np.int32 and np.array_equal(got, orc.gemm_i32(a, b))

    def test_pair_and_direct_b_give_the_same_integers(self, gpu):
        a, b = int8_inputs(512, 384, 1024, seed=9)
        want = orc.gemm_i32(a, b)
        assert np.array_equal(gemm(a, b, dtype_ab="i8", dtype_c="i32", cta_group=2, tile_n=128), want)
        assert np.array_equal(gemm(a, b, dtype_ab="i8", dtype_c="i32", b_layout="packed", tile_n=128), want)

    def test_full_size_rows_sample(self, gpu):
        # 4096 x 4096 x 8192 on the GPU; the oracle checks a fixed sample of 256 rows
        a, b = int8_inputs(4096, 4096, 8192, seed=12)
        got = gemm(a, b, dtype_ab="i8", dtype_c="i32")
        rows = np.sort(np.random.default_rng(0).choice(4096, 256, replace=False))
        assert np.array_equal(got[rows], orc.gemm_i32(a[rows], b))

    @pytest.mark.parametrize("dtype_c", ["f32", "bf16"])
    def test_dequantised_output_with_epilogue(self, gpu, dtype_c):
        a, b = int8_inputs(256, 200, 512, seed=5, lo=-20, hi=21)  # |sums| < 2^24: the float conversion is exact
        bias = (np.random.default_rng(6).standard_normal(200) * 3).astype(np.float32)
        got = gemm(a, b, dtype_ab="i8", dtype_c=dtype_c, bias=bias, relu=True, scale_a=0.05, scale_b=0.02)
        want = orc.gemm(a, b, "i8", dtype_c, bias=bias, relu=True, scale_a=0.05, scale_b=0.02)
        if dtype_c == "f32":
            assert np.allclose(got, want, rtol=1e-6, atol=1e-6)  # one fused multiply-add rounding apart at most
        else:
            assert np.max(orc.bf16_ulp_distance(got, want)) <= 1

    def test_refusals(self, gpu):
        with pytest.raises(nat.B200Error, match="do not split K"):
            GemmPlan(16, 256, 4096, "i8", "i32", split_k=4)
        with pytest.raises(nat.B200Error, match="i32 output needs i8 inputs"):
            GemmPlan(128, 128, 128, "bf16", "i32")
        with pytest.raises(nat.B200Error, match="need f32 or bf16 output"):
            GemmPlan(128, 128, 128, "i8", "i32", epilogue="bias")
        a, b = int8_inputs(64, 64, 64, seed=1)
        with pytest.raises(nat.B200Error, match="scales need f32 or bf16 output"):
            gemm(a, b, dtype_ab="i8", dtype_c="i32", scale_a=0.5)
        # auto split (-1) simply does not split
        assert GemmPlan(16, 256, 4096, "i8", "i32", split_k=-1).resources().split_k == 1


class TestE5M2:
    def test_known_answers(self, gpu):
        # 1.5 x 2.0 over K = 32 -> 96, as the reference's fp8 known answer with other constants
        a = from_f32(np.full((16, 32), 1.5, np.float32), "e5m2")
        b = from_f32(np.full((16, 32), 2.0, np.float32), "e5m2")
        assert np.array_equal(gemm(a, b, dtype_ab="e5m2", dtype_c="f32"), np.full((16, 16), 96.0, np.float32))

    @pytest.mark.parametrize("dtype_ab", ["e5m2", "e5m2_e4m3", "e4m3_e5m2"])
    @pytest.mark.parametrize("shape", [(128, 128, 128), (200, 136, 272), (512, 512, 2048)])
    def test_against_oracle(self, gpu, dtype_ab, shape):
        M, N, K = shape
        ta, tb = orc.operand_types(dtype_ab)
        rng = np.random.default_rng(M + K)
        a = orc.encode(rng.standard_normal((M, K)).astype(np.float32), ta)
        b = orc.encode(rng.standard_normal((N, K)).astype(np.float32), tb)
        for dtype_c in ("f32", "bf16"):
            got = gemm(a, b, dtype_ab=dtype_ab, dtype_c=dtype_c)
            want = orc.decode(orc.encode(orc.gemm_f32(a, b, dtype_ab), dtype_c), dtype_c)
            assert orc.rel_frobenius(orc.decode(got, dtype_c), want) <= 1e-3

    def test_mixed_types_are_not_symmetric(self, gpu):
        # the same bytes read as (e5m2, e4m3) and as (e4m3, e5m2) give different products
        rng = np.random.default_rng(2)
        a = rng.integers(0, 0x58, (128, 128), dtype=np.uint8)
        b = rng.integers(0, 0x58, (128, 128), dtype=np.uint8)
        x = gemm(a, b, dtype_ab="e5m2_e4m3", dtype_c="f32")
        y = gemm(a, b, dtype_ab="e4m3_e5m2", dtype_c="f32")
        assert orc.rel_frobenius(x, orc.gemm_f32(a, b, "e5m2_e4m3")) <= 1e-3
        assert orc.rel_frobenius(y, orc.gemm_f32(a, b, "e4m3_e5m2")) <= 1e-3
        assert not np.allclose(x, y)


def test_int8_through_the_operator_surface(gpu, tmp_path):
    """compile_fn / execute_fn with an i8 -> i32 instance: the label carries the types."""
    from aster_b200.gemm_config import B200GemmInstance, make_b200_instance
    from aster_b200.multitile_gemm import compile_multitile_gemm, execute_multitile_hsaco

    cfg = make_b200_instance(384, 256, 512, dtype_ab="i8", dtype_c="i32")
    assert B200GemmInstance.from_label(cfg.label).label == cfg.label and "_b200_i8_oi32_" in cfg.label
    path, _ = compile_multitile_gemm(cfg, str(tmp_path / "i8.json"))
    a, b = int8_inputs(384, 256, 512, seed=3)
    c, times = execute_multitile_hsaco(cfg, path, 3, a, b, skip_gpu_check=True)
    assert len(times) == 3 and c.dtype == np.int32 and np.array_equal(c.reshape(384, 256), orc.gemm_i32(a, b))


def mx_inputs(M, N, K, seed, elem="e4m3", spread=True):
    """Random operands whose 32-element blocks differ in magnitude by orders, so that the block
    scales matter; quantised by the oracle's own block-by-block routine."""
    rng = np.random.default_rng(seed)

    def draw(rows):
        x = rng.standard_normal((rows, K)).astype(np.float32)
        if spread:
            x *= np.repeat(np.exp2(rng.integers(-12, 13, (rows, K // 32))).astype(np.float32), 32, axis=1)
        return x

    a, b = draw(M), draw(N)
    (qa, sa), (qb, sb) = orc.mx_quantize(a, elem), orc.mx_quantize(b, elem)
    return a, b, qa, sa, qb, sb


class TestBlockScaledFp8:
    """E8M0 scales per 32 elements of K, applied inside the tensor core (the reference's
    v_mfma_scale_f32_16x16x128_f8f6f4 tests, test/integration/test_mfma_f8f6f4_e2e.py:39-95)."""

    def test_known_answers(self, gpu):
        # 1.75 x 1.25 over K = 128 with scales 4 and 2 -> 1.75 * 1.25 * 128 * 8 = 2240
        M = N = 16
        a = from_f32(np.full((M, 128), 1.75, np.float32), "e4m3")
        b = from_f32(np.full((N, 128), 1.25, np.float32), "e4m3")
        sa, sb = np.full((M, 4), 129, np.uint8), np.full((N, 4), 128, np.uint8)
        got = gemm(a, b, dtype_ab="mxe4m3", dtype_c="f32", block_scales_a=sa, block_scales_b=sb)
        assert np.array_equal(got, np.full((M, N), 2240.0, np.float32))
        # two halves of K with different scales: 64 * (1 * 1) * 2 + 64 * (1.5 * 1) * 0.5 = 176
        a = from_f32(np.concatenate([np.full((M, 64), 1.0), np.full((M, 64), 1.5)], axis=1).astype(np.float32), "e4m3")
        b = from_f32(np.ones((N, 128), np.float32), "e4m3")
        sa = np.repeat(np.uint8([[128, 128, 126, 126]]), M, axis=0)
        sb = np.full((N, 4), 127, np.uint8)
        got = gemm(a, b, dtype_ab="mxe4m3", dtype_c="f32", block_scales_a=sa, block_scales_b=sb)
        assert np.array_equal(got, np.full((M, N), 176.0, np.float32))

    def test_each_row_and_block_uses_its_own_scale(self, gpu):
        # ones everywhere; scales chosen so that C[m, n] = sum_kb 2^(ea[m, kb] + eb[n, kb]) * 32 is distinct per (m, n)
        M, N, K = 256, 128, 256
        rng = np.random.default_rng(1)
        sa = rng.integers(124, 131, (M, K // 32)).astype(np.uint8)  # sums stay within 24 significant bits
        sb = rng.integers(124, 131, (N, K // 32)).astype(np.uint8)
        ones = from_f32(np.ones((max(M, N), K), np.float32), "e4m3")
        got = gemm(ones[:M], ones[:N], dtype_ab="mxe4m3", dtype_c="f32", block_scales_a=sa, block_scales_b=sb)
        want = 32.0 * (np.exp2(sa.astype(np.float64) - 127) @ np.exp2(sb.astype(np.float64) - 127).T)
        assert np.array_equal(got, want.astype(np.float32))  # powers of two: exact

    @pytest.mark.parametrize("cta_group", [1, 2])
    @pytest.mark.parametrize("tile_n", [128, 256])
    @pytest.mark.parametrize("elem", ["e4m3", "e5m2"])
    @pytest.mark.parametrize("shape", [(128, 128, 128), (256, 384, 1024), (200, 136, 160), (1000, 520, 2080), (512, 512, 8192)])
    def test_against_oracle(self, gpu, elem, shape, tile_n, cta_group):
        M, N, K = shape
        a, b, qa, sa, qb, sb = mx_inputs(M, N, K, seed=M + K, elem=elem)
        want = orc.gemm_mx(qa, qb, sa, sb, elem)
        for dtype_c in ("f32", "bf16"):
            got = gemm(qa, qb, dtype_ab="mx" + elem, dtype_c=dtype_c, block_scales_a=sa, block_scales_b=sb, tile_n=tile_n, cta_group=cta_group)
            want_c = orc.decode(orc.encode(want, dtype_c), dtype_c)
            assert orc.rel_frobenius(orc.decode(got, dtype_c), want_c) <= 1e-3
        # against the unquantised product the error is the quantisation noise of the format
        noise = orc.rel_frobenius(orc.gemm_mx(qa, qb, sa, sb, elem), a.astype(np.float64) @ b.astype(np.float64).T)
        assert noise < (0.08 if elem == "e4m3" else 0.16)

    def test_epilogue_split_k_and_tail_split(self, gpu):
        M, N, K = 384, 256, 4096
        _, _, qa, sa, qb, sb = mx_inputs(M, N, K, seed=4, spread=False)
        bias = np.random.default_rng(5).standard_normal(N).astype(np.float32)
        want = np.maximum(orc.gemm_mx(qa, qb, sa, sb) + bias[None, :], 0)
        kw = dict(dtype_ab="mxe4m3", dtype_c="f32", block_scales_a=sa, block_scales_b=sb, bias=bias, relu=True)
        for extra in ({}, {"split_k": 3}, {"max_ctas": 4, "tail_split": True}, {"stages": 2}, {"tile_n": 256}, {"tile_n": 256, "max_ctas": 2},
                      {"tile_n": 256, "split_k": 2, "stages": 3}, {"cta_group": 1}, {"cta_group": 1, "tile_n": 128, "max_ctas": 3, "tail_split": True},
                      {"cta_group": 2, "tile_n": 128, "split_k": 2}, {"cta_group": 2, "tile_n": 256, "max_ctas": 2, "tail_split": True},
                      {"static_b": True}, {"static_b": True, "cta_group": 1, "stages": 2}):
            assert orc.rel_frobenius(gemm(qa, qb, **kw, **extra), want) <= 1e-3, extra

    def test_refusals(self, gpu):
        with pytest.raises(nat.B200Error, match="K %% 32 == 0|K % 32 == 0"):
            GemmPlan(128, 128, 144, "mxe4m3", "f32")
        with pytest.raises(nat.B200Error, match="tile_n=128 or 256"):
            GemmPlan(256, 256, 128, "mxe4m3", "f32", tile_n=64)
        with pytest.raises(nat.B200Error, match="not block-scaled"):
            GemmPlan(128, 128, 128, "e4m3", "f32").set_mx_scales(16, 16)
        plan = GemmPlan(128, 128, 128, "mxe4m3", "f32")
        with pytest.raises(nat.B200Error, match="needs its scales first"):
            plan.run(1024, 2048, 4096)
