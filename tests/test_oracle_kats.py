"""Pins the CPU oracle: the reference's known-answer tests, restated on the oracle, plus
cross-checks of the oracle's pieces against each other and against the product's host code."""

import numpy as np
import pytest

from aster_b200 import dtypes as pd
from aster_b200.kittens_helpers import shuffle_weight as product_shuffle
from oracle import gemm_oracle as orc


def full(shape, value, dtype):
    return orc.encode(np.full(shape, value, dtype=np.float32), dtype)


class TestKnownAnswers:
    def test_f16_ones_times_twos_16(self):
        # test/integration/test_mfma_e2e.py:36-46: A = 1, B = 2, 16x16x16 -> every C == 32.
        c = orc.gemm_f32(full((16, 16), 1.0, "f16"), full((16, 16), 2.0, "f16"), "f16")
        assert np.all(c == 32.0)

    def test_fp8_ones_k32(self):
        # test/integration/test_mfma_fp8_e2e.py:39-60: ones, K = 32 -> 32.
        c = orc.gemm_f32(full((16, 32), 1.0, "e4m3"), full((16, 32), 1.0, "e4m3"), "e4m3")
        assert np.all(c == 32.0)

    def test_fp8_with_initial_accumulator(self):
        # test_mfma_fp8_e2e.py:62-95: 1.5 * 2.0 * 32 + 10 = 106; the initial accumulator is a bias here.
        acc = orc.gemm_f32(full((16, 32), 1.5, "e4m3"), full((16, 32), 2.0, "e4m3"), "e4m3")
        c = orc.gemm_epilogue(acc, bias=np.full(16, 10.0, np.float32))
        assert np.all(c == 106.0)

    @pytest.mark.parametrize("dtype", ["f16", "bf16"])
    def test_doubled_k_ones(self, dtype):
        # test/integration/test_mfma_cdna4_doubled_k_e2e.py:48-164: ones, K = 32 -> 32; 32x32x16 -> 16.
        assert np.all(orc.gemm_f32(full((16, 32), 1.0, dtype), full((16, 32), 1.0, dtype), dtype) == 32.0)
        assert np.all(orc.gemm_f32(full((32, 16), 1.0, dtype), full((32, 16), 1.0, dtype), dtype) == 16.0)

    def test_scaled_fp8(self):
        # test/integration/test_mfma_f8f6f4_e2e.py:39-66: 1.75 * 1.25 * 128 * (4 * 2) = 2240,
        # with the block scales (4, 2) expressed as per-tensor scales.
        a, b = full((16, 128), 1.75, "e4m3"), full((16, 128), 1.25, "e4m3")
        c = orc.decode(orc.gemm(a, b, "e4m3", "f32", scale_a=4.0, scale_b=2.0), "f32")
        assert np.all(c == 2240.0)

    def test_scaled_fp8_two_halves(self):
        # test_mfma_f8f6f4_e2e.py:68-95: 64*1*2 + 64*1.5*0.5 + 10 = 186 (two K halves with
        # different scales, then the initial accumulator).
        ones = full((16, 64), 1.0, "e4m3")
        first = orc.gemm_epilogue(orc.gemm_f32(ones, ones, "e4m3"), alpha=2.0)
        second = orc.gemm_epilogue(orc.gemm_f32(full((16, 64), 1.5, "e4m3"), ones, "e4m3"), alpha=0.5)
        assert np.all(first + second + 10.0 == 186.0)

    def test_bf16_amx_tile(self):
        # contrib/cpu/test/integration/test_tdpbf16ps_e2e.py:29-38: A = 1 (16x32), B = 2 -> 64.
        assert np.all(orc.gemm_f32(full((16, 32), 1.0, "bf16"), full((16, 32), 2.0, "bf16"), "bf16") == 64.0)

    def test_vector_add(self):
        # examples/03_vector_add/run.py:44-53.
        a, b = np.arange(64, dtype=np.int32), np.full(64, 100, dtype=np.int32)
        assert np.array_equal(orc.vector_add(a, b), np.arange(100, 164, dtype=np.int32))
        big = np.array([2**31 - 1], dtype=np.int32)
        assert orc.vector_add(big, np.array([1], dtype=np.int32))[0] == -(2**31)  # v_add_u32 wraps

    def test_copy_keeps_sentinel_outside(self):
        # examples/06_copy_layout/copy_2d_padded.py:131-143.
        src = np.arange(64 * 300, dtype=np.float32).reshape(64, 300)
        dst = np.full((64, 300), -999.0, np.float32)
        assert np.array_equal(orc.copy_2d_padded(src, dst), src)

    def test_add_relu(self):
        # examples/07_simple_fusion/simple_fusion.py:133-144.
        a = np.array([1.0, -2.0, 3.0, -4.0], np.float32)
        b = np.array([-0.5, 1.0, -4.0, 5.0], np.float32)
        assert np.allclose(orc.add_relu(a, b), [0.5, 0.0, 0.0, 1.0], atol=1e-5)


class TestOracleConsistency:
    @pytest.mark.parametrize("dtype", ["f16", "bf16", "e4m3"])
    def test_blas_matches_plain_loop(self, dtype):
        inp = orc.make_inputs(24, 40, 96, dtype, "normal", 11)
        blas = orc.gemm_f32(inp["A"], inp["B"], dtype)
        loop = orc.gemm_scalar_f32(inp["A"], inp["B"], dtype)
        assert np.max(np.abs(blas - loop)) <= 1e-4 * max(1.0, float(np.abs(loop).max()))

    def test_reference_random_case(self):
        # The reference's own random case: seed 42+M+N+K, randn * 0.1 in f16, rtol = atol = 1e-2
        # (test_102_gemm_python_multitile_lds_cdna3.py:492-505), here oracle vs plain loop.
        M, N, K = 48, 32, 128
        np.random.seed(42 + M + N + K)
        A = (np.random.randn(M, K) * 0.1).astype(np.float16)
        B = (np.random.randn(N, K) * 0.1).astype(np.float16)
        orc.assert_reference_close(orc.gemm_f32(A, B), orc.gemm_scalar_f32(A, B))

    def test_transposed_store_identity(self):
        # python/test/integration/test_layout_mfma_e2e.py:88-92: (A @ B.T).T == B @ A.T.
        inp = orc.make_inputs(16, 16, 16, "f16", "normal", 3)
        np.testing.assert_allclose(orc.gemm_f32(inp["A"], inp["B"]).T, orc.gemm_f32(inp["B"], inp["A"]), rtol=1e-6)

    def test_shuffle_weight_golden(self, golden):
        small = np.arange(16 * 32, dtype=np.int16).reshape(16, 32)
        assert orc.shuffle_weight(small).reshape(-1).tolist() == golden["shuffle_weight"]["small_16x32"]
        # Row 0 of the packed buffer: lanes 0 and 1 of lane-group 0, each [k0..3, k16..19].
        assert orc.shuffle_weight(small)[0, :16].tolist() == [0, 1, 2, 3, 16, 17, 18, 19, 32, 33, 34, 35, 48, 49, 50, 51]

    def test_shuffle_weight_big_golden_and_inverse(self, golden):
        import hashlib

        big = (np.arange(64 * 128, dtype=np.int64) * 7 % 65521).astype(np.uint16).reshape(64, 128)
        s = orc.shuffle_weight(big)
        assert hashlib.sha256(s.tobytes()).hexdigest() == golden["shuffle_weight"]["big_64x128_sha256"]
        assert np.array_equal(orc.unshuffle_weight(s), big)
        assert np.array_equal(product_shuffle(big), s)

    def test_gemm_invariant_under_shuffle_roundtrip(self):
        inp = orc.make_inputs(32, 48, 64, "f16", "normal", 5)
        b2 = orc.unshuffle_weight(orc.shuffle_weight(inp["B"]))
        assert np.array_equal(orc.gemm_f32(inp["A"], b2), orc.gemm_f32(inp["A"], inp["B"]))

    def test_shuffle_weight_rejects_bad_shapes(self):
        with pytest.raises(AssertionError):
            orc.shuffle_weight(np.zeros((15, 32), np.float16))
        with pytest.raises(AssertionError):
            product_shuffle(np.zeros((16, 48), np.float16))


class TestElementTypes:
    """The product's host conversions against the oracle's (independent implementations)."""

    def test_bf16_encode_matches(self):
        x = np.random.default_rng(0).standard_normal(100000).astype(np.float32) * np.float32(37.0)
        assert np.array_equal(pd.f32_to_bf16_bits(x), orc.bf16_encode(x))
        assert np.array_equal(pd.bf16_bits_to_f32(pd.f32_to_bf16_bits(x)), orc.bf16_decode(orc.bf16_encode(x)))

    def test_bf16_ties_to_even(self):
        # 1 + 2^-8 is exactly between two bf16 values; even mantissa wins.
        x = np.array([1.0 + 2.0**-8, 1.0 + 3 * 2.0**-8], np.float32)
        assert pd.bf16_bits_to_f32(pd.f32_to_bf16_bits(x)).tolist() == [1.0, 1.0 + 2.0**-6]

    def test_e4m3_all_codes_roundtrip(self):
        codes = np.arange(256, dtype=np.uint8)
        vals = pd.e4m3_bits_to_f32(codes)
        assert np.array_equal(np.isnan(vals), (codes & 0x7F) == 0x7F)
        finite = ~np.isnan(vals)
        assert np.array_equal(pd.f32_to_e4m3_bits(vals[finite]) & 0x7F, codes[finite] & 0x7F)
        assert np.array_equal(orc.e4m3_decode(codes)[finite], vals[finite])
        assert vals[0x7E] == 448.0 and vals[0x01] == 2.0**-9

    def test_e4m3_encode_matches(self):
        rng = np.random.default_rng(1)
        for scale in (0.01, 1.0, 100.0):
            x = np.clip(rng.standard_normal(50000).astype(np.float32) * np.float32(scale), -448, 448)
            assert np.array_equal(pd.f32_to_e4m3_bits(x), orc.e4m3_encode(x))

    def test_quantize_scale(self):
        x = np.random.default_rng(3).standard_normal((64, 64)).astype(np.float32)
        bits, scale = pd.quantize_e4m3(x)
        obits, oscale = orc.quantize_e4m3(x)
        assert scale == oscale == np.float32(np.abs(x).max() / np.float32(448.0))
        assert np.array_equal(bits, obits)
        assert np.abs(pd.e4m3_bits_to_f32(bits)).max() == 448.0

    def test_fp8_error_budget(self):
        # Quantisation noise alone is ~3-4 % relative Frobenius against unquantised inputs, so
        # the 2 % bound is only meaningful against the oracle built from the same quantised inputs.
        rng = np.random.default_rng(3)
        a = rng.standard_normal((128, 1024)).astype(np.float32)
        b = rng.standard_normal((128, 1024)).astype(np.float32)
        (qa, sa), (qb, sb) = orc.quantize_e4m3(a), orc.quantize_e4m3(b)
        q = orc.decode(orc.gemm(qa, qb, "e4m3", "f32", scale_a=sa, scale_b=sb), "f32")
        rel = orc.rel_frobenius(q, a @ b.T)
        assert 0.02 < rel < 0.06


def test_e5m2_and_int8_conversions_and_oracle():
    """Product-side e5m2 conversion against the oracle's (ml_dtypes when present) on every code
    and on random values; integer oracle against an int64 product."""
    from aster_b200 import dtypes as dt

    codes = np.arange(256, dtype=np.uint8)
    a, b = dt.e5m2_bits_to_f32(codes), orc.e5m2_decode(codes)
    assert np.array_equal(np.isnan(a), np.isnan(b)) and np.array_equal(a[~np.isnan(a)], b[~np.isnan(b)])
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(50000) * rng.choice([1e-6, 1e-3, 1.0, 100.0, 2e4], 50000)).astype(np.float32)
    x = np.concatenate([x, a[np.isfinite(a)], np.float32([0.0, -0.0, 2.0**-16, 2.0**-17, 1.5 * 2.0**-16, 57344.0, 1e9, -1e9])])
    assert np.array_equal(dt.f32_to_e5m2_bits(x), orc.e5m2_encode(x))
    ia = rng.integers(-128, 128, (24, 96), dtype=np.int8)
    ib = rng.integers(-128, 128, (40, 96), dtype=np.int8)
    assert np.array_equal(orc.gemm_i32(ia, ib), (ia.astype(np.int64) @ ib.astype(np.int64).T).astype(np.int32))
    assert np.array_equal(orc.gemm(ia, ib, "i8", "i32"), orc.gemm_i32(ia, ib))
    assert orc.operand_types("e5m2_e4m3") == ("e5m2", "e4m3") and orc.operand_types("bf16") == ("bf16", "bf16")
