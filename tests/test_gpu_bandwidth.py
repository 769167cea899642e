"""Bit-exact parity of the bandwidth kernels on a B200 against the CPU oracle, at the
reference's own shapes and at sizes that exercise every tail path."""

import numpy as np
import pytest

from aster_b200 import bandwidth as bw
from oracle import gemm_oracle as orc

pytestmark = pytest.mark.gpu


class TestVectorAdd:
    def test_reference_case(self, gpu):
        # examples/03_vector_add/run.py:44-53
        a, b = np.arange(64, dtype=np.int32), np.full(64, 100, dtype=np.int32)
        assert np.array_equal(bw.vector_add(a, b), orc.vector_add(a, b))

    @pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 4096, 4096 * 4 + 1, (1 << 22) + 3, 1 << 24])
    def test_sizes_int32(self, gpu, n):
        rng = np.random.default_rng(5)
        a = rng.integers(-2**30, 2**30, n, dtype=np.int64).astype(np.int32)
        b = rng.integers(-2**30, 2**30, n, dtype=np.int64).astype(np.int32)
        assert np.array_equal(bw.vector_add(a, b), orc.vector_add(a, b))

    def test_wraparound(self, gpu):
        a = np.full(1000, 2**31 - 1, dtype=np.int32)
        b = np.arange(1000, dtype=np.int32)
        assert np.array_equal(bw.vector_add(a, b), orc.vector_add(a, b))

    @pytest.mark.parametrize("n", [7, 100000, (1 << 20) + 1])
    def test_float32(self, gpu, n):
        rng = np.random.default_rng(5)
        a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        assert np.array_equal(bw.vector_add(a, b), orc.vector_add(a, b))

    def test_unaligned_device_pointers(self, gpu):
        from aster_b200 import _native as nat
        from aster_b200.execution import GpuBuffer
        import ctypes as C

        n = 10001
        rng = np.random.default_rng(6)
        a = rng.integers(-1000, 1000, n + 1).astype(np.int32)
        b = rng.integers(-1000, 1000, n + 1).astype(np.int32)
        da, db, dc = GpuBuffer(a.nbytes), GpuBuffer(b.nbytes), GpuBuffer(a.nbytes)
        da.copy_from_host(a), db.copy_from_host(b), dc.zero()
        nat.call("b200_vector_add_i32", C.c_void_p(da.ptr_value + 4), C.c_void_p(db.ptr_value + 4), C.c_void_p(dc.ptr_value + 4), n, None)
        out = np.empty(n + 1, np.int32)
        dc.copy_to_host(out)
        assert out[0] == 0 and np.array_equal(out[1:], a[1:] + b[1:])
        for buf in (da, db, dc):
            buf.free()


class TestCopy2dPadded:
    @pytest.mark.parametrize("depth", [1, 2, 4])
    def test_reference_case(self, gpu, depth):
        # python/test/test_copy_examples.py:21-23: 64 x 300, depth in {1, 2, 4}, 8 workgroups
        src = np.arange(64 * 300, dtype=np.float32).reshape(64, 300)
        assert np.array_equal(bw.copy_2d_padded(src, depth=depth, num_ctas=8), src)

    @pytest.mark.parametrize("shape", [(1, 4), (3, 1024), (7, 1028), (64, 300), (257, 2052), (5, 16380), (1024, 4096), (0, 8), (8, 0)])
    @pytest.mark.parametrize("depth", [1, 3, 8])
    def test_shapes(self, gpu, shape, depth):
        src = np.random.default_rng(6).standard_normal(shape).astype(np.float32)
        assert np.array_equal(bw.copy_2d_padded(src, depth=depth), src)

    def test_sentinel_outside_stays(self, gpu):
        # A 60 x 300 copy into the top of a 64 x 300 sentinel-filled destination.
        from aster_b200.execution import GpuBuffer
        from aster_b200 import _native as nat

        src = np.arange(60 * 300, dtype=np.float32).reshape(60, 300)
        dst = np.full((64, 300), bw.SENTINEL, np.float32)
        ds, dd = GpuBuffer(src.nbytes), GpuBuffer(dst.nbytes)
        ds.copy_from_host(src), dd.copy_from_host(dst)
        nat.call("b200_copy_2d_padded_f32", ds.ptr, dd.ptr, 60, 300, 2, 0, None)
        dd.copy_to_host(dst)
        assert np.array_equal(dst, orc.copy_2d_padded(src, np.full((64, 300), bw.SENTINEL, np.float32)))
        ds.free(), dd.free()

    def test_rejects_bad_n(self, gpu):
        with pytest.raises(ValueError):
            bw.copy_2d_padded(np.zeros((4, 6), np.float32))


class TestAddRelu:
    def test_reference_case(self, gpu):
        # examples/07_simple_fusion/simple_fusion.py:133-144
        a = np.array([1.0, -2.0, 3.0, -4.0], np.float32)
        b = np.array([-0.5, 1.0, -4.0, 5.0], np.float32)
        np.testing.assert_allclose(bw.add_relu(a, b), orc.add_relu(a, b), atol=1e-5)

    @pytest.mark.parametrize("n", [1, 4, 1000, 1 << 20])
    def test_bit_exact(self, gpu, n):
        rng = np.random.default_rng(7)
        a, b = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        assert np.array_equal(bw.add_relu(a, b), orc.add_relu(a, b))
