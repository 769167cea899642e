"""Runtime wrappers on a GPU, following the reference's test/integration/test_execution_core.py
(:196-514): buffer round trips, idempotent frees, events, memory-manager identity semantics."""

import numpy as np
import pytest

from aster_b200 import _native as nat
from aster_b200.execution import (
    FlushL2, GpuBuffer, GpuEvent, GpuStream, InOutArray, InputArray, MemoryManager, OutputArray, execute_hsaco, execute_launch,
    system_has_gpu,
)
from aster_b200 import bandwidth as bw

pytestmark = pytest.mark.gpu


def test_system_has_gpu(gpu):
    assert system_has_gpu("sm_100a")
    assert nat.device_count() >= 1
    assert gpu.sm_count >= 100 and gpu.max_smem_per_block_optin >= 227 * 1024 and gpu.l2_bytes > 0


def test_buffer_roundtrip_and_idempotent_free(gpu):
    a = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    buf = GpuBuffer(a.nbytes)
    assert buf.size_bytes == a.nbytes and buf.ptr_value != 0
    buf.copy_from_host(a)
    out = np.zeros_like(a)
    buf.copy_to_host(out)
    assert np.array_equal(a, out)
    with pytest.raises(ValueError):
        buf.copy_from_host(np.zeros(2000, np.float32))
    with pytest.raises(TypeError):
        buf.copy_from_host([1, 2, 3])
    buf.free()
    buf.free()


def test_events_and_streams(gpu):
    e0, e1, s = GpuEvent(), GpuEvent(), GpuStream()
    e0.record()
    e1.record()
    e1.synchronize()
    assert e1.elapsed_ms(e0) >= 0.0 and isinstance(e1.elapsed_ns(e0), int)
    s.synchronize()
    for obj in (e0, e1, s):
        obj.destroy()
        obj.destroy()


def test_memory_manager_identity(gpu):
    mm = MemoryManager()
    a = np.arange(16, dtype=np.float32)
    buf = mm.register(a)
    assert mm.register(a) is buf and mm.get_buffer(a) is buf
    a[:] = 7
    mm.sync_to_gpu(a)
    a[:] = 0
    mm.sync_from_gpu(a)
    assert (a == 7).all()
    with pytest.raises(KeyError):
        mm.get_buffer(np.arange(16, dtype=np.float32))
    with pytest.raises(TypeError):
        mm.register([1, 2])
    mm.release(a)
    with pytest.raises(KeyError):
        mm.release(a)
    mm.release_all()


def test_execute_launch_argument_protocol(gpu):
    n = 4096
    a = np.arange(n, dtype=np.int32)
    b = np.full(n, 100, dtype=np.int32)
    c = np.zeros(n, dtype=np.int32)
    seen = []

    def launch(da, db, dc, count):
        bw.vector_add_device(da, db, dc, count)

    times = execute_launch(launch, [InputArray(a), InputArray(b), OutputArray(c), n], num_iterations=5,
                           flush_llc=FlushL2(), verify_fn=lambda args: seen.append(len(args)))
    assert len(times) == 5 and all(t > 0 for t in times) and seen == [4]
    assert np.array_equal(c, a + b)
    # raw ndarray = in/out
    x = np.arange(8, dtype=np.float32)
    y = np.ones(8, dtype=np.float32)
    execute_launch(lambda dx, dy, dz: bw.add_relu_device(dx, dy, dx, 8), [x, InputArray(y), InOutArray(np.zeros(1, np.float32))])
    assert np.array_equal(x, np.arange(8) + 1.0)


def test_error_paths_leave_the_context_usable(gpu):
    with pytest.raises(nat.B200Error) as e:
        nat.call("b200_set_device", 4096)
    assert e.value.status == nat.ERR_CUDA and "CUDA error at" in e.value.message
    nat.call("b200_clear_last_error")
    assert nat.last_error() == ""
    assert np.array_equal(bw.vector_add(np.arange(4, dtype=np.int32), np.arange(4, dtype=np.int32)), 2 * np.arange(4))
    before = nat.launch_count()
    bw.add_relu(np.ones(4, np.float32), np.ones(4, np.float32))
    assert nat.launch_count() == before + 1


def test_execute_hsaco_runs_the_example_kernels(gpu, tmp_path):
    """The three example kernels through the reference's entry point, called the way the
    reference's examples runner calls it (examples/_gpu_runner.py:35-41): inputs wrapped as
    InputArray, outputs as OutputArray, kernel chosen by name, grid and block passed along."""
    # examples/03_vector_add/run.py:44-53
    a, b, c = np.arange(64, dtype=np.int32), np.full(64, 100, dtype=np.int32), np.zeros(64, dtype=np.int32)
    times = execute_hsaco(hsaco_path=str(tmp_path / "vector_add.hsaco"), kernel_name="kernel",
                          arguments=[InputArray(a), InputArray(b), OutputArray(c)], grid_dim=(1, 1, 1), block_dim=(64, 1, 1))
    assert np.array_equal(c, a + b) and len(times) == 1 and times[0] > 0
    # examples/06_copy_layout/copy_2d_padded.py:131-143, depths as python/test/test_copy_examples.py:21-23
    for depth in (1, 2, 4):
        (tmp_path / "copy.json").write_text('{"depth": %d}' % depth)
        src = np.arange(64 * 300, dtype=np.float32).reshape(64, 300)
        dst = np.full_like(src, -999.0)
        execute_hsaco(str(tmp_path / "copy.json"), "copy_2d_padded", [InputArray(src), OutputArray(dst)], grid_dim=(304, 1, 1), block_dim=(64, 1, 1))
        assert np.array_equal(src, dst)
    # examples/07_simple_fusion/simple_fusion.py:133-144
    rng = np.random.default_rng(7)
    x, y, out = rng.standard_normal(4).astype(np.float32), rng.standard_normal(4).astype(np.float32), np.zeros(4, np.float32)
    seen = []
    times = execute_hsaco(None, "fused", [InputArray(x), InputArray(y), OutputArray(out)], grid_dim=(1, 1, 1), block_dim=(1, 1, 1),
                          num_iterations=3, flush_llc=FlushL2(), verify_fn=lambda args: seen.append(len(args)))
    assert np.allclose(out, np.maximum(x + y, 0.0), atol=1e-5) and len(times) == 3 and seen == [3]
    with pytest.raises(RuntimeError, match="no kernel named"):
        execute_hsaco(None, "does_not_exist", [])


def test_execute_hsaco_runs_a_compiled_gemm(gpu, tmp_path):
    from aster_b200.gemm_config import make_b200_instance
    from aster_b200.multitile_gemm import compile_multitile_gemm
    from oracle import gemm_oracle as orc

    cfg = make_b200_instance(256, 384, 512)  # f16 in, f32 out, as the reference's generators
    path, _ = compile_multitile_gemm(cfg, str(tmp_path / "gemm.b200plan.json"))
    inp = orc.make_inputs(256, 384, 512, "f16", "normal", 0)
    C = np.zeros(256 * 384, dtype=np.float32)
    # the call of execute_multitile_hsaco (test_102_gemm_python_multitile_lds_cdna3.py:424-434)
    times = execute_hsaco(hsaco_path=path, kernel_name=cfg.kernel_name,
                          arguments=[InputArray(inp["A"].flatten()), InputArray(inp["B"].flatten()), OutputArray(C)],
                          grid_dim=(cfg.num_workgroups, 1, 1), block_dim=(cfg.num_threads, 1, 1), num_iterations=3)
    assert len(times) == 3
    want = orc.gemm_f32(inp["A"], inp["B"], "f16")
    assert float(np.max(np.abs(C.reshape(256, 384) - want))) <= orc.abs_bound(inp["A"], inp["B"], "f16")
    orc.assert_reference_close(C.reshape(256, 384), want)


def test_gpu_runner_protocol(gpu, tmp_path):
    """The child process of the reference's examples (arrays in .npy files, one JSON argument)."""
    from aster_b200 import gpu_runner

    a, b, c = np.arange(64, dtype=np.int32), np.full(64, 100, dtype=np.int32), np.zeros(64, dtype=np.int32)
    files = {}
    for name, arr in (("a", a), ("b", b), ("c", c)):
        files[name] = str(tmp_path / f"{name}.npy")
        np.save(files[name], arr)
    out = gpu_runner.run({"hsaco_path": "unused.hsaco", "kernel_name": "kernel", "grid": [1, 1, 1], "block": [64, 1, 1],
                          "input_files": [files["a"], files["b"]], "output_files": [files["c"]]})
    assert len(out["times"]) == 1 and np.array_equal(np.load(files["c"]), a + b)


def test_weak_scaled_family_compile_and_execute(gpu, tmp_path):
    """compile_gemm + execute_gemm_hsaco (test_perf_001_gemm_fp16_weak_scaled.py:181-272) on a plain
    WeakScaledMappedGemmInstance, checked the way that file checks (:358): numpy, rtol = atol = 1e-2."""
    from aster_b200.gemm_config import GemmMappingSpec, GemmSpec, WeakScaledMappedGemmInstance
    from aster_b200.multitile_gemm import compile_gemm, execute_gemm_hsaco

    cfg = WeakScaledMappedGemmInstance(GemmSpec.from_sizes(256, 256, 128), GemmMappingSpec([2, 2, 1], [2, 2, 1], [4, 4, 1]))
    path, _ = compile_gemm(cfg, str(tmp_path / "w.b200plan.json"))
    np.random.seed(42)
    A = (np.random.randn(256, 128) * 0.1).astype(np.float16)
    B = (np.random.randn(256, 128) * 0.1).astype(np.float16)
    C, times = execute_gemm_hsaco(cfg, path, 2, A, B)
    assert len(times) == 2
    np.testing.assert_allclose(C.reshape(256, 256), A.astype(np.float32) @ B.astype(np.float32).T, rtol=1e-2, atol=1e-2)
