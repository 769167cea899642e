"""Runtime wrappers on a GPU, following the reference's test/integration/test_execution_core.py
(:196-514): buffer round trips, idempotent frees, events, memory-manager identity semantics."""

import numpy as np
import pytest

from aster_b200 import _native as nat
from aster_b200.execution import (
    FlushL2, GpuBuffer, GpuEvent, GpuStream, InOutArray, InputArray, MemoryManager, OutputArray, execute_launch, system_has_gpu,
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
