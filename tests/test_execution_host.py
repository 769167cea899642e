"""Host-side logic of the execution layer without a GPU: the native calls are replaced by a
recording fake, so the argument protocol of the timed launch loop (which arrays are uploaded,
which are only allocated, when results are copied back, identity-keyed buffers, idempotent
frees) can be checked on any machine.  Mirrors the no-GPU half of the reference's
test/integration/test_execution_core.py (:51-190)."""

import ctypes as C

import numpy as np
import pytest

from aster_b200 import _native as nat
from aster_b200 import execution as ex


class FakeNative:
    """Stands in for ``_native.call``: hands out fake device addresses, keeps 'device memory'
    in host bytearrays, records every call."""

    def __init__(self):
        self.calls = []
        self.mem = {}
        self.next_ptr = 0x10000
        self.clock = 0.0

    def __call__(self, name, *args):
        self.calls.append(name)
        if name == "b200_malloc":
            out, size = args
            out._obj.value = self.next_ptr
            self.mem[self.next_ptr] = bytearray(max(int(size), 1))
            self.next_ptr += 0x10000
        elif name == "b200_free":
            self.mem.pop(args[0].value, None)
        elif name == "b200_memcpy_h2d":
            dst, src, n = args
            self.mem[dst.value][:n] = C.string_at(src.value, n)
        elif name == "b200_memcpy_d2h":
            dst, src, n = args
            C.memmove(dst.value, bytes(self.mem[src.value][:n]), n)
        elif name in ("b200_event_create", "b200_stream_create"):
            args[0]._obj.value = self.next_ptr
            self.next_ptr += 16
        elif name == "b200_event_elapsed_ms":
            self.clock += 0.5
            args[2]._obj.value = self.clock

    def count(self, name):
        return self.calls.count(name)


@pytest.fixture
def fake(monkeypatch):
    f = FakeNative()
    monkeypatch.setattr(nat, "call", f)
    monkeypatch.setattr(nat, "init_current", lambda: f("b200_init", 0) or 0)
    return f


def test_argument_protocol_of_the_timed_loop(fake):
    a = np.arange(8, dtype=np.float32)
    b = np.ones(8, dtype=np.float32)
    c = np.zeros(8, dtype=np.float32)
    raw = np.full(4, 7.0, dtype=np.float32)
    launches, verified = [], []

    def launch(da, db, dc, draw, scalar):
        assert isinstance(da, ex.GpuBuffer) and scalar == 3
        launches.append((da.ptr_value, db.ptr_value, dc.ptr_value, draw.ptr_value))
        # "kernel": c = a + b on the fake device memory
        out = np.frombuffer(bytes(fake.mem[da.ptr_value]), np.float32) + np.frombuffer(bytes(fake.mem[db.ptr_value]), np.float32)
        fake.mem[dc.ptr_value][:] = out.tobytes()

    times = ex.execute_launch(launch, [ex.InputArray(a), ex.InputArray(b), ex.OutputArray(c), raw, 3], num_iterations=3,
                              verify_fn=lambda args: verified.append([type(x).__name__ for x in args]))
    assert len(times) == 3 and all(isinstance(t, int) and t > 0 for t in times)
    assert len(launches) == 3 and len(set(launches)) == 1  # the same buffers every iteration
    assert np.array_equal(c, a + b)
    # inputs and the raw array (= in/out) are uploaded once; the output is not uploaded
    assert fake.count("b200_memcpy_h2d") == 3
    # output and in/out arrays come back once, after iteration 0
    assert fake.count("b200_memcpy_d2h") == 2
    assert verified == [["InputArray", "InputArray", "OutputArray", "InOutArray", "int"]]
    assert fake.count("b200_malloc") == 4 and fake.count("b200_free") == 4 and not fake.mem
    assert fake.calls[0] == "b200_init" and fake.calls[1] == "b200_clear_last_error"


def test_memory_manager_identity_and_errors(fake):
    mm = ex.MemoryManager()
    a = np.arange(4, dtype=np.int32)
    twin = a.copy()
    buf = mm.register(a)
    assert mm.register(a) is buf and mm.get_buffer(a) is buf
    with pytest.raises(KeyError):
        mm.get_buffer(twin)  # equal contents, different object
    with pytest.raises(TypeError):
        mm.register([1, 2, 3])
    no_upload = mm.register(twin, upload=False)
    assert fake.count("b200_memcpy_h2d") == 1 and no_upload is not buf
    mm.release(a)
    with pytest.raises(KeyError):
        mm.release(a)
    mm.release_all()
    mm.release_all()
    assert not fake.mem


def test_buffers_events_streams_are_idempotent(fake):
    buf = ex.GpuBuffer(64)
    with pytest.raises(ValueError):
        buf.copy_from_host(np.zeros(100, np.float32))
    with pytest.raises(TypeError):
        buf.copy_to_host("not an array")
    with pytest.raises(ValueError):
        buf.copy_to_host(np.zeros((4, 8), np.float32)[:, ::2])
    buf.free()
    buf.free()
    e, s = ex.GpuEvent(), ex.GpuStream()
    e.destroy(), e.destroy(), s.destroy(), s.destroy()
    assert fake.count("b200_free") == 1 and fake.count("b200_event_destroy") == 1 and fake.count("b200_stream_destroy") == 1


def test_flush_protocol_runs_before_every_launch(fake):
    order = []

    class Flush:
        def initialize(self):
            order.append("init")

        def flush_llc(self):
            order.append("flush")

        def cleanup(self):
            order.append("cleanup")

    ex.execute_launch(lambda: order.append("launch"), [], num_iterations=2, flush_llc=Flush())
    assert order == ["init", "flush", "launch", "flush", "launch", "cleanup"]


def test_system_has_gpu_is_false_without_a_device(monkeypatch):
    monkeypatch.setattr(nat, "device_count", lambda: 0)
    assert ex.system_has_gpu("sm_100a") is False


def test_execute_hsaco_keeps_the_reference_signature():
    """Parameter names, order and defaults of python/aster/execution/core.py:605-617."""
    import inspect

    from aster_b200.execution import HSACO_KERNELS, execute_hsaco

    params = inspect.signature(execute_hsaco).parameters
    assert list(params) == ["hsaco_path", "kernel_name", "arguments", "grid_dim", "block_dim", "cluster_dim", "num_iterations",
                            "device_id", "flush_llc", "verify_fn", "memory_manager"]
    assert params["grid_dim"].default == (1, 1, 1) and params["block_dim"].default == (64, 1, 1)
    assert params["num_iterations"].default == 1 and params["cluster_dim"].default is None
    # the reference's kernel names: examples 03, 06, 07 and the GEMM generators
    assert {"kernel", "copy_2d_padded", "fused", "gemm_multitile"} <= set(HSACO_KERNELS)
