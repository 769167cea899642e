"""Worker loops for the harness tests: they speak the protocol of
``aster_b200.bench_workers.persistent_worker_loop`` but never touch a GPU.  Failures are made on
the host: a child that exits, one that kills itself, one that never answers."""

import os
import signal
import time


def _serve(cmd_conn, result_conn, handle):
    while True:
        try:
            item = cmd_conn.recv()
        except EOFError:
            break
        if item is None:
            break
        result_conn.send(handle(item))
    result_conn.close()


def timing_loop(cmd_conn, result_conn, gpu_id, lock_path=None):
    """Times follow from the label: ``..._ns<N>`` gives N ns per launch; ``crash`` exits the
    process, ``kill`` raises SIGKILL on itself, ``hang`` sleeps, ``raise`` reports an error."""
    from aster_b200.bench_workers import gpu_lock

    def handle(item):
        label, num_iter = item[0], item[8]
        if "crash" in label:
            os._exit(7)
        if "kill" in label:
            os.kill(os.getpid(), signal.SIGKILL)
        if "hang" in label:
            time.sleep(120)
        if "raise" in label:
            return label, None, "CUDA error at somewhere.cu:1 - made up"
        ns = int(label.rsplit("_ns", 1)[1]) if "_ns" in label else 1000
        with gpu_lock(lock_path):
            return label, [ns + gpu_id] * num_iter, None

    _serve(cmd_conn, result_conn, handle)


def verify_loop(cmd_conn, result_conn, gpu_id, lock_path=None):
    def handle(item):
        label = item[0]
        if "wrong" in label:
            return label, None, "numeric: max_abs_diff=1.5 mismatched=3"
        if "crash" in label:
            os._exit(9)
        return label, None, None

    _serve(cmd_conn, result_conn, handle)


def lock_probe_loop(cmd_conn, result_conn, gpu_id, lock_path=None):
    """Holds the GPU lock for a moment and reports when it held it."""
    from aster_b200.bench_workers import gpu_lock

    def handle(item):
        with gpu_lock(lock_path):
            t0 = time.monotonic()
            time.sleep(0.15)
            t1 = time.monotonic()
        return item[0], [int(t0 * 1e9), int(t1 * 1e9)], None

    _serve(cmd_conn, result_conn, handle)
