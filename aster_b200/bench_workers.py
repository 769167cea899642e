"""Process model of the bench harness: one persistent worker process per GPU, crash isolation,
per-GPU exclusivity across processes, verification on all GPUs, the pipelined compile + execute
sweep and its command-line arguments.

Follows contrib/kittens/test/bench/bench_harness.py of the reference: visible-device handling
and the per-physical-GPU lock file (:305-355), the persistent worker loops (:707-859), the
worker wrapper that respawns its child after a crash or a timeout (:866-968), the per-GPU queue
thread (:971-996), ``run_on_gpus`` (:999-1105), ``verify_on_gpus`` (:1121-1194),
``bench_perf_sweep_pipelined`` (:1271-1501) and the CLI builders (:1856-1965).  The work item is
the reference's tuple ``(label, artifact_path, kernel_name, num_workgroups, num_threads, m, n, k,
num_iterations, direct_b, direct_a, init_mode)``; a result is ``(label, times_ns or None,
error or None)``.

A GPU is never reset or otherwise touched from here when a worker dies: the child is killed,
its context goes with it, and a fresh child starts for the next item.  The lock is the
reference's own file (``<tmp>/aster-gpu-locks/gpu_<physical id>.lock``), so harnesses of both
kinds sharing a host take turns on a device.
"""

from __future__ import annotations

import argparse
import contextlib
import fcntl
import json
import os
import queue
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from typing import Callable, Optional

import numpy as np

from .bench_harness import (
    INIT_DEFAULT, NUM_ITERATIONS, WARMUP_ITERATIONS, InitMode, _compute_stats, emit_one_result, make_inputs, peak_tflops,
    verify_against_numpy,
)

DEFAULT_COMPILE_WORKERS = 4
DEFAULT_COMPILE_TIMEOUT = 60
DEFAULT_EXEC_TIMEOUT = 120
DEFAULT_VERIFY_TIMEOUT = 180


# ---------------------------------------------------------------------------------------------
# devices and locks
# ---------------------------------------------------------------------------------------------
def visible_device_ids(environ=None) -> Optional[list]:
    """The GPUs the operator allotted to this process, as physical ids, from
    ``CUDA_VISIBLE_DEVICES`` (a comma list of integers); ``None`` when it is unset or empty."""
    environ = os.environ if environ is None else environ
    v = environ.get("CUDA_VISIBLE_DEVICES")
    if v is None or v.strip() == "":
        return None
    ids = []
    for part in v.split(","):
        part = part.strip()
        if part.lstrip("-").isdigit():
            ids.append(int(part))
    return ids or None


# Captured at import, before any child's initialiser narrows the variable for its own process.
_VISIBLE_GPU_IDS = visible_device_ids()


def physical_gpu_id(gpu_id: int, visible: Optional[list] = None) -> int:
    """Dense worker index -> physical device id, through the allotted set."""
    visible = _VISIBLE_GPU_IDS if visible is None else visible
    return visible[gpu_id % len(visible)] if visible else gpu_id


def detect_num_gpus(mcpu: str = "sm_100a") -> int:
    """Number of usable GPUs of architecture ``mcpu`` (0 when there is none), never more than
    the operator allotted."""
    try:
        from . import _native as nat
        from .execution import system_has_gpu

        if not system_has_gpu(mcpu):
            return 0
        n = nat.device_count()
        if _VISIBLE_GPU_IDS is not None:
            n = min(n, len(_VISIBLE_GPU_IDS))
        return max(1, n)
    except Exception:
        return 0


GPU_LOCK_DIR = os.path.join(tempfile.gettempdir(), "aster-gpu-locks")


def gpu_lock_path(gpu_id: int, lock_dir: Optional[str] = None, visible: Optional[list] = None) -> str:
    """The lock file of the PHYSICAL GPU behind worker index ``gpu_id``: stable across runs,
    phases and processes."""
    lock_dir = lock_dir or GPU_LOCK_DIR
    os.makedirs(lock_dir, exist_ok=True)
    return os.path.join(lock_dir, f"gpu_{physical_gpu_id(gpu_id, visible)}.lock")


@contextlib.contextmanager
def gpu_lock(path: Optional[str]):
    """Exclusive ``flock`` on ``path`` for the duration (no-op for ``None``).  The kernel drops
    the lock when the holder dies, so a crashed worker cannot leave a GPU locked."""
    if not path:
        yield
        return
    fd = os.open(path, os.O_WRONLY | os.O_CREAT, 0o644)
    try:
        fcntl.flock(fd, fcntl.LOCK_EX)
        yield
    finally:
        try:
            fcntl.flock(fd, fcntl.LOCK_UN)
        finally:
            os.close(fd)


def gpu_init(gpu_id: int, quiet: bool = True) -> None:
    """Initialiser of a worker process: pin it to its physical GPU through
    ``CUDA_VISIBLE_DEVICES`` (before the CUDA runtime loads) and silence its stdout / stderr;
    errors travel back as results, not as text."""
    import io

    os.environ["CUDA_VISIBLE_DEVICES"] = str(physical_gpu_id(gpu_id))
    if quiet:
        devnull = os.open(os.devnull, os.O_WRONLY)
        os.dup2(devnull, 1)
        os.dup2(devnull, 2)
        os.close(devnull)
        sys.stdout = io.StringIO()
        sys.stderr = io.StringIO()


def work_item(cfg, artifact_path: str, num_iterations: int, init_mode=INIT_DEFAULT) -> tuple:
    m, n, k = cfg.gemm_size
    return (cfg.label, artifact_path, cfg.kernel_name, cfg.num_workgroups, cfg.num_threads, m, n, k, num_iterations,
            bool(getattr(cfg.mapping, "direct_b", False)), False, InitMode(init_mode).value)


def _first_line(e: BaseException) -> str:
    text = str(e).split("\n")[0][:200]
    return text or type(e).__name__


def _config_of(label: str, direct_b: bool):
    from .multitile_gemm import BENCH_HOOKS, BENCH_HOOKS_DIRECT_B

    hooks = BENCH_HOOKS_DIRECT_B if direct_b else BENCH_HOOKS
    return hooks["from_label"](label)


# ---------------------------------------------------------------------------------------------
# worker loops (run in the child process)
# ---------------------------------------------------------------------------------------------
def persistent_worker_loop(cmd_conn, result_conn, gpu_id: int, lock_path: Optional[str] = None) -> None:
    """Long-lived child: initialise the device once, then time one config per work item until a
    ``None`` arrives.  Host operands are kept while the problem (sizes, element type, init mode)
    stays the same; the per-GPU lock is held only across the launches."""
    gpu_init(gpu_id)
    from .multitile_gemm import execute_multitile_hsaco

    cached_key, cached_inputs = None, None
    while True:
        try:
            item = cmd_conn.recv()
        except EOFError:
            break
        if item is None:
            break
        label, path, _kernel, _wg, _threads, m, n, k, num_iter, *extra = item
        direct_b = bool(extra[0]) if extra else False
        init_mode = extra[2] if len(extra) > 2 else INIT_DEFAULT
        try:
            cfg = _config_of(label, direct_b)
            key = (m, n, k, cfg.dtype_ab, str(init_mode))
            if key != cached_key:
                cached_inputs, cached_key = make_inputs(cfg, init_mode=init_mode), key
            inputs = cached_inputs
            kw = dict(scale_a=inputs[2], scale_b=inputs[3]) if len(inputs) == 4 else {}
            with gpu_lock(lock_path):
                _, times = execute_multitile_hsaco(cfg, path, num_iter, inputs[0], inputs[1], skip_gpu_check=True, **kw)
            result_conn.send((label, [int(t) for t in times], None))
        except Exception as e:  # reported, and the loop goes on with the next item
            result_conn.send((label, None, _first_line(e)))
    result_conn.close()


def persistent_verify_loop(cmd_conn, result_conn, gpu_id: int, lock_path: Optional[str] = None) -> None:
    """Long-lived child for correctness: one launch per item, compared with numpy
    (``A.f32 @ B.f32.T``, rtol = atol = 1e-2).  Same protocol; a result's error is ``None``
    (passed), ``"numeric: ..."`` or the first line of an exception."""
    gpu_init(gpu_id)
    from .multitile_gemm import execute_multitile_hsaco

    while True:
        try:
            item = cmd_conn.recv()
        except EOFError:
            break
        if item is None:
            break
        label, path, _kernel, _wg, _threads, m, n, k, *extra = item
        direct_b = bool(extra[0]) if extra else False
        init_mode = extra[2] if len(extra) > 2 else INIT_DEFAULT
        try:
            cfg = _config_of(label, direct_b)
            inputs = make_inputs(cfg, init_mode=init_mode)
            kw = dict(scale_a=inputs[2], scale_b=inputs[3]) if len(inputs) == 4 else {}
            with gpu_lock(lock_path):
                C, _ = execute_multitile_hsaco(cfg, path, 1, inputs[0], inputs[1], skip_gpu_check=True, **kw)
            why = verify_against_numpy(cfg, C, inputs[0], inputs[1]) if len(inputs) == 2 else None
            result_conn.send((label, None, None if why is None else f"numeric: {why}"))
        except Exception as e:
            result_conn.send((label, None, _first_line(e)))
    result_conn.close()


# ---------------------------------------------------------------------------------------------
# parent side
# ---------------------------------------------------------------------------------------------
class PersistentGpuWorker:
    """A long-lived child process on one GPU, respawned after a crash or a timeout.

    ``execute(item, timeout)`` sends one work item and returns its result; when the child dies
    the result is ``(label, None, "worker crash (signal N)")``, when it does not answer within
    ``timeout`` seconds it is killed and the result says so.  Either way the next ``execute``
    starts a fresh child.  ``loop_fn(cmd_conn, result_conn, gpu_id, lock_path)`` is what the
    child runs (a module-level function: the child is spawned, not forked).
    """

    def __init__(self, gpu_id: int, loop_fn: Optional[Callable] = None, lock_path: Optional[str] = None) -> None:
        self.gpu_id = gpu_id
        self._loop_fn = loop_fn or persistent_worker_loop
        self._lock_path = lock_path
        self._proc = None
        self._cmd = None  # parent -> child
        self._res = None  # child -> parent
        self.spawns = 0

    def _spawn(self) -> None:
        import multiprocessing as mp

        ctx = mp.get_context("spawn")
        cmd_reader, cmd_writer = ctx.Pipe(duplex=False)
        res_reader, res_writer = ctx.Pipe(duplex=False)
        p = ctx.Process(target=self._loop_fn, args=(cmd_reader, res_writer, self.gpu_id, self._lock_path), daemon=True)
        p.start()
        cmd_reader.close()  # the parent keeps only its own ends
        res_writer.close()
        self._proc, self._cmd, self._res = p, cmd_writer, res_reader
        self.spawns += 1

    def ensure_alive(self) -> None:
        if self._proc is None or not self._proc.is_alive():
            if self._proc is not None:
                self._cleanup()
            self._spawn()

    def execute(self, item: tuple, timeout: float = DEFAULT_EXEC_TIMEOUT) -> tuple:
        label = item[0]
        self.ensure_alive()
        try:
            self._cmd.send(item)
        except (BrokenPipeError, OSError):
            return self._crashed(label)
        if not self._res.poll(timeout):
            if self._proc.is_alive():
                self._proc.kill()
                self._proc.join(timeout=10)
                self._cleanup()
                return label, None, f"execution timed out after {timeout:g}s"
            return self._crashed(label)
        try:
            return self._res.recv()
        except (EOFError, ConnectionResetError, OSError):
            return self._crashed(label)

    def _crashed(self, label) -> tuple:
        self._proc.join(timeout=10)
        code = self._proc.exitcode
        self._cleanup()
        kind = "signal" if code is not None and code < 0 else "exit"
        return label, None, f"worker crash ({kind} {-code if code is not None and code < 0 else code})"

    def shutdown(self) -> None:
        if self._proc is not None and self._proc.is_alive():
            try:
                self._cmd.send(None)
                self._proc.join(timeout=5)
            except (BrokenPipeError, OSError):
                pass
            if self._proc.is_alive():
                self._proc.kill()
                self._proc.join(timeout=10)
        self._cleanup()

    def _cleanup(self) -> None:
        for c in (self._cmd, self._res):
            if c is not None:
                try:
                    c.close()
                except OSError:
                    pass
        self._proc = self._cmd = self._res = None


def run_gpu_queue(gpu_id: int, items, result_queue, timeout: float = DEFAULT_EXEC_TIMEOUT, lock_path: Optional[str] = None,
                  loop_fn: Optional[Callable] = None) -> None:
    """Work through ``items`` on one GPU with one persistent worker.  ``items`` is a list, or a
    ``queue.Queue`` fed while this runs (``None`` ends it).  Every result goes to
    ``result_queue`` as it completes; a crashed or hung item is reported as failed and the next
    one proceeds in a fresh child."""
    worker = PersistentGpuWorker(gpu_id, loop_fn=loop_fn, lock_path=lock_path)
    try:
        if isinstance(items, queue.Queue):
            while True:
                item = items.get()
                if item is None:
                    break
                result_queue.put(worker.execute(item, timeout=timeout))
        else:
            for item in items:
                result_queue.put(worker.execute(item, timeout=timeout))
    finally:
        worker.shutdown()


def _collect(result_q, threads, total: int, on_result: Callable) -> int:
    collected = 0
    try:
        while collected < total:
            try:
                res = result_q.get(timeout=0.5)
            except queue.Empty:
                if not any(t.is_alive() for t in threads) and result_q.empty():
                    break
                continue
            collected += 1
            on_result(res)
    except KeyboardInterrupt:
        print(f"\nCtrl+C -- stopping ({collected}/{total} done), keeping what was measured", file=sys.stderr)
    for t in threads:
        t.join(timeout=5.0)
    return collected


def _stats_of(cfg, times):
    return _compute_stats(times[WARMUP_ITERATIONS:], cfg.total_flops, peak_tflops(cfg.mapping.mcpu, getattr(cfg, "dtype_ab", "f16")))


def run_on_gpus(configs, artifact_paths: dict, num_iterations: int, num_gpus: int, *, bench: str = "unknown", results_file: Optional[str] = None,
                init_mode=INIT_DEFAULT, timeout: float = DEFAULT_EXEC_TIMEOUT, loop_fn: Optional[Callable] = None, use_locks: bool = True,
                lock_dir: Optional[str] = None):
    """Time the compiled configs, all GPUs at once, round-robin: one thread and one persistent
    worker per GPU.  Returns ``(results, failed)``: ``[(cfg, PerfStats)]`` and ``[(cfg, reason)]``."""
    per_gpu = [[] for _ in range(max(1, num_gpus))]
    by_label = {}
    for i, cfg in enumerate(c for c in configs if c.label in artifact_paths):
        per_gpu[i % len(per_gpu)].append(work_item(cfg, artifact_paths[cfg.label], num_iterations, init_mode))
        by_label[cfg.label] = cfg
    total = sum(len(g) for g in per_gpu)
    results, failed = [], []
    result_q: queue.Queue = queue.Queue()
    threads = []
    for gpu_id, items in enumerate(per_gpu):
        if not items:
            continue
        lock = gpu_lock_path(gpu_id, lock_dir) if use_locks else None
        t = threading.Thread(target=run_gpu_queue, args=(gpu_id, items, result_q), kwargs=dict(timeout=timeout, lock_path=lock, loop_fn=loop_fn),
                             daemon=True)
        t.start()
        threads.append(t)
    stream = open(results_file, "a") if results_file else None

    def on_result(res):
        label, times, err = res
        cfg = by_label.get(label)
        if cfg is None:
            return
        if err or times is None:
            failed.append((cfg, err or "unknown"))
            return
        stats = _stats_of(cfg, times)
        if stats is None:
            failed.append((cfg, "no valid measurements"))
            return
        results.append((cfg, stats))
        emit_one_result(stream, bench, cfg, stats)

    try:
        _collect(result_q, threads, total, on_result)
    finally:
        if stream is not None:
            stream.close()
    return results, failed


def verify_on_gpus(configs, artifact_paths: dict, num_gpus: int, init_mode=INIT_DEFAULT, *, timeout: float = DEFAULT_VERIFY_TIMEOUT,
                   loop_fn: Optional[Callable] = None, use_locks: bool = True, lock_dir: Optional[str] = None):
    """Check the compiled configs against numpy on all GPUs at once.  ``init_mode`` must be the
    one the timing run used.  Returns ``(number passed, ["label: reason", ...])``."""
    per_gpu = [[] for _ in range(max(1, num_gpus))]
    idx = 0
    for cfg in configs:
        if cfg.label not in artifact_paths:
            continue
        item = work_item(cfg, artifact_paths[cfg.label], 1, init_mode)
        per_gpu[idx % len(per_gpu)].append(item[:8] + item[9:])  # the verify item carries no iteration count
        idx += 1
    total = sum(len(g) for g in per_gpu)
    state = {"passed": 0}
    errors = []
    result_q: queue.Queue = queue.Queue()
    threads = []
    for gpu_id, items in enumerate(per_gpu):
        if not items:
            continue
        lock = gpu_lock_path(gpu_id, lock_dir) if use_locks else None
        t = threading.Thread(target=run_gpu_queue, args=(gpu_id, items, result_q),
                             kwargs=dict(timeout=timeout, lock_path=lock, loop_fn=loop_fn or persistent_verify_loop), daemon=True)
        t.start()
        threads.append(t)

    def on_result(res):
        label, _, err = res
        if err:
            errors.append(f"{label}: {err}")
        else:
            state["passed"] += 1

    _collect(result_q, threads, total, on_result)
    return state["passed"], errors


def verify_top_configs(results, artifact_paths: dict, *, top_n: int, num_gpus: int, init_mode=INIT_DEFAULT, **kw) -> set:
    """Verify the ``top_n`` fastest of ``results`` (``[(cfg, stats)]``, fastest first); returns
    the labels that passed (the role of ``verify_top_configs``, bench_search.py:499-560)."""
    top = [cfg for cfg, _ in results[:top_n]]
    _, errors = verify_on_gpus(top, artifact_paths, num_gpus, init_mode, **kw)
    bad = {e.split(": ", 1)[0] for e in errors}
    return {cfg.label for cfg in top if cfg.label in artifact_paths and cfg.label not in bad}


def compile_one(cfg, artifact_dir: str, compile_fn: Callable):
    """Compile one config into ``artifact_dir`` (reusing an artifact of the same label that is
    already there).  Returns ``(label, path, resources)``."""
    path = os.path.join(artifact_dir, f"{cfg.label}.b200plan.json")
    if os.path.isfile(path):
        with open(path) as f:
            return cfg.label, path, json.load(f).get("resources")
    _, text = compile_fn(cfg, path)
    return cfg.label, path, json.loads(text).get("resources")


def bench_perf_sweep_pipelined(configs, compile_fn: Callable, repro_cmd_fn: Optional[Callable] = None, *, mcpu: str = "sm_100a", bench: str = "unknown",
                               num_gpus: Optional[int] = None, compile_workers: Optional[int] = None, post_compile_filter: Optional[Callable] = None,
                               init_mode=INIT_DEFAULT, iterations: Optional[int] = None, hsaco_dir: Optional[str] = None,
                               results_file: Optional[str] = None, exec_timeout: float = DEFAULT_EXEC_TIMEOUT, loop_fn: Optional[Callable] = None,
                               use_locks: bool = True, lock_dir: Optional[str] = None, log=print):
    """Compile and execute in a pipeline: a config goes to a GPU's queue the moment its artifact
    exists and passes ``post_compile_filter(cfg, resources) -> None | reason``.  One persistent
    worker per GPU, per-physical-GPU lock around the launches.  Returns ``(results,
    artifact_paths)`` with ``results = [(cfg, PerfStats)]`` fastest first; compile and execution
    failures are logged with ``repro_cmd_fn(cfg)``.  ``num_gpus=0`` compiles only."""
    iterations = NUM_ITERATIONS if iterations is None else iterations
    num_gpus = detect_num_gpus(mcpu) if num_gpus is None else num_gpus
    compile_workers = compile_workers or DEFAULT_COMPILE_WORKERS
    active = list(configs)
    by_label = {c.label: c for c in active}
    artifact_dir = hsaco_dir or tempfile.mkdtemp(prefix="bench_b200plan_")
    os.makedirs(artifact_dir, exist_ok=True)
    log(f"Pipelined sweep: {len(active)} configs, {compile_workers} compile + {num_gpus} exec workers, init={InitMode(init_mode).value}")

    result_q: queue.Queue = queue.Queue()
    work_queues, threads = [], []
    for gpu_id in range(num_gpus):
        wq: queue.Queue = queue.Queue()
        lock = gpu_lock_path(gpu_id, lock_dir) if use_locks else None
        t = threading.Thread(target=run_gpu_queue, args=(gpu_id, wq, result_q), kwargs=dict(timeout=exec_timeout, lock_path=lock, loop_fn=loop_fn),
                             daemon=True)
        t.start()
        work_queues.append(wq)
        threads.append(t)

    artifact_paths, compile_failed, exec_failed, results = {}, [], [], []
    stream = open(results_file, "a") if results_file else None
    submitted = 0

    def drain(block_s: float = 0.0) -> None:
        while True:
            try:
                label, times, err = result_q.get(timeout=block_s) if block_s else result_q.get_nowait()
            except queue.Empty:
                return
            cfg = by_label.get(label)
            if cfg is None:
                continue
            if err or times is None:
                exec_failed.append((cfg, err or "unknown"))
                continue
            stats = _stats_of(cfg, times)
            if stats is None:
                exec_failed.append((cfg, "no valid measurements"))
            else:
                results.append((cfg, stats))
                emit_one_result(stream, bench, cfg, stats)

    try:
        with ThreadPoolExecutor(max_workers=compile_workers) as pool:
            futs = {pool.submit(compile_one, c, artifact_dir, compile_fn): c for c in active}
            try:
                for rr, fut in enumerate(as_completed(futs)):
                    cfg = futs[fut]
                    try:
                        label, path, res = fut.result()
                        artifact_paths[label] = path
                        reason = None
                        if post_compile_filter is not None:
                            reason = "metadata missing" if not res else post_compile_filter(cfg, res)
                        if reason:
                            compile_failed.append((cfg, f"compile: {reason.split(' -- ', 1)[0]}"))
                        elif work_queues:
                            work_queues[submitted % len(work_queues)].put(work_item(cfg, path, iterations, init_mode))
                            submitted += 1
                    except Exception as e:
                        compile_failed.append((cfg, f"compile: {_first_line(e)}"))
                    drain()
            except KeyboardInterrupt:
                log("Ctrl+C -- cancelling pending compilations, draining what is in flight")
                for f in futs:
                    f.cancel()
        for wq in work_queues:
            wq.put(None)
        deadline = time.monotonic() + (exec_timeout + 30.0) * max(1, submitted)
        while len(results) + len(exec_failed) < submitted and time.monotonic() < deadline:
            drain(0.2)
            if not any(t.is_alive() for t in threads) and result_q.empty():
                break
        for t in threads:
            t.join(timeout=5.0)
        drain()
    finally:
        if stream is not None:
            stream.close()
    results.sort(key=lambda r: r[1].p50_tf, reverse=True)
    log(f"Compiled: {len(artifact_paths)} ok, {len(compile_failed)} rejected or failed")
    if submitted:
        log(f"Executed: {len(results) + len(exec_failed)}/{submitted}, {len(exec_failed)} failed")
    elif num_gpus == 0:
        log("No GPUs -- execution skipped.")
    for cfg, why in compile_failed + exec_failed:
        repro = ""
        if repro_cmd_fn is not None:
            try:
                repro = f" | repro: {repro_cmd_fn(cfg)}"
            except Exception:
                pass
        log(f"  FAILED {why}: {cfg.label}{repro}")
    if results:
        best_cfg, best = results[0]
        log(f"Best: {best_cfg.label}: {best.p50_tf:.1f} TF p50 ({best.p50_pct:.1f}%)")
    return results, artifact_paths


# ---------------------------------------------------------------------------------------------
# command-line arguments shared by the bench scripts
# ---------------------------------------------------------------------------------------------
def add_sweep_cli_args(parser: argparse.ArgumentParser) -> None:
    a = parser.add_argument
    a("--mcpu", type=str, required=True, help="Target architecture (sm_100a); explicit so that nothing is silently built for the wrong part")
    a("--compile-only", action="store_true", help="Build the plan artifacts, skip execution and verification (required on a host without a matching GPU)")
    a("--compile-sample", type=int, default=512, help="Configs to compile per tier (0 = all)")
    a("--seed", type=int, default=42, help="Random seed of the tier sampling")
    a("--num-gpus", type=int, default=None, help="GPUs to use (default: all visible)")
    a("--compile-workers", type=int, default=DEFAULT_COMPILE_WORKERS)
    a("--compile-timeout", type=int, default=DEFAULT_COMPILE_TIMEOUT, help="accepted for command-line compatibility; building a plan takes milliseconds")
    a("--no-reg-filter", action="store_true", help="Disable the resource filter")
    a("--iterations", type=int, default=NUM_ITERATIONS, help=f"Launches per config (default {NUM_ITERATIONS}; the first {WARMUP_ITERATIONS} are dropped)")
    a("--init", type=InitMode, default=INIT_DEFAULT, choices=list(InitMode), help="Input initialisation")
    a("--direct-b", action=argparse.BooleanOptionalAction, default=None, help="B through the direct-B path (packed once)")
    a("--hsaco-dir", type=str, default=None, help="Directory that keeps the plan artifacts between runs (default: a temporary one)")
    a("--results-file", type=str, default=None, help="Append BENCH_RESULT_JSON lines to this file")
    a("--tier-time-budget", type=float, default=None, help="Wall-clock seconds per tier; a tier that runs out returns what it has")
    a("--dry-run", action="store_true", help="Print the first tier's candidate labels and exit")


def add_single_cli_args(parser: argparse.ArgumentParser) -> None:
    a = parser.add_argument
    a("--mcpu", type=str, required=True, help="Target architecture (sm_100a)")
    a("--hsaco", type=str, default=None, help="A plan artifact built earlier")
    a("--compile-only", action="store_true")
    a("--print-ir-after-all", action="store_true", help="accepted and ignored (there is no IR)")
    a("--print-asm", action="store_true", help="print the plan artifact")
    a("--force", action="store_true", help="Run despite resource-filter violations")
    a("--num-vgprs", type=int, default=None, help="accepted and ignored")
    a("--num-agprs", type=int, default=None, help="accepted and ignored")
    a("--num-wg-per-cu", type=int, default=1)
    a("--iterations", type=int, default=NUM_ITERATIONS)
    a("--init", type=InitMode, default=INIT_DEFAULT, choices=list(InitMode))
    a("--results-file", type=str, default=None)


def require_gpu_or_compile_only(args) -> None:
    """Stop at once when there is no matching GPU and ``--compile-only`` was not given, instead
    of compiling for minutes and measuring nothing."""
    if getattr(args, "compile_only", False):
        print(f"Compile-only mode ({args.mcpu}); execution will be skipped.")
        return
    if getattr(args, "dry_run", False):
        return
    n = detect_num_gpus(args.mcpu)
    if n == 0:
        sys.exit(f"ERROR: no {args.mcpu} GPU detected. Pass --compile-only to build the artifacts without running them.")
    print(f"Detected {n} {args.mcpu} GPU(s).")
