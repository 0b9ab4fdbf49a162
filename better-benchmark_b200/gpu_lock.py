"""Per-GPU advisory file lock that serialises timing windows between processes.

Mirrors the protocol of the reference (``oracle_harness.py:1614-1692`` and
``scripts/gpu_lock.py:164-205``): one ``gpu_<id>.gate`` and one ``gpu_<id>.lock`` file per
physical GPU under a shared directory, taken with ``flock`` (gate first, then lock), holder
metadata written into the lock file, re-entrant within a process, and a stale-holder check that
reports a lock whose recorded PID is dead instead of waiting for ever.

Environment (same names as the reference):
  INDUCTOR_GPU_BENCH_LOCK / TORCHINDUCTOR_GPU_BENCH_LOCK = 1   force the lock on
  INDUCTOR_GPU_BENCH_LOCK_DIR / TORCHINDUCTOR_GPU_BENCH_LOCK_DIR / COMPILE_UTILS_GPU_LOCK_DIR
  COMPILE_UTILS_GPU_LOCK_STALE_GRACE_S  seconds a dead holder is tolerated (default 5)
"""
from __future__ import annotations

import contextlib
import fcntl
import os
import re
import tempfile
import threading
import time

_state = threading.local()
_mutex = threading.RLock()


def _flag(name: str) -> bool:
    return os.environ.get(name, "").strip().lower() in ("1", "true", "yes", "on")


def lock_forced() -> bool:
    return _flag("INDUCTOR_GPU_BENCH_LOCK") or _flag("TORCHINDUCTOR_GPU_BENCH_LOCK")


def lock_dir() -> str:
    return (os.environ.get("INDUCTOR_GPU_BENCH_LOCK_DIR")
            or os.environ.get("TORCHINDUCTOR_GPU_BENCH_LOCK_DIR")
            or os.environ.get("COMPILE_UTILS_GPU_LOCK_DIR")
            or os.path.join(tempfile.gettempdir(), "compile_utils_gpu_locks"))


def stale_grace_s() -> float:
    return float(os.environ.get("COMPILE_UTILS_GPU_LOCK_STALE_GRACE_S", "5"))


def physical_gpu_id() -> str:
    """The GPU this process times on: the first entry of CUDA_VISIBLE_DEVICES, else "0"."""
    visible = [d.strip() for d in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if d.strip()]
    raw = visible[0] if visible else "0"
    return re.sub(r"[^A-Za-z0-9_.-]+", "_", raw) or "unknown"


def read_lock_metadata(path: str) -> dict:
    meta = {}
    try:
        with open(path) as f:
            for line in f:
                if "=" in line:
                    k, v = line.strip().split("=", 1)
                    meta[k] = v
    except OSError:
        pass
    return meta


def pid_alive(pid) -> bool | None:
    """True/False when it can be told, None when the metadata has no usable PID."""
    try:
        pid = int(pid)
    except (TypeError, ValueError):
        return None
    if pid <= 0:
        return None
    try:
        os.kill(pid, 0)
    except ProcessLookupError:
        return False
    except PermissionError:
        return True
    return True


def _write_metadata(fd: int, gpu: str, mode: str, label: str) -> None:
    try:
        os.ftruncate(fd, 0)
        os.lseek(fd, 0, os.SEEK_SET)
        os.write(fd, (f"pid={os.getpid()}\ngpu={gpu}\nmode={mode}\nlabel={label}\n"
                      f"acquired_unix={time.time():.0f}\n").encode())
        os.fsync(fd)
    except OSError:
        pass


def _acquire(fd: int, path: str, timeout_s: float | None, poll_s: float) -> None:
    """flock(LOCK_EX) with stale-holder detection and an optional timeout."""
    start = time.monotonic()
    stale_since = None
    while True:
        try:
            fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
            return
        except BlockingIOError:
            pass
        now = time.monotonic()
        meta = read_lock_metadata(path)
        if pid_alive(meta.get("pid")) is False:
            stale_since = stale_since if stale_since is not None else now
            if now - stale_since >= stale_grace_s():
                raise TimeoutError(f"GPU lock appears stale: {path} reports dead holder "
                                   f"pid={meta.get('pid')} label={meta.get('label')}")
        else:
            stale_since = None
        if timeout_s is not None and now - start >= timeout_s:
            raise TimeoutError(f"timed out waiting for {path} (holder pid={meta.get('pid')} "
                               f"label={meta.get('label')})")
        time.sleep(poll_s)


@contextlib.contextmanager
def gpu_exclusive_lock(label: str = "oracle_bench", *, disabled: bool = False,
                       timeout_s: float | None = None, poll_s: float = 0.05):
    """Hold the exclusive timing lock of this process's GPU.

    On by default. ``disabled=True`` skips it unless an environment flag forces it on. Nested
    use inside one thread just counts depth.
    """
    if disabled and not lock_forced():
        yield
        return
    depth = getattr(_state, "depth", 0)
    if depth > 0:
        _state.depth = depth + 1
        try:
            yield
        finally:
            _state.depth -= 1
        return
    directory = lock_dir()
    os.makedirs(directory, exist_ok=True)
    gpu = physical_gpu_id()
    lock_path = os.path.join(directory, f"gpu_{gpu}.lock")
    gate_path = os.path.join(directory, f"gpu_{gpu}.gate")
    with _mutex:
        fd = gate_fd = None
        try:
            fd = os.open(lock_path, os.O_CREAT | os.O_RDWR, 0o666)
            gate_fd = os.open(gate_path, os.O_CREAT | os.O_RDWR, 0o666)
            _acquire(gate_fd, gate_path, timeout_s, poll_s)
            _acquire(fd, lock_path, timeout_s, poll_s)
            _write_metadata(fd, gpu, "exclusive", label)
            _state.depth = 1
            try:
                yield
            finally:
                _state.depth = 0
        finally:
            for f in (fd, gate_fd):
                if f is not None:
                    try:
                        fcntl.flock(f, fcntl.LOCK_UN)
                    finally:
                        os.close(f)
