"""The per-GPU timing lock (CPU): exclusion between processes, re-entrancy, stale holders,
environment switches. Failures are made on the host (a pre-held flock, a dead PID in the metadata)."""
import fcntl
import os
import subprocess
import sys
import time

import pytest

from better_benchmark_b200 import gpu_lock


@pytest.fixture
def lock_env(tmp_path, monkeypatch):
    monkeypatch.setenv("COMPILE_UTILS_GPU_LOCK_DIR", str(tmp_path))
    monkeypatch.delenv("INDUCTOR_GPU_BENCH_LOCK", raising=False)
    monkeypatch.delenv("TORCHINDUCTOR_GPU_BENCH_LOCK", raising=False)
    monkeypatch.delenv("INDUCTOR_GPU_BENCH_LOCK_DIR", raising=False)
    monkeypatch.delenv("TORCHINDUCTOR_GPU_BENCH_LOCK_DIR", raising=False)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3")
    return tmp_path


def test_lock_files_metadata_and_reentrancy(lock_env):
    with gpu_lock.gpu_exclusive_lock("outer"):
        meta = gpu_lock.read_lock_metadata(str(lock_env / "gpu_3.lock"))
        assert meta["pid"] == str(os.getpid()) and meta["label"] == "outer" and meta["mode"] == "exclusive"
        assert (lock_env / "gpu_3.gate").exists()
        with gpu_lock.gpu_exclusive_lock("inner"):       # nests without deadlock
            pass
    fd = os.open(lock_env / "gpu_3.lock", os.O_RDWR)     # released: another holder can take it
    fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
    fcntl.flock(fd, fcntl.LOCK_UN)
    os.close(fd)


def test_disabled_skips_unless_forced(lock_env, monkeypatch):
    with gpu_lock.gpu_exclusive_lock("x", disabled=True):
        assert not (lock_env / "gpu_3.lock").exists()
    monkeypatch.setenv("INDUCTOR_GPU_BENCH_LOCK", "1")
    with gpu_lock.gpu_exclusive_lock("x", disabled=True):
        assert (lock_env / "gpu_3.lock").exists()


def _hold_lock_in_child(path, seconds, fake_pid=None):
    code = (
        "import fcntl,os,sys,time\n"
        f"fd=os.open({str(path)!r},os.O_CREAT|os.O_RDWR,0o666)\n"
        "fcntl.flock(fd,fcntl.LOCK_EX)\n"
        f"os.write(fd,('pid=%s\\nlabel=child\\n' % ({fake_pid!r} or os.getpid())).encode())\n"
        "print('held',flush=True)\n"
        f"time.sleep({seconds})\n")
    p = subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, text=True)
    assert p.stdout.readline().strip() == "held"
    return p


def test_waits_for_a_live_holder_then_acquires(lock_env):
    child = _hold_lock_in_child(lock_env / "gpu_3.lock", 0.6)
    t0 = time.monotonic()
    with gpu_lock.gpu_exclusive_lock("waiter", timeout_s=10):
        waited = time.monotonic() - t0
    child.wait()
    assert waited >= 0.3


def test_times_out_on_a_live_holder(lock_env):
    child = _hold_lock_in_child(lock_env / "gpu_3.lock", 3)
    with pytest.raises(TimeoutError, match="timed out"):
        with gpu_lock.gpu_exclusive_lock("waiter", timeout_s=0.3):
            pass
    child.kill()
    child.wait()


def test_reports_a_stale_holder_whose_pid_is_dead(lock_env, monkeypatch):
    monkeypatch.setenv("COMPILE_UTILS_GPU_LOCK_STALE_GRACE_S", "0.2")
    dead = subprocess.Popen([sys.executable, "-c", "pass"])
    dead.wait()
    child = _hold_lock_in_child(lock_env / "gpu_3.lock", 3, fake_pid=dead.pid)
    with pytest.raises(TimeoutError, match="stale"):
        with gpu_lock.gpu_exclusive_lock("waiter", timeout_s=5):
            pass
    child.kill()
    child.wait()


def test_gpu_id_comes_from_visible_devices(monkeypatch):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "GPU-abc/def, 5")
    assert gpu_lock.physical_gpu_id() == "GPU-abc_def"
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES")
    assert gpu_lock.physical_gpu_id() == "0"
    assert gpu_lock.pid_alive(os.getpid()) is True and gpu_lock.pid_alive("x") is None
