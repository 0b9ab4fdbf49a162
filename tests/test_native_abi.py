"""The shared library loads on a machine without a GPU and exports the whole declared C ABI.
No compute entry point is called here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "b200_oracles.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for expected in ("b200_row_reduce", "b200_softmax", "b200_norm_fwd", "b200_norm_bwd",
                     "b200_batch_norm_fwd", "b200_last_error", "b200_version"):
        assert expected in names


def test_library_exports_every_declared_symbol():
    from better_benchmark_b200 import native
    if not native.LIB_PATH.exists():
        from better_benchmark_b200.build import build_library
        build_library()
    lib = ctypes.CDLL(str(native.LIB_PATH))
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert missing == []


def test_binding_table_matches_header():
    from better_benchmark_b200 import native
    assert sorted(native.SIGNATURES) == declared_symbols()
    lib = native.load()
    assert lib.b200_version() >= 1
    assert native.last_error() == "" or isinstance(native.last_error(), str)


def test_wrappers_refuse_cpu_tensors_and_missing_library(monkeypatch, tmp_path):
    import torch
    from better_benchmark_b200 import kernels, native
    with pytest.raises(native.KernelArgumentError):
        kernels.row_reduce(torch.zeros(4, 4), "sum")
    with pytest.raises(native.KernelArgumentError):
        kernels.norm_fwd(torch.zeros(4, 8), None, None, eps=1e-5)
    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setattr(native, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(native.NativeLibraryError):
        native.load()
