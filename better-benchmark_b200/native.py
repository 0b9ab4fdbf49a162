"""ctypes binding of the C ABI in ``include/b200_oracles.h``.

The shared library is built in-tree (``csrc/libb200_oracles.so``) by ``build.py``. There is no
fallback of any kind: if the library is missing or a symbol cannot be resolved, loading raises
``NativeLibraryError`` and every kernel wrapper fails with it.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_double, c_int32, c_int64, c_void_p
from pathlib import Path

import os

# B200_ORACLES_LIB names another build of the library (a measurement variant); default: the in-tree one
LIB_PATH = Path(os.environ.get("B200_ORACLES_LIB") or Path(__file__).resolve().parent / "csrc" / "libb200_oracles.so")

# dtype codes shared with csrc/common.cuh
F32, BF16, F16 = 0, 1, 2

# status codes shared with csrc/common.cuh
OK = 0
ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_DEVICE_WAIT = -1, -2, -3, -4, -5


class NativeLibraryError(RuntimeError):
    """The CUDA library is not built or does not export the expected C ABI."""


class KernelArgumentError(ValueError):
    """An entry point rejected its arguments before launching anything (negative status)."""


class KernelLaunchError(RuntimeError):
    """A CUDA launch was rejected (positive status = cudaError_t). The text names CUDA so that
    sweep workers treat it as a device failure and restart."""


_P64 = ctypes.POINTER(c_int64)
_PF = c_void_p  # float* passed as raw address

# name -> (restype, argtypes); mirrors include/b200_oracles.h declaration by declaration
SIGNATURES = {
    "b200_last_error": (c_char_p, []),
    "b200_version": (c_int32, []),
    "b200_sm_count": (c_int32, []),
    "b200_l2_bytes": (c_int32, []),
    "b200_launch_count": (c_int64, []),
    "b200_last_kernel": (c_char_p, []),
    "b200_check_status": (c_int32, [c_void_p, c_void_p]),
    "b200_row_reduce": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, _P64,
                                  c_int64, c_int32, c_int32, c_int32, c_void_p]),
    "b200_softmax": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                               _P64, _P64, _P64, c_int32, c_int32, c_double, c_int32, c_void_p]),
    "b200_norm_fwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, _PF, _PF, _PF, c_int64,
                                c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, c_double,
                                c_double, c_int32, c_void_p]),
    "b200_norm_fwd_residual": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, _PF, _PF, _PF,
                                         c_int64, c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, c_double,
                                         c_double, c_int32, c_void_p]),
    "b200_norm_fwd_wait_timeouts": (c_int64, []),
    "b200_norm_bwd_wait_timeouts": (c_int64, []),
    "b200_norm_bwd_scratch_bytes": (c_int64, [c_int64]),
    "b200_norm_bwd": (c_int32, [c_void_p, c_void_p, c_void_p, _PF, _PF, c_void_p, _PF, _PF, c_int64,
                                c_int64, c_int64, c_int64, c_int32, c_int32, c_int32, c_int64,
                                c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64, c_int32,
                                c_void_p]),
    "b200_batch_norm_wait_timeouts": (c_int64, []),
    "b200_batch_norm_scratch_bytes": (c_int64, [c_int64]),
    "b200_batch_norm_fwd": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, _PF, _PF, _PF, _PF,
                                      c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32,
                                      c_int32, c_double, c_double, c_int32, c_void_p, c_int64,
                                      c_void_p]),
    "b200_batch_norm_fwd_ex": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, _PF, _PF, _PF, _PF,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_int32,
                                         c_int32, c_double, c_double, c_double, c_int32, c_void_p, c_int64,
                                         c_void_p]),
    "b200_batch_norm_bwd_ex": (c_int32, [c_void_p] * 9 + [c_int64] * 6 + [c_int32, c_int32, c_double, c_double,
                                                                          c_void_p, c_int64, c_void_p]),
    "b200_batch_norm_fwd_static_scratch": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, _PF, _PF, _PF,
                                                     _PF, c_int64, c_int64, c_int64, c_int64, c_int64,
                                                     c_int64, c_int32, c_int32, c_double, c_double, c_int32,
                                                     c_void_p]),
    "b200_batch_norm_bwd_scratch_bytes": (c_int64, [c_int64]),
    "b200_batch_norm_bwd": (c_int32, [c_void_p] * 9 + [c_int64] * 6 + [c_int32, c_int32, c_double, c_void_p,
                                                                       c_int64, c_void_p]),
    "b200_col_reduce": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                  c_int32, c_int32, c_int32, c_void_p, c_int64, c_void_p]),
    "b200_permute_copy": (c_int32, [c_void_p, c_void_p, _P64, _P64, c_int32, c_int32, c_double, c_int32,
                                    c_void_p]),
    "b200_transpose_copy": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                      c_int32, c_int32, c_double, c_int32, c_void_p]),
    "b200_cast_scale": (c_int32, [c_void_p, c_void_p, c_int64, c_int32, c_int32, c_double, c_int32, c_void_p]),
    "b200_dropout_rms_norm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_double,
                                        c_double, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_int64, c_int32, c_void_p]),
    "b200_softmax_dropout": (c_int32, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                                       c_int64, c_int64, c_void_p, c_int32, c_double, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int32, c_void_p]),
    "b200_dropout_add": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_double, c_void_p, c_void_p, c_int64,
                                   c_int32, c_void_p]),
    "b200_dropout_layer_norm": (c_int32, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_double,
                                          c_double, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                          c_int32, c_void_p]),
}

_lib = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """Load the library once per process and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise NativeLibraryError(
                f"{LIB_PATH} is not built. Run `python -m better_benchmark_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or eager fallback.")
        try:
            lib = ctypes.CDLL(str(LIB_PATH))
        except OSError as e:
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
        for name, (restype, argtypes) in SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise NativeLibraryError(f"{LIB_PATH} does not export {name}") from e
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
        return lib


def last_error() -> str:
    msg = load().b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, what: str) -> None:
    """Turn an entry point's status into a Python exception."""
    if status == 0:
        return
    text = last_error()
    if status < 0:
        raise KernelArgumentError(f"{what}: status {status}: {text}")
    raise KernelLaunchError(f"{what}: CUDA error {status}: {text}")


def i64_array(values) -> ctypes.Array:
    vals = [int(v) for v in values]
    return (c_int64 * len(vals))(*vals)
