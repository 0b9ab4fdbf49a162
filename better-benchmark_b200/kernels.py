"""Tensor-level wrappers over the C ABI.

Each function validates device, dtype and layout, allocates its outputs with torch (so that CUDA
graph capture sees ordinary caching-allocator memory), and launches on the current CUDA stream
without synchronising. Layouts the kernels cannot address directly raise ``UnsupportedLayout``;
nothing is ever copied, made contiguous or computed by torch behind the caller's back.
"""
from __future__ import annotations

import torch

from . import native
from .native import F32, BF16, F16, check, i64_array, load

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

REDUCE_SUM, REDUCE_MEAN, REDUCE_AMAX, REDUCE_AMIN = 0, 1, 2, 3
_REDUCE_CODES = {"sum": REDUCE_SUM, "mean": REDUCE_MEAN, "amax": REDUCE_AMAX, "amin": REDUCE_AMIN}

SOFTMAX_LOG = 1          # log_softmax instead of softmax
SOFTMAX_SCALE = 2        # multiply by `scale` first
SOFTMAX_ROUND = 4        # multiply/add in the 16-bit input dtype, results rounded to it


class UnsupportedLayout(ValueError):
    """The tensor's strides or dtype have no kernel; the caller must pick another oracle."""


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise UnsupportedLayout(f"dtype {t.dtype} has no kernel (float32, bfloat16, float16 only)")


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise native.KernelArgumentError(
                "CUDA tensors required: this backend has no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise native.KernelArgumentError("all tensors must be on one device")
    return dev


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def collapse_outer(shape, strides_list):
    """Merge adjacent outer dimensions that every tensor addresses contiguously.

    ``shape`` is the common outer shape, ``strides_list`` one stride tuple per tensor (0 for
    broadcast dimensions). Returns (dims, strides_per_tensor) with at most three dimensions,
    padded with size-1 / stride-0 entries at the end, in the row = (i0*d1 + i1)*d2 + i2 order the
    kernels use. Raises UnsupportedLayout when more than three dimensions remain.
    """
    dims = []
    strs = [[] for _ in strides_list]
    for i, size in enumerate(shape):
        if size == 1:
            continue
        cur = [s[i] for s in strides_list]
        if dims and all(strs[k][-1] == cur[k] * size for k in range(len(cur))):
            dims[-1] *= size
            for k in range(len(cur)):
                strs[k][-1] = cur[k]
        else:
            dims.append(size)
            for k in range(len(cur)):
                strs[k].append(cur[k])
    if len(dims) > 3:
        raise UnsupportedLayout(f"outer dimensions {list(shape)} do not collapse to three")
    while len(dims) < 3:
        dims.append(1)
        for s in strs:
            s.append(0)
    return dims, strs


def _is_dense(t: torch.Tensor) -> bool:
    """True when the tensor covers its storage range exactly once (some permutation of a
    contiguous layout), so an output may reuse its strides."""
    if t.is_contiguous():
        return True
    expected = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(t.shape, t.stride()) if sz != 1),
                               key=lambda p: p[1]):
        if stride != expected:
            return False
        expected *= size
    return True


def _outer(t: torch.Tensor):
    return tuple(t.shape[:-1]), tuple(t.stride()[:-1])


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def row_reduce(x: torch.Tensor, op: str, *, keepdim: bool = False,
               out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """sum / mean / amax / amin over the last dimension (which must have stride 1)."""
    _require_cuda(x)
    if x.dim() < 1:
        raise UnsupportedLayout("row_reduce needs at least one dimension")
    n = x.shape[-1]
    if n > 1 and x.stride(-1) != 1:
        raise UnsupportedLayout("row_reduce: the reduced dimension must be contiguous")
    out_dtype = out_dtype or x.dtype
    oshape, ostrides = _outer(x)
    rows = _numel(oshape)
    out_shape = list(oshape) + ([1] if keepdim else [])
    out = torch.empty(out_shape, dtype=out_dtype, device=x.device)
    if rows == 0:
        return out
    if n == 0:
        # Nothing to read: the result is the reduction's identity (a fill, not a computation).
        if op in ("amax", "amin"):
            raise native.KernelArgumentError(f"row_reduce: {op} of an empty row is undefined")
        return out.fill_(0.0 if op == "sum" else float("nan"))
    dims, (xs,) = collapse_outer(oshape, [ostrides])
    lib = load()
    check(lib.b200_row_reduce(_ptr(x), _ptr(out), rows, n, dims[1], dims[2], i64_array(xs), 1,
                              _code(x), _DTYPE_CODE[out_dtype], _REDUCE_CODES[op], _stream()),
          "b200_row_reduce")
    return out


def softmax(x: torch.Tensor, *, mask: torch.Tensor | None = None, scale: float | None = None,
            log: bool = False, out_dtype: torch.dtype | None = None,
            round_intermediates: bool = True, out: torch.Tensor | None = None) -> torch.Tensor:
    """softmax / log_softmax over the last dimension of ``x [* scale] [+ mask]``.

    ``mask`` broadcasts against ``x`` over the outer dimensions and must have the full last
    dimension and x's dtype. With ``round_intermediates`` the scaled and masked values are rounded
    to x's dtype, which is what a 16-bit aten graph does when the multiply and add run before the
    conversion to fp32; pass False when the graph converts first.
    """
    _require_cuda(x, mask, out)
    n = x.shape[-1]
    if n > 1 and x.stride(-1) != 1:
        raise UnsupportedLayout("softmax: the last dimension must be contiguous")
    out_dtype = out_dtype or x.dtype
    if out is None:
        if _is_dense(x):
            out = torch.empty_strided(x.shape, x.stride(), dtype=out_dtype, device=x.device)
        else:
            out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    elif out.shape != x.shape or (n > 1 and out.stride(-1) != 1):
        raise UnsupportedLayout("softmax: out must match x's shape with a contiguous last dim")
    if x.numel() == 0:
        return out
    oshape, xstr = _outer(x)
    _, ystr = _outer(out)
    tensors = [xstr, ystr]
    if mask is not None:
        if mask.dtype != x.dtype:
            raise UnsupportedLayout("softmax: mask dtype must equal the input dtype")
        if mask.shape[-1] != n or (n > 1 and mask.stride(-1) != 1):
            raise UnsupportedLayout("softmax: mask needs the full, contiguous last dimension")
        m = mask.expand(x.shape)
        tensors.append(tuple(m.stride()[:-1]))
    dims, strs = collapse_outer(oshape, tensors)
    rows = _numel(oshape)
    flags = (SOFTMAX_LOG if log else 0) | (SOFTMAX_SCALE if scale is not None else 0)
    if round_intermediates and x.dtype != torch.float32:
        flags |= SOFTMAX_ROUND
    lib = load()
    check(lib.b200_softmax(_ptr(x), _ptr(mask), _ptr(out), rows, n, dims[1], dims[2],
                           i64_array(strs[0]), i64_array(strs[2]) if mask is not None else None,
                           i64_array(strs[1]), _code(x), _DTYPE_CODE[out_dtype],
                           float(scale) if scale is not None else 1.0, flags, _stream()),
          "b200_softmax")
    return out


def _rows_2d(t: torch.Tensor, what: str):
    """View a tensor as [rows, n] with one uniform row stride; no copy."""
    n = t.shape[-1]
    if n > 1 and t.stride(-1) != 1:
        raise UnsupportedLayout(f"{what}: the last dimension must be contiguous")
    oshape, ostr = _outer(t)
    dims, (s,) = collapse_outer(oshape, [ostr])
    if dims[1] != 1 or dims[2] != 1:
        raise UnsupportedLayout(f"{what}: rows must be evenly strided (outer dims {list(oshape)})")
    rows = _numel(oshape)
    return rows, n, (s[0] if rows > 1 else n)


def norm_fwd(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None, *,
             eps: float, rms: bool = False, out_dtype: torch.dtype | None = None,
             want_y: bool = True, want_mean: bool = False, want_rstd: bool = False,
             want_var: bool = False, correction: float = 0.0, keepdim: bool = True):
    """LayerNorm (rms=False) or RMSNorm (rms=True) forward over the last dimension.

    Returns (y, mean, rstd, var) with None for the outputs not requested. Statistics are fp32 with
    x's outer shape (plus a trailing 1 when ``keepdim``).
    """
    _require_cuda(x, weight, bias)
    rows, n, x_stride = _rows_2d(x, "norm_fwd")
    out_dtype = out_dtype or x.dtype
    w_code = F32
    for p in (weight, bias):
        if p is not None:
            if p.dim() != 1 or p.shape[0] != n or not p.is_contiguous():
                raise UnsupportedLayout("norm_fwd: weight/bias must be contiguous [n]")
            w_code = _code(p)
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        raise UnsupportedLayout("norm_fwd: weight and bias must share a dtype")
    y = None
    y_stride = n
    if want_y:
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    stat_shape = list(x.shape[:-1]) + ([1] if keepdim else [])

    def stat(flag):
        return torch.empty(stat_shape, dtype=torch.float32, device=x.device) if flag else None

    mean, rstd, var = stat(want_mean and not rms), stat(want_rstd), stat(want_var)
    lib = load()
    check(lib.b200_norm_fwd(_ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _ptr(mean), _ptr(rstd),
                            _ptr(var), rows, n, x_stride, y_stride, _code(x), w_code,
                            _DTYPE_CODE[out_dtype], float(eps), float(correction), 1 if rms else 0,
                            _stream()),
          "b200_norm_fwd")
    return y, mean, rstd, var
