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
    if dev is not None and dev.index is not None and dev.index != torch.cuda.current_device():
        # the library launches on the current device's current stream and reads that device's
        # properties: pointers of another GPU would fault there, or silently cross NVLink
        raise native.KernelArgumentError(
            f"tensors live on cuda:{dev.index} but the current device is cuda:{torch.cuda.current_device()}; "
            "make their device current first (torch.cuda.set_device or `with torch.cuda.device(...)`)")
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
            round_intermediates: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """softmax / log_softmax over the last dimension of ``x [* scale] [+ mask]``.

    ``mask`` broadcasts against ``x`` over the outer dimensions and must have the full last
    dimension and x's dtype. By default the scale and the mask are applied in fp32 and nothing is
    rounded before the softmax: that is how a fused kernel (the reference's own oracles, Inductor)
    evaluates a 16-bit graph, and what the reference's numerics gate compares against (its anchor is
    the graph evaluated on fp64 inputs, where the 16-bit roundings of intermediates do not exist).
    With ``round_intermediates`` the scaled and masked values are rounded to x's dtype the way the
    eager 16-bit graph materialises them.
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


_NORM_PROLOGUES = {None: 0, "gelu_erf": 2}


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


_SUM_FORMS = {False: 0, True: 4, "both": 8}   # bits 2 and 3 of b200_norm_fwd_residual's mode word


def norm_fwd(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None, *,
             eps: float, rms: bool = False, out_dtype: torch.dtype | None = None,
             want_y: bool = True, want_mean: bool = False, want_rstd: bool = False,
             want_var: bool = False, correction: float = 0.0, keepdim: bool = True,
             prologue: str | None = None, residual: torch.Tensor | None = None, want_sum: bool = False,
             round_sum: bool | str = False):
    """LayerNorm (rms=False) or RMSNorm (rms=True) forward over the last dimension.

    ``prologue="gelu_erf"`` normalises ``gelu(x)`` (exact, erf form) rounded to x's dtype instead
    of x: the activation that the graph materialises in front of the norm is fused into the load.
    ``residual`` (x's shape, dtype and strides) normalises ``x + residual``; ``want_sum`` returns the
    sum, rounded to x's dtype, as a fifth value. The sum that is normalised stays in fp32 (Inductor's
    fused form, which the reference's fp64-anchored gate accepts) unless ``round_sum`` asks for the
    eager graph's materialised 16-bit intermediate (``True``) or for both (``"both"``, LayerNorm
    only): each element then takes the fp32 form where that form's output exceeds 3 in magnitude and
    the rounded form elsewhere, which is what the reference's own oracles for these regions return
    (repros/canonical/var_mean_45f7dfd4a983/oracle.py:96-107) - small outputs equal the eager
    module's, large ones carry no intermediate rounding.

    Returns (y, mean, rstd, var) with None for the outputs not requested. Statistics are fp32 with
    x's outer shape (plus a trailing 1 when ``keepdim``).
    """
    _require_cuda(x, weight, bias, residual)
    rows, n, x_stride = _rows_2d(x, "norm_fwd")
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype or residual.stride() != x.stride():
            raise UnsupportedLayout("norm_fwd: residual must have x's shape, dtype and strides")
        if out_dtype not in (None, x.dtype):
            raise UnsupportedLayout("norm_fwd: with a residual y has x's dtype")
    elif want_sum:
        raise native.KernelArgumentError("norm_fwd: want_sum needs a residual")
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
    if residual is None:
        check(lib.b200_norm_fwd(_ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _ptr(mean), _ptr(rstd),
                                _ptr(var), rows, n, x_stride, y_stride, _code(x), w_code,
                                _DTYPE_CODE[out_dtype], float(eps), float(correction),
                                (1 if rms else 0) | _NORM_PROLOGUES[prologue], _stream()),
              "b200_norm_fwd")
        return y, mean, rstd, var
    total = torch.empty(x.shape, dtype=x.dtype, device=x.device) if want_sum else None
    check(lib.b200_norm_fwd_residual(_ptr(x), _ptr(residual), _ptr(total), _ptr(weight), _ptr(bias), _ptr(y),
                                     _ptr(mean), _ptr(rstd), _ptr(var), rows, n, x_stride, y_stride, _code(x),
                                     w_code, _DTYPE_CODE[out_dtype], float(eps), float(correction),
                                     (1 if rms else 0) | _NORM_PROLOGUES[prologue] | _SUM_FORMS[round_sum], _stream()),
          "b200_norm_fwd_residual")
    return (y, mean, rstd, var, total) if want_sum else (y, mean, rstd, var)


# ---------------------------------------------------------------------------------------------
# Scratch memory. Kernels that combine per-CTA partial results take a caller-provided scratch
# buffer. One zero-initialised buffer per device is kept here; the first 256 bytes hold the
# grid-barrier words, which every kernel leaves at zero when it finishes. Kernels on one stream run
# in order, so sharing the buffer is safe there; callers that launch on several streams at once must
# pass their own ``scratch``. A request for more bytes than the buffer holds allocates a larger one,
# but the smaller ones are never released: a CUDA graph captured earlier still holds their address.
# Growing while the current stream is being captured is refused (the new buffer would belong to
# that graph's private pool while later, uncaptured calls keep using it).
# ---------------------------------------------------------------------------------------------
_scratch_by_device: dict = {}   # (type, index) -> [buffers, newest and largest last]
SCRATCH_DEFAULT_BYTES = 64 << 20  # covers every kernel of the library for rows of up to 4096 elements


def _device_key(device: torch.device):
    return device.type, device.index if device.index is not None else torch.cuda.current_device()


def scratch_buffer(device: torch.device, nbytes: int) -> torch.Tensor:
    bufs = _scratch_by_device.setdefault(_device_key(device), [])
    if bufs and bufs[-1].numel() >= nbytes:
        return bufs[-1]
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError(
            f"the shared scratch buffer would have to grow to {int(nbytes)} bytes during CUDA graph capture; "
            "run the call once before capturing, or pass scratch= explicitly")
    buf = torch.zeros(max(int(nbytes), SCRATCH_DEFAULT_BYTES), dtype=torch.uint8, device=device)
    bufs.append(buf)  # superseded buffers stay alive: captured graphs may still point at them
    return buf


def check_scratch_status(device: torch.device | None = None) -> None:
    """Raise if a cooperative kernel on this device gave up a grid-wide wait (synchronises)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    lib = load()
    for buf in _scratch_by_device.get(_device_key(device), []):
        status = lib.b200_check_status(_ptr(buf), _stream())
        if status != 0:
            buf[:16].zero_()
            check(status, "b200_check_status")


NORM_BWD_TWO_LAUNCH = 1  # flag: main kernel + finalize kernel instead of one cooperative launch
NORM_BWD_DY_SCALAR = 2   # flag: dy is one element that stands for the whole tensor (an expanded 0-dim gradient)


def norm_bwd(x: torch.Tensor, dy: torch.Tensor, weight: torch.Tensor | None, rstd: torch.Tensor, *,
             mean: torch.Tensor | None = None, rms: bool, heads: int | None = None,
             want_dweight: bool = True, want_dbias: bool = False, two_launch: bool = False,
             scratch: torch.Tensor | None = None):
    """LayerNorm / RMSNorm backward over the last dimension (flattened over trailing dims for 4-D).

    ``dy`` may also be a single element (0-dim, or expanded to x's shape with zero strides): the
    kernels then read it as a scalar. ``x`` and ``dy`` are [..., n] or, with ``heads``, [B, S, H, D] (n = H*D): dx is then returned
    as a contiguous [B, H, S, D] tensor, the permute fused into the store. ``rstd`` (and ``mean``
    for LayerNorm) are fp32 with one value per row. Returns (dx, dweight, dbias); the gradients of
    weight and bias are fp32 [n].
    """
    _require_cuda(x, dy, weight, rstd, mean, scratch)
    # a 0-dim (or fully expanded one-element) dy is read as a scalar by the kernel: nothing is materialised
    dy_scalar = dy.numel() == 1 or (dy.shape == x.shape and all(st == 0 for st in dy.stride()))
    if x.dtype != dy.dtype or (not dy_scalar and x.shape != dy.shape):
        raise UnsupportedLayout("norm_bwd: x and dy must agree in shape and dtype")
    if heads is not None:
        if x.dim() != 4 or x.shape[2] != heads or not x.is_contiguous() or not (dy_scalar or dy.is_contiguous()):
            raise UnsupportedLayout("norm_bwd: heads= needs contiguous [B, S, H, D] inputs")
        b, s, h, d = x.shape
        rows, n = b * s, h * d
        x_stride = dy_stride = n
        dx = torch.empty((b, h, s, d), dtype=x.dtype, device=x.device)
        seq, head_dim = s, d
        dx_batch, dx_seq, dx_head = h * s * d, d, s * d
    else:
        rows, n, x_stride = _rows_2d(x, "norm_bwd")
        dy_stride = 0 if dy_scalar else _rows_2d(dy, "norm_bwd")[2]
        dx = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        seq, head_dim = 1, n
        dx_batch, dx_seq, dx_head = n, 0, n
    if rstd.dtype != torch.float32 or rstd.numel() != rows or not rstd.is_contiguous():
        raise UnsupportedLayout("norm_bwd: rstd must be contiguous fp32 with one value per row")
    if not rms:
        if mean is None or mean.dtype != torch.float32 or mean.numel() != rows or not mean.is_contiguous():
            raise UnsupportedLayout("norm_bwd: LayerNorm needs a contiguous fp32 mean per row")
    w_code = F32
    if weight is not None:
        if weight.dim() != 1 or weight.shape[0] != n or not weight.is_contiguous():
            raise UnsupportedLayout("norm_bwd: weight must be contiguous [n]")
        w_code = _code(weight)
    dw = torch.empty(n, dtype=torch.float32, device=x.device) if want_dweight else None
    db = torch.empty(n, dtype=torch.float32, device=x.device) if (want_dbias and not rms) else None
    lib = load()
    nbytes = 0
    if dw is not None or db is not None:
        nbytes = int(lib.b200_norm_bwd_scratch_bytes(n))
        if scratch is None:
            scratch = scratch_buffer(x.device, nbytes)
        nbytes = scratch.numel() * scratch.element_size()
    check(lib.b200_norm_bwd(_ptr(x), _ptr(dy), _ptr(weight), _ptr(mean), _ptr(rstd), _ptr(dx),
                            _ptr(dw), _ptr(db), rows, n, x_stride, dy_stride, _code(x), w_code,
                            1 if rms else 0, seq, head_dim, dx_batch, dx_seq, dx_head,
                            _ptr(scratch), nbytes,
                            (NORM_BWD_TWO_LAUNCH if two_launch else 0) | (NORM_BWD_DY_SCALAR if dy_scalar else 0),
                            _stream()),
          "b200_norm_bwd")
    return dx, dw, db


def batch_norm_fwd(x: torch.Tensor, weight: torch.Tensor | None, bias: torch.Tensor | None,
                   running_mean: torch.Tensor | None, running_var: torch.Tensor | None, *,
                   eps: float, momentum: float, relu: bool = False,
                   unbiased_factor: float | None = None, scratch: torch.Tensor | None = None):
    """BatchNorm2d training forward (+ optional ReLU) on a dense NCHW or channels-last tensor.

    Returns (y, mean, invstd): y has x's dtype and strides, mean/invstd are fp32 [C].
    ``running_mean`` / ``running_var`` (fp32 [C]) are updated in place when given.
    ``unbiased_factor`` replaces n / (n - 1) in the running-variance update: a captured graph
    holds that factor as a literal of the shape it was captured at.
    """
    _require_cuda(x, weight, bias, running_mean, running_var, scratch)
    if x.dim() != 4:
        raise UnsupportedLayout("batch_norm_fwd: expected a 4-D [N, C, H, W] tensor")
    n, c, h, w = x.shape
    sn, sc, sh, sw = x.stride()
    if x.numel() == 0:
        raise native.KernelArgumentError("batch_norm_fwd: empty input has no statistics")
    if h > 1 and w > 1 and sh != w * sw:
        raise UnsupportedLayout("batch_norm_fwd: H and W must collapse into one strided dimension")
    ss = sw if w > 1 else (sh if h > 1 else 1)
    if not _is_dense(x):
        raise UnsupportedLayout("batch_norm_fwd: x must be dense (NCHW or channels-last)")
    w_code = F32
    for prm in (weight, bias):
        if prm is not None:
            if prm.dim() != 1 or prm.shape[0] != c or not prm.is_contiguous():
                raise UnsupportedLayout("batch_norm_fwd: weight/bias must be contiguous [C]")
            w_code = _code(prm)
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        raise UnsupportedLayout("batch_norm_fwd: weight and bias must share a dtype")
    for stat in (running_mean, running_var):
        if stat is not None and (stat.dtype != torch.float32 or stat.shape != (c,) or not stat.is_contiguous()):
            raise UnsupportedLayout("batch_norm_fwd: running statistics must be contiguous fp32 [C]")
    y = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device)
    mean = torch.empty(c, dtype=torch.float32, device=x.device)
    invstd = torch.empty(c, dtype=torch.float32, device=x.device)
    lib = load()
    nbytes = int(lib.b200_batch_norm_scratch_bytes(c))
    if scratch is None:
        scratch = scratch_buffer(x.device, nbytes)
    check(lib.b200_batch_norm_fwd_ex(_ptr(x), _ptr(y), _ptr(weight), _ptr(bias), _ptr(running_mean),
                                     _ptr(running_var), _ptr(mean), _ptr(invstd), n, c, h * w, sn, sc, ss,
                                     _code(x), w_code, float(eps), float(momentum),
                                     float(unbiased_factor) if unbiased_factor else 0.0, 1 if relu else 0,
                                     _ptr(scratch), scratch.numel() * scratch.element_size(), _stream()),
          "b200_batch_norm_fwd")
    return y, mean, invstd


def batch_norm_bwd(dy: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, invstd: torch.Tensor,
                   weight: torch.Tensor | None, *, act: torch.Tensor | None = None, slope: float = 0.0,
                   want_dx: bool = True, inv_count: float | None = None, scratch: torch.Tensor | None = None):
    """BatchNorm2d training backward on dense NCHW or channels-last tensors of one layout.

    Returns (dx, dweight, dbias): dx has x's dtype and strides, the other two are fp32 [C].
    ``mean`` / ``invstd`` are the saved statistics (fp32, C elements, any shape). With ``act`` the
    gradient first goes through the activation backward ``act > 0 ? dy : dy * slope``.
    ``inv_count`` replaces 1 / (N*H*W): a captured graph holds it as a literal of the shape it was
    captured at.
    """
    _require_cuda(dy, x, mean, invstd, weight, act, scratch)
    if x.dim() != 4 or dy.shape != x.shape or dy.dtype != x.dtype or dy.stride() != x.stride():
        raise UnsupportedLayout("batch_norm_bwd: dy and x must be 4-D with the same shape, dtype and strides")
    if act is not None and (act.shape != x.shape or act.dtype != x.dtype or act.stride() != x.stride()):
        raise UnsupportedLayout("batch_norm_bwd: act must match x in shape, dtype and strides")
    n, c, h, w = x.shape
    for t, name in ((mean, "mean"), (invstd, "invstd")):
        if t.dtype != torch.float32 or t.numel() != c or not t.is_contiguous():
            raise UnsupportedLayout(f"batch_norm_bwd: {name} must be contiguous fp32 with one value per channel")
    if weight is not None and (weight.dim() != 1 or weight.shape[0] != c or not weight.is_contiguous()):
        raise UnsupportedLayout("batch_norm_bwd: weight must be contiguous [C]")
    sn, sc, sh, sw = x.stride()
    if w > 1 and h > 1 and sh != sw * w:
        raise UnsupportedLayout("batch_norm_bwd: H and W must be mergeable into one spatial dimension")
    ss = sw if w > 1 else (sh if h > 1 else 1)
    dx = torch.empty_strided(x.shape, x.stride(), dtype=x.dtype, device=x.device) if want_dx else None
    dw = torch.empty(c, dtype=torch.float32, device=x.device)
    db = torch.empty(c, dtype=torch.float32, device=x.device)
    if x.numel() == 0:
        dw.zero_(); db.zero_()
        return dx, dw, db
    lib = load()
    need = int(lib.b200_batch_norm_bwd_scratch_bytes(c)) + 256
    if scratch is None:
        scratch = scratch_buffer(x.device, need)
    usable = scratch[256:]  # the barrier words at the head of the shared buffer stay untouched
    check(lib.b200_batch_norm_bwd_ex(_ptr(dy), _ptr(x), _ptr(act), _ptr(mean), _ptr(invstd), _ptr(weight),
                                     _ptr(dx), _ptr(dw), _ptr(db), n, c, h * w, sn, sc, ss, _code(x),
                                     _code(weight) if weight is not None else F32, float(slope),
                                     float(inv_count) if inv_count else 0.0, _ptr(usable), usable.numel(), _stream()),
          "b200_batch_norm_bwd")
    return dx, dw, db


COL_SUM, COL_MEAN, COL_AMAX = 0, 1, 2
_COL_CODES = {"sum": COL_SUM, "mean": COL_MEAN, "amax": COL_AMAX}


def col_reduce(x: torch.Tensor, op: str, *, out_dtype: torch.dtype | None = None,
               scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Reduce ``x`` [batch, rows, cols] (or [rows, cols]) over rows; cols must be contiguous.

    Returns [batch, cols] (or [cols]). A channels-last spatial mean is
    ``col_reduce(x.permute(0, 2, 3, 1).reshape(N, H*W, C), "mean")`` on views, without copies.
    """
    _require_cuda(x, scratch)
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(0)
    if x.dim() != 3:
        raise UnsupportedLayout("col_reduce: expected [batch, rows, cols] or [rows, cols]")
    b, r, c = x.shape
    if c > 1 and x.stride(2) != 1:
        raise UnsupportedLayout("col_reduce: the kept dimension must be contiguous")
    out_dtype = out_dtype or x.dtype
    out = torch.empty((b, c), dtype=out_dtype, device=x.device)
    if out.numel() == 0:
        return out[0] if squeeze else out
    if r == 0:
        if op == "amax":
            raise native.KernelArgumentError("col_reduce: amax over zero rows is undefined")
        out.fill_(0.0 if op == "sum" else float("nan"))
        return out[0] if squeeze else out
    if scratch is None:
        scratch = scratch_buffer(x.device, 1 << 20)
    # the barrier words at the head of the shared scratch buffer stay untouched
    usable = scratch[256:]
    lib = load()
    check(lib.b200_col_reduce(_ptr(x), _ptr(out), b, r, c, x.stride(0) if b > 1 else r * x.stride(1),
                              x.stride(1) if r > 1 else c, c, _code(x), _DTYPE_CODE[out_dtype],
                              _COL_CODES[op], _ptr(usable), usable.numel(), _stream()),
          "b200_col_reduce")
    return out[0] if squeeze else out


def permute_copy(x: torch.Tensor, dims, *, scale: float | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x.permute(dims)`` materialised contiguously, with an optional scale and dtype conversion.

    Up to four dimensions after adjacent dimensions that stay adjacent have been merged. A swap of
    the two innermost dimensions goes through the shared-memory transpose kernel.
    """
    _require_cuda(x)
    out_dtype = out_dtype or x.dtype
    view = x.permute(*dims)
    out = torch.empty(view.shape, dtype=out_dtype, device=x.device)
    if out.numel() == 0:
        return out
    shape, (strides,) = _collapse_all(tuple(view.shape), [tuple(view.stride())])
    lib = load()
    has_scale = 1 if scale is not None else 0
    sc = float(scale) if scale is not None else 1.0
    # [..., P, C] -> [..., C, P]: innermost output dim strided, the one before it unit-stride
    if len(shape) >= 2 and strides[-2] == 1 and strides[-1] != 1 and len(shape) <= 3:
        batch = shape[0] if len(shape) == 3 else 1
        bstride = strides[0] if len(shape) == 3 else 0
        cols, rows = shape[-2], shape[-1]          # output [batch, cols, rows], input [batch, rows, cols]
        check(lib.b200_transpose_copy(_ptr(x), _ptr(out), batch, rows, cols, bstride, strides[-1],
                                      _code(x), _DTYPE_CODE[out_dtype], sc, has_scale, _stream()),
              "b200_transpose_copy")
        return out
    if len(shape) > 4:
        raise UnsupportedLayout(f"permute_copy: {len(shape)} dimensions remain after merging (max 4)")
    pad = 4 - len(shape)
    shape4 = [1] * pad + list(shape)
    strides4 = [0] * pad + list(strides)
    check(lib.b200_permute_copy(_ptr(x), _ptr(out), i64_array(shape4), i64_array(strides4), _code(x),
                                _DTYPE_CODE[out_dtype], sc, has_scale, _stream()),
          "b200_permute_copy")
    return out


def _collapse_all(shape, strides_list):
    """collapse_outer over ALL dimensions (no reserved last dimension, no limit of three)."""
    dims, strs = [], [[] for _ in strides_list]
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
    if not dims:
        dims, strs = [1], [[1] for _ in strides_list]
    return dims, strs


_ACTIVATIONS = {None: 0, "relu": 2, "gelu_erf": 4, "silu": 8}


def cast_scale(x: torch.Tensor, out_dtype: torch.dtype, *, scale: float | None = None, relu: bool = False,
               activation: str | None = None) -> torch.Tensor:
    """Element-wise ``act(x * scale).to(out_dtype)`` (scale and the activation optional; ``relu=True``
    is ``activation="relu"``; also "gelu_erf", "silu") in fp32 for a dense tensor in any dimension
    order; the result keeps x's strides."""
    if relu:
        activation = "relu"
    _require_cuda(x)
    if not _is_dense(x):
        raise UnsupportedLayout("cast_scale: x must be dense")
    out = torch.empty_strided(x.shape, x.stride(), dtype=out_dtype, device=x.device)
    lib = load()
    check(lib.b200_cast_scale(_ptr(x), _ptr(out), x.numel(), _code(x), _DTYPE_CODE[out_dtype],
                              float(scale) if scale is not None else 1.0,
                              (1 if scale is not None else 0) | _ACTIVATIONS[activation], _stream()),
          "b200_cast_scale")
    return out


def dropout_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, seeds: torch.Tensor,
                     seed_index0: int, seed_index1: int, *, p: float, eps: float):
    """Dropout -> residual add -> RMSNorm -> dropout over the last dimension.

    x [rows, cols] bf16/fp16, residual fp32 with the same number of elements (any leading shape),
    weight fp32 [cols], seeds int64 (the two seeds are read on the device). Returns
    ``(keep0, sum, rstd, keep1, y)``: the masks as bool and ``sum`` shaped like ``residual``, ``rstd``
    as ``residual.shape[:-1] + (1,)``, ``y`` shaped like ``x``."""
    for t in (x, residual, weight, seeds):
        _require_cuda(t)
    cols = x.shape[-1]
    if residual.shape[-1] != cols or residual.numel() != x.numel() or weight.numel() != cols:
        raise native.KernelArgumentError("dropout_rms_norm: x, residual and weight disagree on the row length")
    if residual.dtype != torch.float32 or weight.dtype != torch.float32 or seeds.dtype != torch.int64:
        raise native.KernelArgumentError("dropout_rms_norm: residual and weight must be fp32, seeds int64")
    if not (x.is_contiguous() and residual.is_contiguous() and weight.is_contiguous() and seeds.is_contiguous()):
        raise UnsupportedLayout("dropout_rms_norm: tensors must be contiguous")
    if not (0 <= seed_index0 < seeds.numel() and 0 <= seed_index1 < seeds.numel()):
        raise native.KernelArgumentError("dropout_rms_norm: seed index outside the seed tensor")
    rows = x.numel() // cols if cols else 0
    dev = x.device
    keep0 = torch.empty(residual.shape, dtype=torch.bool, device=dev)
    keep1 = torch.empty(residual.shape, dtype=torch.bool, device=dev)
    total = torch.empty_like(residual)
    rstd = torch.empty(tuple(residual.shape[:-1]) + (1,), dtype=torch.float32, device=dev)
    y = torch.empty_like(x)
    lib = load()
    check(lib.b200_dropout_rms_norm(_ptr(x), _ptr(residual), _ptr(weight), _ptr(seeds), int(seed_index0),
                                    int(seed_index1), float(p), float(eps), _ptr(keep0), _ptr(total),
                                    _ptr(rstd), _ptr(keep1), _ptr(y), rows, cols, _code(x), _stream()),
          "b200_dropout_rms_norm")
    return keep0, total, rstd, keep1, y


def dropout_layer_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                       seeds: torch.Tensor, seed_index: int, *, p: float, eps: float):
    """Dropout -> residual add -> LayerNorm over the last dimension.

    x [rows, cols] bf16/fp16, residual fp32 with the same number of elements (any leading shape),
    weight and bias fp32 [cols], seeds int64. Returns ``(keep, xhat, y, rstd_over_n)``: the mask as
    bool, ``xhat`` and ``y`` fp32 shaped like ``residual``, ``rstd / cols`` as
    ``residual.shape[:-1] + (1,)``."""
    for t in (x, residual, weight, bias, seeds):
        _require_cuda(t)
    cols = x.shape[-1]
    if residual.shape[-1] != cols or residual.numel() != x.numel() or weight.numel() != cols \
            or bias.numel() != cols:
        raise native.KernelArgumentError("dropout_layer_norm: tensors disagree on the row length")
    if any(t.dtype != torch.float32 for t in (residual, weight, bias)) or seeds.dtype != torch.int64:
        raise native.KernelArgumentError("dropout_layer_norm: residual, weight and bias must be fp32, seeds int64")
    if not all(t.is_contiguous() for t in (x, residual, weight, bias, seeds)):
        raise UnsupportedLayout("dropout_layer_norm: tensors must be contiguous")
    if not 0 <= seed_index < seeds.numel():
        raise native.KernelArgumentError("dropout_layer_norm: seed index outside the seed tensor")
    rows = x.numel() // cols if cols else 0
    dev = x.device
    keep = torch.empty(residual.shape, dtype=torch.bool, device=dev)
    xhat = torch.empty_like(residual)
    y = torch.empty_like(residual)
    rstd_over_n = torch.empty(tuple(residual.shape[:-1]) + (1,), dtype=torch.float32, device=dev)
    lib = load()
    check(lib.b200_dropout_layer_norm(_ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(seeds),
                                      int(seed_index), float(p), float(eps), _ptr(keep), _ptr(xhat), _ptr(y),
                                      _ptr(rstd_over_n), rows, cols, _code(x), _stream()),
          "b200_dropout_layer_norm")
    return keep, xhat, y, rstd_over_n


def softmax_dropout(x: torch.Tensor, bias: torch.Tensor, seeds: torch.Tensor, seed_index: int, *, p: float):
    """``dropout(softmax(x + bias))`` over the last dimension, mask drawn in the kernel.

    x: contiguous bf16/fp16 ``[B*H, Sq, Sk]``; bias: fp32 ``[B, H, Sq, Sk]`` with ANY strides (read in
    place); seeds int64. Returns ``(logits, amax, sum, keep, y)``: the rounded logits ``[B, H, Sq, Sk]``
    in x's dtype, row maximum and row sum of the exponentials fp32 ``[B, H, Sq, 1]``, the mask as bool
    ``[B, H, Sq, Sk]`` and the dropped probabilities ``[B*H, Sq, Sk]`` in x's dtype, all contiguous."""
    for t in (x, bias, seeds):
        _require_cuda(t)
    if x.dim() != 3 or bias.dim() != 4:
        raise native.KernelArgumentError("softmax_dropout: x must be [B*H, Sq, Sk] and bias [B, H, Sq, Sk]")
    b, h, sq, sk = bias.shape
    if tuple(x.shape) != (b * h, sq, sk):
        raise native.KernelArgumentError(f"softmax_dropout: x {tuple(x.shape)} does not match bias {tuple(bias.shape)}")
    if bias.dtype != torch.float32 or seeds.dtype != torch.int64:
        raise native.KernelArgumentError("softmax_dropout: bias must be fp32, seeds int64")
    if not x.is_contiguous() or not seeds.is_contiguous():
        raise UnsupportedLayout("softmax_dropout: x and seeds must be contiguous")
    if not 0 <= seed_index < seeds.numel():
        raise native.KernelArgumentError("softmax_dropout: seed index outside the seed tensor")
    dev = x.device
    logits = torch.empty((b, h, sq, sk), dtype=x.dtype, device=dev)
    amax = torch.empty((b, h, sq, 1), dtype=torch.float32, device=dev)
    total = torch.empty((b, h, sq, 1), dtype=torch.float32, device=dev)
    keep = torch.empty((b, h, sq, sk), dtype=torch.bool, device=dev)
    y = torch.empty_like(x)
    lib = load()
    sb, sh, ssq, ssk = bias.stride()
    check(lib.b200_softmax_dropout(_ptr(x), _ptr(bias), b, h, sq, sk, sb, sh, ssq, ssk, _ptr(seeds), int(seed_index),
                                   float(p), _ptr(logits), _ptr(amax), _ptr(total), _ptr(keep), _ptr(y), _code(x),
                                   _stream()), "b200_softmax_dropout")
    return logits, amax, total, keep, y


def dropout_add(x: torch.Tensor, residual: torch.Tensor, seeds: torch.Tensor, seed_index: int, *, p: float):
    """``residual + dropout(x)``: x bf16/fp16, residual fp32 with the same number of elements. Returns
    ``(keep, sum)`` shaped like ``residual`` (bool, fp32)."""
    for t in (x, residual, seeds):
        _require_cuda(t)
    if residual.numel() != x.numel():
        raise native.KernelArgumentError("dropout_add: x and residual differ in size")
    if residual.dtype != torch.float32 or seeds.dtype != torch.int64:
        raise native.KernelArgumentError("dropout_add: residual must be fp32, seeds int64")
    if not all(t.is_contiguous() for t in (x, residual, seeds)):
        raise UnsupportedLayout("dropout_add: tensors must be contiguous")
    if not 0 <= seed_index < seeds.numel():
        raise native.KernelArgumentError("dropout_add: seed index outside the seed tensor")
    keep = torch.empty(residual.shape, dtype=torch.bool, device=x.device)
    total = torch.empty_like(residual)
    lib = load()
    check(lib.b200_dropout_add(_ptr(x), _ptr(residual), _ptr(seeds), int(seed_index), float(p), _ptr(keep),
                               _ptr(total), x.numel(), _code(x), _stream()), "b200_dropout_add")
    return keep, total
