"""Minimum-bytes (speed-of-light) model of a fused region.

Same accounting rules as the reference's ``byte_accounting.count_bytes_effective``
(``byte_accounting.py:54-66`` and ``:142-293``), restated with a single table of tensor records:

  * every external input is charged once, by the largest portion of it that any op actually
    reads (a view or slice charges the narrowed portion, never more than the whole tensor);
  * a sparse source (embedding / gather / index / index_select / take) charges the bytes of the
    gathered result instead of the whole table;
  * every distinct output tensor is charged once, unless it is an input returned unchanged;
    outputs of index_put / scatter are charged by the bytes they update;
  * intermediates cost nothing: a fused kernel never writes them.

The byte count of a kernel launch divided by its duration is the "achieved GB/s" the benchmark
reports, and the same count over the measured HBM bandwidth is its speed-of-light time.
"""
from __future__ import annotations

import torch
from torch.utils import _pytree
from torch.utils._python_dispatch import TorchDispatchMode

VIEW_OPS = {
    "aten.alias.default", "aten.as_strided.default", "aten.detach.default", "aten.expand.default",
    "aten.flatten.using_ints", "aten.permute.default", "aten.reshape.default", "aten.select.int",
    "aten.slice.Tensor", "aten.squeeze.default", "aten.squeeze.dim", "aten.t.default",
    "aten.transpose.int", "aten.unsqueeze.default", "aten.view.default", "aten._unsafe_view.default",
}
SPARSE_SOURCE_OPS = {
    "aten.embedding.default", "aten.gather.default", "aten.index.Tensor",
    "aten.index_select.default", "aten.take.default",
}


def tensor_nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _tensors(values):
    return [v for v in _pytree.tree_leaves(values) if isinstance(v, torch.Tensor)]


def _alias_key(t: torch.Tensor):
    try:
        ptr = t.untyped_storage().data_ptr()
    except RuntimeError:
        ptr = t.data_ptr()
    return (ptr, t.storage_offset(), t.nelement(), t.element_size())


def unique_bytes(values) -> int:
    seen, total = set(), 0
    for t in _tensors(values):
        key = _alias_key(t)
        if key not in seen:
            seen.add(key)
            total += tensor_nbytes(t)
    return total


def count_bytes_naive(inputs, outputs) -> int:
    """All tensor inputs plus unique outputs (``byte_accounting.py:49-51``)."""
    return sum(tensor_nbytes(t) for t in _tensors(inputs)) + unique_bytes(outputs)


class _Counter(TorchDispatchMode):
    def __init__(self):
        super().__init__()
        self.alive = []          # keeps ids stable for the lifetime of the count
        self.produced = set()    # ids of tensors created inside the region
        self.parent = {}         # view id -> id of the tensor it views
        self.inputs = {}         # root id -> {"size", "dense", "dense_read", "sparse"}
        self.sparse_out = {}     # id of a sparse-update result -> bytes written

    def _root(self, tid):
        seen = set()
        while tid in self.parent and tid not in seen:
            seen.add(tid)
            tid = self.parent[tid]
        return tid

    def _note_input(self, t):
        rid = self._root(id(t))
        if rid not in self.produced and rid not in self.inputs:
            self.inputs[rid] = {"size": tensor_nbytes(t), "dense": False, "dense_read": 0, "sparse": 0}

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        name = str(func)
        operands = _tensors((args, kwargs))
        for t in operands:
            self._note_input(t)
        result = func(*args, **kwargs)
        results = _tensors(result)
        self.alive.extend(results)
        for t in results:
            self.produced.add(id(t))

        first = args[0] if args and isinstance(args[0], torch.Tensor) else None
        if name in VIEW_OPS and first is not None:
            for t in results:
                self.parent[id(t)] = self._root(id(first))
            return result

        skip = set()
        if name in SPARSE_SOURCE_OPS and first is not None:
            skip.add(id(first))
            self._sparse_read(first, unique_bytes(result))
        if name.startswith(("aten.scatter.", "aten.scatter_add.", "aten.scatter_reduce.")):
            written = self._scatter_bytes(args, result)
            if len(args) >= 4 and isinstance(args[3], torch.Tensor):
                skip.add(id(args[3]))
                self._sparse_read(args[3], written)
            for t in results:
                self.sparse_out[id(t)] = written
        if name == "aten.index_put.default":
            values = args[2] if len(args) >= 3 else None
            written = (min(tensor_nbytes(values), unique_bytes(result))
                       if isinstance(values, torch.Tensor) else unique_bytes(result))
            if isinstance(values, torch.Tensor):
                skip.add(id(values))
                self._sparse_read(values, written)
            for t in results:
                self.sparse_out[id(t)] = written
        for t in operands:
            if id(t) in skip:
                continue
            rec = self.inputs.get(self._root(id(t)))
            if rec is not None:
                rec["dense"] = True
                rec["dense_read"] = max(rec["dense_read"], tensor_nbytes(t))
        return result

    def _sparse_read(self, t, nbytes):
        rec = self.inputs.get(self._root(id(t)))
        if rec is not None:
            rec["sparse"] += nbytes

    @staticmethod
    def _scatter_bytes(args, result):
        if len(args) >= 4 and isinstance(args[3], torch.Tensor):
            return min(tensor_nbytes(args[3]), unique_bytes(result))
        index = args[2] if len(args) >= 3 else None
        if isinstance(index, torch.Tensor):
            outs = _tensors(result)
            elem = outs[0].element_size() if outs else 1
            return min(index.numel() * elem, unique_bytes(result))
        return unique_bytes(result)

    def total(self, outputs) -> int:
        read = 0
        for rec in self.inputs.values():
            read += min(rec["dense_read"], rec["size"]) if rec["dense"] else min(rec["sparse"], rec["size"])
        written, seen = 0, set()
        for t in _tensors(outputs):
            key = _alias_key(t)
            if key in seen:
                continue
            seen.add(key)
            if self._root(id(t)) in self.inputs and id(t) not in self.produced:
                continue  # an input handed back untouched
            if id(t) in self.sparse_out:
                written += min(self.sparse_out[id(t)], tensor_nbytes(t))
            else:
                written += tensor_nbytes(t)
        return read + written


def count_bytes_effective(mod, inputs) -> int:
    """Minimum bytes a fused implementation of ``mod(*inputs)`` must move."""
    with _Counter() as counter:
        with torch.no_grad():
            outputs = mod(*inputs)
    return counter.total(outputs)
