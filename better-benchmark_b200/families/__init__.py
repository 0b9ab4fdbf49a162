"""``oracle_forward(inputs)`` bodies, one module per repro family.

Each takes the positional input list of the repro's ``forward`` (tensors, lifted shape lists,
scalars) and returns the outputs in the eager module's order, with its shapes, dtypes and
strides, computed by the CUDA kernels in ``csrc/``. A canonical directory's ``oracle.py`` is a
registration stub around one of these.
"""
