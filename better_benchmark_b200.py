"""Import alias: ``import better_benchmark_b200`` loads the package directory ``better-benchmark_b200/``.

The directory name carries a hyphen, which the ``import`` statement cannot spell. This module
loads that directory's ``__init__.py`` under the name ``better_benchmark_b200`` (so there is a
single copy of the package and its sub-modules are ``better_benchmark_b200.<name>``).
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "better-benchmark_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
