"""Import alias for the package folder ``hf.cpu_b200``.

The folder carries the project's name, which is not a valid Python identifier
(it holds a dot), so ``import hfcpu_b200`` loads it under this name instead.
After the import, ``sys.modules["hfcpu_b200"]`` is the package itself and
``hfcpu_b200.config`` and the other sub-packages resolve inside that folder.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hf.cpu_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
