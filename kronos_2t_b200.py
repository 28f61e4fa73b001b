"""Import shim: the package directory is named `kronos-2t_b200`, which is not a valid Python
identifier, so `import kronos_2t_b200` loads it from that directory under this name."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kronos-2t_b200")
_spec = importlib.util.spec_from_file_location(
    "kronos_2t_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules["kronos_2t_b200"] = _mod
_spec.loader.exec_module(_mod)
