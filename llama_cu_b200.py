"""Import shim: the package directory is `llama.cu_b200/` (a dot cannot appear in a
module name), so it is loaded by path and registered as `llama_cu_b200`."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama.cu_b200")
_spec = importlib.util.spec_from_file_location("llama_cu_b200", os.path.join(_dir, "__init__.py"),
                                               submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["llama_cu_b200"] = _mod
_spec.loader.exec_module(_mod)
