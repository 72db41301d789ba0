"""Import shim: the package directory is named after the project
(`emel.cpp_b200/`), which is not a valid Python module name; this file makes it
importable as `emel_cpp_b200`."""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "emel.cpp_b200")
_spec = importlib.util.spec_from_file_location(
    "emel_cpp_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["emel_cpp_b200"] = _mod
_spec.loader.exec_module(_mod)
