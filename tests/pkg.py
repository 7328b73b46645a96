"""Imports the package directory `x-deeplearning_b200` (not a valid Python identifier)
under the module name x_deeplearning_b200."""
import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load():
    name = "x_deeplearning_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "x-deeplearning_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(path, "__init__.py"),
                                                  submodule_search_locations=[path])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod
