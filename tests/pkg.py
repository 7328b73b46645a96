"""The package directory `x-deeplearning_b200` is not a valid Python identifier: the loader that imports it
under the module name x_deeplearning_b200 lives in __graft_entry__.py at the repository root."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from __graft_entry__ import load_package as load  # noqa: E402,F401
