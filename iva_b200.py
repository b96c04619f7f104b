"""Import alias for the package directory ``iva1.0_b200/``.

A directory name with a dot in it cannot be named in an ``import`` statement,
so this module loads that directory as the package ``iva_b200`` and replaces
itself in ``sys.modules``.  After ``import iva_b200`` every submodule is
reachable as ``iva_b200.<name>``.
"""

import importlib.util
import os
import sys

_PKG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "iva1.0_b200")
_spec = importlib.util.spec_from_file_location(
    "iva_b200",
    os.path.join(_PKG_DIR, "__init__.py"),
    submodule_search_locations=[_PKG_DIR],
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules["iva_b200"] = _mod
_spec.loader.exec_module(_mod)
