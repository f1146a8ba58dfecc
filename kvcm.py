"""Import shim: makes the folder ``kv-cache-manager_b200/`` importable as the package ``kvcm``.

The product folder carries a hyphen in its name, which the ``import`` statement cannot spell.
This module loads that folder's ``__init__.py`` under the name ``kvcm`` and replaces itself in
``sys.modules``, so that ``import kvcm`` and ``from kvcm.engine import Engine`` work from the
repository root (or from anywhere once the root is on ``sys.path``).
"""
import importlib.util
import os
import sys

_PKG_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kv-cache-manager_b200")
_spec = importlib.util.spec_from_file_location(
    "kvcm", os.path.join(_PKG_DIR, "__init__.py"), submodule_search_locations=[_PKG_DIR])
_mod = importlib.util.module_from_spec(_spec)
sys.modules["kvcm"] = _mod
_spec.loader.exec_module(_mod)
