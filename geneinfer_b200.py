"""Import name of the engine package.

The package lives in the folder ``gene-llm-inference-engine_b200`` whose name is not a valid
Python identifier; this module loads that folder as the package ``geneinfer_b200`` so that
``import geneinfer_b200`` and ``from geneinfer_b200.cache import CacheManager`` work from the
repository root.
"""
import importlib.util as _util
import os as _os
import sys as _sys

_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "gene-llm-inference-engine_b200")
_spec = _util.spec_from_file_location(
    __name__, _os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir])
_mod = _util.module_from_spec(_spec)
_sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
