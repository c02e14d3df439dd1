"""Import name for the package directory ``cuda-llm_b200/``.

The directory name carries a hyphen, which Python cannot import directly; this
module loads it under the name ``cuda_llm_b200`` (sub-modules included).
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cuda-llm_b200")
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_dir, "__init__.py"),
                                               submodule_search_locations=[_dir])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
