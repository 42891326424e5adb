"""Import alias for the package directory ``v620-inference-engine_b200``.

The directory name carries a hyphen, so it cannot be imported by name.  This
module loads the directory's ``__init__.py`` as the package ``qwb200`` (with the
directory as its submodule search path) and replaces itself in ``sys.modules``,
so ``import qwb200.ops`` and relative imports inside the package work normally.
"""
import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "v620-inference-engine_b200")
_spec = importlib.util.spec_from_file_location(
    __name__, os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
