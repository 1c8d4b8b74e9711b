"""Import name of the package that lives in the folder ``inf-engine_b200``.

A hyphen cannot appear in a Python import, so ``import inf_engine_b200`` loads
this one-file stand-in, which replaces itself in ``sys.modules`` with the
package read from the hyphenated folder beside it.  Submodules then import as
``inf_engine_b200.config`` and so on.
"""

import importlib.util as _util
import os as _os
import sys as _sys

_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "inf-engine_b200")
_spec = _util.spec_from_file_location(
    "inf_engine_b200", _os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_module = _util.module_from_spec(_spec)
_sys.modules["inf_engine_b200"] = _module
_spec.loader.exec_module(_module)
