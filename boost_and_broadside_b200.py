"""Import shim: the package lives in the directory ``boost-and-broadside_b200/`` (not a
legal Python identifier), so this module loads it under the importable name
``boost_and_broadside_b200`` and replaces itself with the real package."""

import importlib.util
import os
import sys

_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "boost-and-broadside_b200")
_spec = importlib.util.spec_from_file_location(
    "boost_and_broadside_b200", os.path.join(_dir, "__init__.py"), submodule_search_locations=[_dir]
)
_pkg = importlib.util.module_from_spec(_spec)
sys.modules["boost_and_broadside_b200"] = _pkg
_spec.loader.exec_module(_pkg)
