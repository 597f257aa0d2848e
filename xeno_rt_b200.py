"""Import name of the package kept in the folder ``xeno-rt_b200/``.

The folder carries the project's name, which holds a hyphen and so cannot be
written in an ``import`` statement.  This module loads that folder as the
package ``xeno_rt_b200`` and replaces itself with it, so that
``import xeno_rt_b200.engine`` and relative imports inside the package work
as for any other package.
"""
import importlib.util as _util
import os as _os
import sys as _sys

_dir = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "xeno-rt_b200")
_spec = _util.spec_from_file_location(__name__, _os.path.join(_dir, "__init__.py"),
                                      submodule_search_locations=[_dir])
_module = _util.module_from_spec(_spec)
_sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
