"""Import name of the package whose sources live in the folder `catena-models_b200/`.

A folder name with a hyphen cannot be imported, so this module points its search path at
that folder and runs the folder's own `__init__.py`; `catena_models_b200.config`,
`catena_models_b200.engine` and the other sub-packages are found there.
"""
import os as _os

_SRC = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "catena-models_b200")
__path__.insert(0, _SRC)
with open(_os.path.join(_SRC, "__init__.py")) as _fh:
    exec(compile(_fh.read(), _os.path.join(_SRC, "__init__.py"), "exec"))
del _fh
