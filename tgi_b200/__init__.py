"""Import alias for the framework package.

The framework's sources live in the directory ``text-generation-inference_b200/``
whose name is not a valid Python identifier.  This module makes them importable
as ``tgi_b200`` (``import tgi_b200.models`` resolves inside that directory) by
pointing the package search path at it and executing its ``__init__``.
"""
import os as _os

_real = _os.path.normpath(
    _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "..", "text-generation-inference_b200")
)
__path__ = [_real]
__file__ = _os.path.join(_real, "__init__.py")
with open(__file__, "r") as _f:
    exec(compile(_f.read(), __file__, "exec"), globals())
del _f, _os
