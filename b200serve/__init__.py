"""Importable alias for the package directory ``intel-arc-inference-server_b200``.

The product directory carries the project's name, which contains hyphens and so
cannot be written in an ``import`` statement.  This package redirects its
submodule search path to that directory and runs its ``__init__``; every module
is therefore imported as ``b200serve.<subpackage>.<module>``.
"""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                      "intel-arc-inference-server_b200")
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _f
