"""Import alias for the package directory ``tessweave-engine_b200/``.

A Python identifier cannot hold a hyphen, so the package is imported as
``tessweave_engine_b200``.  This module turns itself into that package: it
points ``__path__`` at the hyphenated directory and runs the directory's
``__init__.py`` in its own namespace, so ``tessweave_engine_b200.cache`` and
relative imports inside the package resolve as for any ordinary package.
"""
import os as _os

_PKG_DIR = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "tessweave-engine_b200")
__path__ = [_PKG_DIR]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
__file__ = _os.path.join(_PKG_DIR, "__init__.py")
with open(__file__, "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f
