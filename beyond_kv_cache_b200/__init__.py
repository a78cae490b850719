"""Import alias: the package sources live in ``beyond-kv-cache_b200/`` (a name Python
cannot import directly); this module makes them importable as ``beyond_kv_cache_b200``."""

import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "beyond-kv-cache_b200")
if not _os.path.isdir(_real):
    raise ImportError(f"package directory {_real} is missing")
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _os, _f, _real
