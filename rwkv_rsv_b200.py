"""Import shim: the package directory is named `rwkv-rsv_b200`, which is not a Python identifier.

`import rwkv_rsv_b200` loads this module, which then behaves as that package: its `__path__` points at the
hyphenated directory and the directory's `__init__.py` is executed in this module's namespace.
"""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "rwkv-rsv_b200")]
__package__ = __name__
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__, "r") as _f:
    exec(compile(_f.read(), __file__, "exec"))
