"""Import shim: `import sm120fp4_b200` resolves to the package directory `sm120-fp4_b200/` (a hyphen cannot appear in
a Python module name, so the directory is mounted under this importable name)."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "sm120-fp4_b200")]
__package__ = __name__
if __spec__ is not None:
    __spec__.submodule_search_locations = __path__
with open(_os.path.join(__path__[0], "__init__.py"), encoding="utf-8") as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
