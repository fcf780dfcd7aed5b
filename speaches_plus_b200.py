"""Import alias: the package directory is `speaches-plus_b200/` (not a valid Python identifier),
so this module loads it under the name `speaches_plus_b200`."""
import importlib.util as _ilu
import pathlib as _pl
import sys as _sys

_dir = _pl.Path(__file__).resolve().parent / "speaches-plus_b200"
_spec = _ilu.spec_from_file_location(__name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)])
_mod = _ilu.module_from_spec(_spec)
_sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
