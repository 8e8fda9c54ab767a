"""Installing uploaded tasklib modules: the base64 source of a module is written under a scratch
directory that mirrors its package path and imported from there (reference:
python/cornserve/services/task_registry/utils.py:12-90)."""

from __future__ import annotations

import importlib
import importlib.util
import shutil
import sys
import types
from pathlib import Path

from ...constants import TASKLIB_DIR


def tasklib_root() -> Path:
    root = Path(TASKLIB_DIR)
    root.mkdir(parents=True, exist_ok=True)
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    return root


def write_to_file_and_import(module_name: str, source: str) -> types.ModuleType:
    """Materialise ``module_name`` from ``source`` and import it.  A module that is already imported with
    identical source is returned as is, so that classes keep their identity across repeated loads."""
    existing = sys.modules.get(module_name)
    if existing is not None and getattr(existing, "__cornserve_source__", None) == source:
        return existing
    root = tasklib_root()
    parts = module_name.split(".")
    pkg_dir = root
    for p in parts[:-1]:
        pkg_dir = pkg_dir / p
        pkg_dir.mkdir(exist_ok=True)
        init = pkg_dir / "__init__.py"
        if not init.exists():
            init.write_text("")
    path = pkg_dir / f"{parts[-1]}.py"
    path.write_text(source)
    importlib.invalidate_caches()
    # packages of the uploaded tree must resolve to the scratch directory, not to an installed copy
    for i in range(1, len(parts)):
        pkg = ".".join(parts[:i])
        mod = sys.modules.get(pkg)
        pkg_path = str(root.joinpath(*parts[:i]))
        if mod is None:
            spec = importlib.util.spec_from_file_location(pkg, Path(pkg_path) / "__init__.py",
                                                          submodule_search_locations=[pkg_path])
            mod = importlib.util.module_from_spec(spec)
            sys.modules[pkg] = mod
            spec.loader.exec_module(mod)
        elif hasattr(mod, "__path__") and pkg_path not in list(mod.__path__):
            mod.__path__.append(pkg_path)
    spec = importlib.util.spec_from_file_location(module_name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[module_name] = module
    try:
        spec.loader.exec_module(module)
    except Exception:
        sys.modules.pop(module_name, None)
        raise
    module.__cornserve_source__ = source
    return module


def purge_tasklib_modules_and_delete_dir() -> None:
    root = Path(TASKLIB_DIR)
    for name, mod in list(sys.modules.items()):
        f = getattr(mod, "__file__", None)
        if f and str(root) in f:
            sys.modules.pop(name, None)
    shutil.rmtree(root, ignore_errors=True)
