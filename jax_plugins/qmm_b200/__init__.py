"""JAX plugin package of the B200 quantized-matmul backend.

JAX discovers a PJRT plugin through the ``jax_plugins`` entry-point group and the ``jax_plugins``
namespace package and calls ``initialize()``.  This mirrors the reference's plugin package
(src/jax_plugins/silicon/__init__.py:147-202, entry point in its pyproject.toml:30-31): find the
shared library, check the jaxlib series, switch off the shardy partitioner (its ``sdy`` ops are not
StableHLO the reader understands) and register the backend with
``xla_bridge.register_plugin(name, priority=500, library_path=..., options={})``.

Two things differ from the reference.  There is no platform check (the reference refuses anything
but darwin).  And registration needs the library to export ``GetPjrtApi``: that table is compiled
only where the PJRT C API header of jaxlib is available at build time, so ``initialize()`` looks
for the symbol first and raises a :class:`QmmPluginError` that says so, instead of letting jaxlib
fail on ``dlsym``.  The operator API (``jax_metallib_b200.quantized``) and the runtime layer
(``jax_metallib_b200.runtime``) do not need the plugin registration.
"""

from __future__ import annotations

import ctypes
import logging
import os
import warnings
from pathlib import Path

_logger = logging.getLogger(__name__)

PLATFORM_NAME = "qmm_b200"
_BUILT_FOR_JAXLIB = (0, 11)  # the jaxlib series the reference targets (its pyproject.toml:9-10)
_LIB_NAME = "libqmm.so"
_LIBRARY_ENV = "QMM_LIBRARY_PATH"


class QmmPluginError(Exception):
    """Raised when the plugin cannot be initialised."""


def _search_paths():
    pkg = Path(__file__).resolve().parent
    root = pkg.parent.parent
    return [
        (pkg / _LIB_NAME, "plugin package directory"),
        (pkg / "lib" / _LIB_NAME, "plugin package lib/ (wheel install)"),
        (root / "jax_metallib_b200" / _LIB_NAME, "jax_metallib_b200/ of the source tree (in-tree build)"),
    ]


def _is_file(path) -> bool:
    try:
        return Path(path).is_file()
    except (OSError, ValueError):
        return False


def find_library():
    """Path of ``libqmm.so``: ``QMM_LIBRARY_PATH`` first, then the package and the source tree."""
    env = os.environ.get(_LIBRARY_ENV)
    if env is not None:
        if _is_file(env):
            return env
        warnings.warn(f"{_LIBRARY_ENV} is set to '{env}', but that is not a file.", stacklevel=2)
    for path, _ in _search_paths():
        if _is_file(path):
            return str(path)
    try:  # the installed kernel package knows where its library lives
        from jax_metallib_b200 import _lib

        if _is_file(_lib.LIB_PATH):
            return _lib.LIB_PATH
    except Exception:  # noqa: BLE001
        pass
    return None


def _check_jaxlib_version():
    try:
        import jaxlib

        parts = getattr(jaxlib, "__version__", "").split(".")
        if len(parts) >= 2 and (int(parts[0]), int(parts[1])) != _BUILT_FOR_JAXLIB:
            warnings.warn(
                f"the {PLATFORM_NAME} plugin targets jaxlib {_BUILT_FOR_JAXLIB[0]}.{_BUILT_FOR_JAXLIB[1]}.x but jaxlib "
                f"{jaxlib.__version__} is installed; the PJRT C API version or the printed StableHLO may differ.",
                stacklevel=2)
    except Exception:  # noqa: BLE001 - the check is advisory
        pass


def exports_pjrt_api(library_path: str) -> bool:
    """Whether the library was built with the PJRT table (``GetPjrtApi``)."""
    try:
        lib = ctypes.CDLL(library_path, mode=ctypes.RTLD_LOCAL)
    except OSError as e:
        raise QmmPluginError(f"cannot load {library_path}: {e}") from e
    return hasattr(lib, "GetPjrtApi")


def _mark_backend_nonexperimental(xb, name):
    try:
        factory = xb._backends[name]
        if hasattr(factory, "options"):
            factory.options["available"] = True
    except (KeyError, TypeError, AttributeError):
        pass


def initialize():
    """Called by JAX's plugin discovery: register the backend under ``JAX_PLATFORMS=qmm_b200``."""
    _check_jaxlib_version()
    library_path = find_library()
    if library_path is None:
        searched = "\n".join(f"  - {desc}: {path}" for path, desc in _search_paths())
        raise QmmPluginError(f"Could not find {_LIB_NAME}. Searched:\n{searched}\nYou can also set {_LIBRARY_ENV}.")
    if not exports_pjrt_api(library_path):
        raise QmmPluginError(
            f"{library_path} does not export GetPjrtApi: the PJRT table is built only where jaxlib's PJRT C API "
            "header (xla/pjrt/c/pjrt_c_api.h) is present at build time. The kernels, the StableHLO planner and the "
            "runtime layer (include/qmm_rt.h) are usable without it.")
    try:
        import jax

        jax.config.update("jax_use_shardy_partitioner", False)
    except Exception as e:  # noqa: BLE001
        warnings.warn(f"Failed to disable the shardy partitioner: {e}. Sharded programs may not compile.", stacklevel=2)
    try:
        from jax._src import xla_bridge as xb
    except ImportError as e:
        raise QmmPluginError(f"Failed to import JAX xla_bridge: {e}") from e
    if not hasattr(xb, "register_plugin"):
        raise QmmPluginError("This JAX version does not support the register_plugin API.")
    try:
        _mark_backend_nonexperimental(xb, PLATFORM_NAME)
        xb.register_plugin(PLATFORM_NAME, priority=500, library_path=library_path, options={})
    except Exception as e:  # noqa: BLE001
        raise QmmPluginError(f"Failed to register the {PLATFORM_NAME} plugin: {e}") from e
