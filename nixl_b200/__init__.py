"""nixl_b200: a Blackwell-native point-to-point transfer library with the NIXL API.

``nixl_agent`` / ``nixl_agent_config`` mirror the Python API of ai-dynamo/nixl
(``src/api/python/_api.py`` there); the native agent, the NVLink backend and the kernels
live in the shared objects built from ``csrc/`` into this package directory.
"""
import os as _os

_HERE = _os.path.dirname(_os.path.abspath(__file__))
# Plugins are looked up next to the core library; an explicit NIXL_PLUGIN_DIR still wins.
_os.environ.setdefault("NIXL_PLUGIN_DIR", _os.path.join(_HERE, "lib", "plugins"))

try:
    from . import _bindings  # noqa: F401
except ImportError as exc:  # pragma: no cover - only without a build
    raise ImportError(
        "nixl_b200 native module is not built; run `make -C csrc -j8` or "
        "`python -c 'import __graft_entry__ as g; g.build()'` from the repository root"
    ) from exc

from ._api import (  # noqa: E402,F401
    DEFAULT_COMM_PORT,
    nixl_agent,
    nixl_agent_config,
    nixl_prepped_dlist_handle,
    nixl_thread_sync_t,
    nixl_xfer_handle,
)



def add_plugin_directory(path: str) -> None:
    """Put ``path`` in front of the process-wide plug-in search path (agents created later see it)."""
    _bindings.add_plugin_directory(path)


#: Engines that answer to the names of the reference's appliance plug-ins (INFINIA, HF3FS, GDS_MT)
#: with local storage.  They are NOT clients of those services and are
#: therefore not on the default search path; ``add_plugin_directory(STANDIN_PLUGIN_DIR)`` opts in.
STANDIN_PLUGIN_DIR = _os.path.join(_HERE, "lib", "standin_plugins")

__version__ = "0.2.0"
