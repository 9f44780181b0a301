"""Python-side logging for the package: one ``nixl`` logger tree whose level follows the same
``NIXL_LOG_LEVEL`` variable as the native library (TRACE and DEBUG both map to ``logging.DEBUG``,
WARN to WARNING, FATAL to CRITICAL), as the reference's src/api/python/logging.py does.

    from nixl_b200.logging import get_logger
    log = get_logger(__name__)
"""
from __future__ import annotations

import logging
import os
import sys

_LEVELS = {"TRACE": logging.DEBUG, "DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARN": logging.WARNING, "WARNING": logging.WARNING,
           "ERROR": logging.ERROR, "FATAL": logging.CRITICAL}
_ROOT = "nixl"
_configured = False


def level_from_env(default: int = logging.INFO) -> int:
    """The level NIXL_LOG_LEVEL asks for; ``default`` when unset; ValueError when it names no level."""
    name = os.environ.get("NIXL_LOG_LEVEL")
    if not name:
        return default
    try:
        return _LEVELS[name.strip().upper()]
    except KeyError:
        raise ValueError(f"NIXL_LOG_LEVEL={name!r} is not one of {sorted(set(_LEVELS))}") from None


def setup_logging(force: bool = False) -> logging.Logger:
    """Installs a stdout handler on the ``nixl`` logger once and applies the level from the environment."""
    global _configured
    root = logging.getLogger(_ROOT)
    if _configured and not force:
        return root
    for h in list(root.handlers):
        if getattr(h, "_nixl_handler", False):
            root.removeHandler(h)
    handler = logging.StreamHandler(sys.stdout)
    handler.setFormatter(logging.Formatter("%(asctime)s NIXL %(levelname)-7s %(filename)s:%(lineno)d %(message)s", "%Y-%m-%d %H:%M:%S"))
    handler._nixl_handler = True
    root.addHandler(handler)
    root.propagate = False
    try:
        root.setLevel(level_from_env())
    except ValueError as e:
        root.setLevel(logging.INFO)
        root.warning("%s; keeping INFO", e)
    logging.raiseExceptions = os.environ.get("NIXL_DEBUG_LOGGING", "").lower() in ("1", "true", "yes", "on")
    _configured = True
    return root


def get_logger(name: str = "") -> logging.Logger:
    """A child of the ``nixl`` logger (``nixl.<name>``); configures the tree on first use."""
    setup_logging()
    if not name or name == _ROOT:
        return logging.getLogger(_ROOT)
    return logging.getLogger(name if name.startswith(_ROOT + ".") else f"{_ROOT}.{name}")
