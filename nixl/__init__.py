"""Import names of the reference's Python package, served by :mod:`nixl_b200`.

Code written against ai-dynamo/nixl (``from nixl._api import nixl_agent, nixl_agent_config``,
``import nixl._bindings``, ``from nixl.logging import get_logger``, ``import nixl._utils``) runs
unchanged: every name below is the ``nixl_b200`` object of the same role, not a copy."""
import sys

import nixl_b200
from nixl_b200 import _api, _bindings, _utils, logging  # noqa: F401
from nixl_b200 import *  # noqa: F401,F403

for _name, _mod in (("_api", _api), ("_bindings", _bindings), ("_utils", _utils), ("logging", logging)):
    sys.modules[__name__ + "." + _name] = _mod

__all__ = getattr(nixl_b200, "__all__", [])
