"""Import name of the reference's expert-parallel package (examples/device/ep/nixl_ep), served by
:mod:`nixl_b200.parallel`: ``nixl_ep.Buffer`` is the dispatch / combine buffer, ``nixl_ep.EventOverlap``
the event wrapper its calls return."""
from nixl_b200.parallel import *  # noqa: F401,F403
from nixl_b200.parallel import Buffer, EventOverlap  # noqa: F401
