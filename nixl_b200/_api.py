"""User-facing Python API: ``nixl_agent`` and ``nixl_agent_config``.

Method names, argument order and return conventions follow the reference's
``src/api/python/_api.py`` (``nixl_agent_config`` :148, ``nixl_agent`` :189 and the methods
listed there) so serving stacks written for it run unchanged:

* descriptors come from torch tensors (``data_ptr``, byte size, CUDA device index), from
  ``(addr, len, dev)`` tuples or from an ``N x 3`` numpy array;
* ``transfer`` / ``check_xfer_state`` return ``"DONE"``, ``"PROC"`` or ``"ERR"``;
* errors from the native layer surface as the typed exceptions of ``_bindings``;
* notifications are ``bytes``.

The default backend name ``"UCX"`` is kept for compatibility; in this library it resolves
to the NVLink backend (hand-written sm_100a copy kernels over peer-mapped memory).
"""
from __future__ import annotations

import enum
import pickle
from typing import Any, Optional, Sequence, Union

import numpy as np

from . import _bindings as nixlBind

try:  # torch is optional for pure-descriptor use
    import torch
except Exception:  # pragma: no cover
    torch = None  # type: ignore

DEFAULT_COMM_PORT = nixlBind.DEFAULT_COMM_PORT

# Opaque handle aliases (integers holding native pointers).
nixl_backend_handle = int


class nixl_thread_sync_t(enum.IntEnum):
    """Thread synchronisation modes of an agent."""

    NIXL_THREAD_SYNC_NONE = nixlBind.NIXL_THREAD_SYNC_NONE
    NIXL_THREAD_SYNC_STRICT = nixlBind.NIXL_THREAD_SYNC_STRICT
    NIXL_THREAD_SYNC_RW = nixlBind.NIXL_THREAD_SYNC_RW
    NIXL_THREAD_SYNC_DEFAULT = nixlBind.NIXL_THREAD_SYNC_DEFAULT


class nixl_agent_config:
    """Agent configuration.

    Args:
        enable_prog_thread: run backend progress threads (notifications are delivered
            without the initiator polling).
        enable_listen_thread: serve peer-to-peer metadata requests on ``listen_port``.
        listen_port: TCP port of the listener.
        capture_telemetry: record per-transfer and agent telemetry.
        num_threads: accepted for compatibility (the NVLink backend needs no worker pool).
        backends: backends to create at start-up.
        sync_mode: thread synchronisation mode; default STRICT with a listener, else NONE.
    """

    def __init__(
        self,
        enable_prog_thread: bool = True,
        enable_listen_thread: bool = False,
        listen_port: int = DEFAULT_COMM_PORT,
        capture_telemetry: bool = False,
        num_threads: int = 0,
        backends: Sequence[str] = ("UCX",),
        sync_mode: Optional[nixl_thread_sync_t] = None,
    ):
        if sync_mode is not None and not isinstance(sync_mode, nixl_thread_sync_t):
            raise TypeError(f"sync_mode must be a nixl_thread_sync_t (got {type(sync_mode).__name__!r})")
        self.backends = list(backends)
        self.enable_pthread = enable_prog_thread
        self.enable_listen = enable_listen_thread
        self.port = listen_port
        self.capture_telemetry = capture_telemetry
        self.num_threads = num_threads
        self.sync_mode = sync_mode


_MEM = {
    "DRAM": nixlBind.DRAM_SEG,
    "VRAM": nixlBind.VRAM_SEG,
    "BLOCK": nixlBind.BLK_SEG,
    "BLK": nixlBind.BLK_SEG,
    "OBJ": nixlBind.OBJ_SEG,
    "FILE": nixlBind.FILE_SEG,
    "cpu": nixlBind.DRAM_SEG,
    "cuda": nixlBind.VRAM_SEG,
}
_OPS = {"READ": nixlBind.NIXL_READ, "WRITE": nixlBind.NIXL_WRITE}


class nixl_prepped_dlist_handle(int):
    """Handle of a prepared descriptor list.  It is the native handle value (an ``int``) with
    ownership: ``release()`` frees it, and so does garbage collection if the caller forgot
    (src/api/python/_api.py:49 in the reference)."""

    def __new__(cls, agent, value: int):
        self = super().__new__(cls, int(value))
        self._agent = agent
        self._released = False
        return self

    def __repr__(self) -> str:
        return f"nixl_prepped_dlist_handle(0x{int(self):x}, released={self._released})"

    def release(self) -> None:
        if not self._released:
            self._agent.releasedDlistH(int(self))
            self._released = True

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class nixl_xfer_handle(int):
    """Handle of a transfer request (the native handle value with ownership).  ``release()`` frees
    it and raises if the backend cannot let go yet; when garbage collection hits that case the
    handle is parked on the agent and released again when the agent goes away
    (src/api/python/_api.py:89 in the reference)."""

    def __new__(cls, owner, value: int):
        self = super().__new__(cls, int(value))
        self._owner = owner  # the nixl_agent wrapper: keeps the native agent alive and holds the leak list
        self._released = False
        return self

    def __repr__(self) -> str:
        return f"nixl_xfer_handle(0x{int(self):x}, released={self._released})"

    def release(self) -> None:
        if self._released:
            return
        st = self._owner.agent.releaseXferReq(int(self))
        if st != 0:  # NIXL_SUCCESS; the literal, not the module constant: this also runs while the interpreter shuts down
            raise _error_for(st, "releaseXferReq")
        self._released = True

    def __del__(self):
        # Runs at any time, also during interpreter shutdown when module globals are already gone: nothing here
        # may fail AFTER the native release succeeded, or the handle would be parked and released a second time.
        if self._released:
            return
        self._released = True
        try:
            refused = self._owner.agent.releaseXferReq(int(self)) != 0
        except Exception:
            refused = True  # the call raises when the backend cannot let go yet: nothing was freed
        if refused:
            try:
                self._owner._leaked_xfer_handles.append(int(self))
            except Exception:
                pass


def _live(handle, what: str) -> int:
    """The native value of a handle; a handle object that was released already is refused here, in Python (its native
    object is gone, and passing the stale value on would be a use after free)."""
    if getattr(handle, "_released", False):
        raise nixlBind.nixlInvalidParamError(f"{what}: the handle was released")
    return int(handle)


def _is_tensor(x: Any) -> bool:
    return torch is not None and isinstance(x, torch.Tensor)


def _tensor_desc(t) -> tuple[int, int, int]:
    if not t.is_contiguous():
        raise ValueError("tensors passed to nixl must be contiguous")
    dev = t.get_device()
    return (t.data_ptr(), t.numel() * t.element_size(), dev if dev >= 0 else 0)


class nixl_agent:
    """A transfer endpoint.

    Args:
        agent_name: unique name of this agent.
        nixl_conf: optional :class:`nixl_agent_config`.
        instantiate_all: create every available backend plugin instead of ``nixl_conf.backends``.
    """

    def __init__(self, agent_name: str, nixl_conf: Optional[nixl_agent_config] = None, instantiate_all: bool = False):
        if nixl_conf is None:
            nixl_conf = nixl_agent_config()
        sync = nixl_conf.sync_mode
        if sync is None:
            sync = (
                nixl_thread_sync_t.NIXL_THREAD_SYNC_STRICT
                if nixl_conf.enable_listen
                else nixl_thread_sync_t.NIXL_THREAD_SYNC_NONE
            )
        cfg = nixlBind.nixlAgentConfig(
            nixl_conf.enable_pthread,
            nixl_conf.enable_listen,
            nixl_conf.port if nixl_conf.enable_listen else 0,
            int(sync),
            1,
            0,
            100000,
            nixl_conf.capture_telemetry,
        )
        self.name = agent_name
        self.agent = nixlBind.nixlAgent(agent_name, cfg)
        self.notifs: dict[str, list[bytes]] = {}
        self._leaked_xfer_handles: list[int] = []
        self.backends: dict[str, int] = {}
        self.backend_mems: dict[str, list[int]] = {}
        self.backend_options: dict[str, dict[str, str]] = {}
        self.plugin_list = self.agent.getAvailPlugins()
        self.plugin_b_options: dict[str, dict[str, str]] = {}
        self.plugin_mem_types: dict[str, list[int]] = {}
        for plugin in self.plugin_list:
            try:
                opts, mems = self.agent.getPluginParams(plugin)
            except nixlBind.nixlError:
                continue
            self.plugin_b_options[plugin] = opts
            self.plugin_mem_types[plugin] = mems

        wanted = list(self.plugin_list) if instantiate_all else nixl_conf.backends
        for name in wanted:
            init: dict[str, str] = {}
            if nixl_conf.num_threads > 0 and name in ("UCX", "OBJ", "GDS_MT"):
                init["num_threads" if name != "GDS_MT" else "thread_count"] = str(nixl_conf.num_threads)
            self.create_backend(name, init)

        self.nixl_mems = dict(_MEM)
        self.nixl_ops = dict(_OPS)

    def __del__(self):
        # Transfer handles that could not be released when they were collected get one more try.
        for h in getattr(self, "_leaked_xfer_handles", []):
            try:
                self.agent.releaseXferReq(h)
            except Exception:
                pass

    # ------------------------------------------------------------------ plugins / backends

    def get_plugin_list(self) -> list[str]:
        return self.plugin_list

    def get_plugin_mem_types(self, backend: str) -> list[str]:
        if backend not in self.plugin_mem_types:
            opts, mems = self.agent.getPluginParams(backend)
            self.plugin_b_options[backend], self.plugin_mem_types[backend] = opts, mems
        return [nixlBind.mem_type_str(m) for m in self.plugin_mem_types[backend]]

    def get_plugin_params(self, backend: str) -> dict[str, str]:
        if backend not in self.plugin_b_options:
            opts, mems = self.agent.getPluginParams(backend)
            self.plugin_b_options[backend], self.plugin_mem_types[backend] = opts, mems
        return self.plugin_b_options[backend]

    def get_backend_mem_types(self, backend: str) -> list[str]:
        return [nixlBind.mem_type_str(m) for m in self.backend_mems[backend]]

    def get_backend_params(self, backend: str) -> dict[str, str]:
        return self.backend_options[backend]

    def create_backend(self, backend: str, initParams: Optional[dict[str, str]] = None) -> None:
        handle = self.agent.createBackend(backend, dict(initParams or {}))
        self.backends[backend] = handle
        opts, mems = self.agent.getBackendParams(handle)
        self.backend_options[backend] = opts
        self.backend_mems[backend] = mems

    def _handles(self, backends: Sequence[str]) -> list[int]:
        return [self.backends[b] for b in backends]

    # ------------------------------------------------------------------ descriptors

    def _mem_type(self, mem_type: Optional[str]) -> int:
        if mem_type is None:
            raise ValueError("mem_type is required for tuple/array descriptors")
        try:
            return _MEM[mem_type]
        except KeyError:
            raise ValueError(f"unknown memory type {mem_type!r}") from None

    def get_xfer_descs(self, descs, mem_type: Optional[str] = None):
        """Build a transfer descriptor list.

        ``descs`` may be a tensor, a list of tensors (all on one device type), a list of
        ``(addr, len, dev)`` tuples, an ``N x 3`` numpy array, or an existing list object.
        """
        if isinstance(descs, nixlBind.nixlXferDList):
            return descs
        if isinstance(descs, nixlBind.nixlRegDList):
            return descs.trim()
        if _is_tensor(descs):
            descs = [descs]
        if isinstance(descs, np.ndarray):
            return nixlBind.nixlXferDList(self._mem_type(mem_type), np.ascontiguousarray(descs, dtype=np.uint64))
        descs = list(descs)
        if not descs:
            raise ValueError("empty descriptor list")
        if _is_tensor(descs[0]):
            kind = descs[0].device.type
            if any(t.device.type != kind for t in descs):
                raise ValueError("all tensors of one descriptor list must live on the same device type")
            return nixlBind.nixlXferDList(_MEM.get(kind, nixlBind.DRAM_SEG), [_tensor_desc(t) for t in descs])
        if isinstance(descs[0], tuple) and len(descs[0]) == 3:
            return nixlBind.nixlXferDList(self._mem_type(mem_type), descs)
        raise TypeError("unsupported descriptor input")

    def get_reg_descs(self, descs, mem_type: Optional[str] = None):
        """Build a registration descriptor list (same inputs; tuples are ``(addr, len, dev, meta)``)."""
        if isinstance(descs, nixlBind.nixlRegDList):
            return descs
        if _is_tensor(descs):
            descs = [descs]
        if isinstance(descs, np.ndarray):
            if descs.ndim != 2 or descs.shape[1] != 3:
                raise ValueError("descriptor array must have shape (N, 3)")
            rows = [(int(a), int(l), int(d), "") for a, l, d in descs.tolist()]
            return nixlBind.nixlRegDList(self._mem_type(mem_type), rows)
        descs = list(descs)
        if not descs:
            raise ValueError("empty descriptor list")
        if _is_tensor(descs[0]):
            kind = descs[0].device.type
            if any(t.device.type != kind for t in descs):
                raise ValueError("all tensors of one descriptor list must live on the same device type")
            return nixlBind.nixlRegDList(_MEM.get(kind, nixlBind.DRAM_SEG), [_tensor_desc(t) + ("",) for t in descs])
        if isinstance(descs[0], tuple) and len(descs[0]) in (3, 4):
            rows = [d if len(d) == 4 else d + ("",) for d in descs]
            return nixlBind.nixlRegDList(self._mem_type(mem_type), rows)
        raise TypeError("unsupported descriptor input")

    def get_remote_descs(self, descs, mem_type: Optional[str] = None):
        """Build a remote descriptor list from ``(addr, len, dev, agent_name)`` tuples."""
        if isinstance(descs, nixlBind.nixlRemoteDList):
            return descs
        return nixlBind.nixlRemoteDList(self._mem_type(mem_type), list(descs))

    def get_serialized_descs(self, descs) -> bytes:
        return pickle.dumps(descs)

    def deserialize_descs(self, serialized: bytes):
        return pickle.loads(serialized)

    # ------------------------------------------------------------------ memory

    def register_memory(self, reg_list, mem_type: Optional[str] = None, backends: Sequence[str] = ()):
        """Register memory with the backends that support it; returns the registration list."""
        reg = self.get_reg_descs(reg_list, mem_type)
        st = self.agent.registerMem(reg, self._handles(backends))
        if st != nixlBind.NIXL_SUCCESS:
            raise _error_for(st, "registerMem")
        return reg

    def deregister_memory(self, dereg_list, backends: Sequence[str] = ()) -> None:
        st = self.agent.deregisterMem(dereg_list, self._handles(backends))
        if st != nixlBind.NIXL_SUCCESS:
            raise _error_for(st, "deregisterMem")

    def query_memory(self, reg_list, backend: str, mem_type: Optional[str] = None) -> list[Optional[dict[str, str]]]:
        return self.agent.queryMem(self.get_reg_descs(reg_list, mem_type), self.backends[backend])

    def make_connection(self, remote_agent: str, backends: Sequence[str] = ()) -> None:
        st = self.agent.makeConnection(remote_agent, self._handles(backends))
        if st != nixlBind.NIXL_SUCCESS:
            raise _error_for(st, "makeConnection")

    # ------------------------------------------------------------------ transfers

    def prep_xfer_dlist(self, agent_name: str, xfer_list, mem_type: Optional[str] = None, backends: Sequence[str] = ()) -> nixl_prepped_dlist_handle:
        """Prepare one side of a transfer. ``agent_name`` "NIXL_INIT_AGENT" (or "") = local side."""
        if agent_name == "NIXL_INIT_AGENT":
            agent_name = nixlBind.NIXL_INIT_AGENT
        return nixl_prepped_dlist_handle(self.agent, self.agent.prepXferDlist(agent_name, self.get_xfer_descs(xfer_list, mem_type), self._handles(backends)))

    def estimate_xfer_cost(self, req_handle: int) -> tuple[int, int, int]:
        """(duration_us, error_margin_us, method)."""
        return self.agent.estimateXferCost(_live(req_handle, "estimate_xfer_cost"))

    def make_prepped_xfer(
        self,
        operation: str,
        local_xfer_side: int,
        local_indices,
        remote_xfer_side: int,
        remote_indices,
        notif_msg: Union[bytes, str] = b"",
        backends: Sequence[str] = (),
        skip_desc_merge: bool = False,
    ) -> nixl_xfer_handle:
        return nixl_xfer_handle(self, self.agent.makeXferReq(
            _OPS[operation],
            _live(local_xfer_side, "make_prepped_xfer (local side)"),
            local_indices,
            _live(remote_xfer_side, "make_prepped_xfer (remote side)"),
            remote_indices,
            notif_msg if notif_msg else None,
            self._handles(backends),
            skip_desc_merge,
        ))

    def initialize_xfer(
        self,
        operation: str,
        local_descs,
        remote_descs,
        remote_agent: str,
        notif_msg: Union[bytes, str] = b"",
        backends: Sequence[str] = (),
    ) -> nixl_xfer_handle:
        return nixl_xfer_handle(self, self.agent.createXferReq(
            _OPS[operation],
            self.get_xfer_descs(local_descs),
            self.get_xfer_descs(remote_descs),
            remote_agent,
            notif_msg if notif_msg else None,
            self._handles(backends),
        ))

    def transfer(self, handle: int, notif_msg: Union[bytes, str] = b"", custom_param: str = "") -> str:
        """Post the transfer. Returns "DONE", "PROC" or "ERR"."""
        try:
            st = self.agent.postXferReq(_live(handle, "transfer"), notif_msg if notif_msg else None, custom_param)
        except nixlBind.nixlError:
            return "ERR"
        return "DONE" if st == nixlBind.NIXL_SUCCESS else "PROC"

    def check_xfer_state(self, handle: int) -> str:
        try:
            st = self.agent.getXferStatus(_live(handle, "check_xfer_state"))
        except nixlBind.nixlError:
            return "ERR"
        return "DONE" if st == nixlBind.NIXL_SUCCESS else "PROC"

    def get_xfer_telemetry(self, handle: int):
        return self.agent.getXferTelemetry(_live(handle, "get_xfer_telemetry"))

    def query_xfer_backend(self, handle: int) -> str:
        b = self.agent.queryXferBackend(_live(handle, "query_xfer_backend"))
        for name, h in self.backends.items():
            if h == b:
                return name
        raise nixlBind.nixlNotFoundError("backend of the transfer is unknown to this wrapper")

    def release_xfer_handle(self, handle: int) -> None:
        if isinstance(handle, nixl_xfer_handle):
            handle.release()
            return
        st = self.agent.releaseXferReq(handle)
        if st != nixlBind.NIXL_SUCCESS:
            raise _error_for(st, "releaseXferReq")

    def release_dlist_handle(self, handle: int) -> None:
        if isinstance(handle, nixl_prepped_dlist_handle):
            handle.release()
            return
        self.agent.releasedDlistH(handle)

    # ------------------------------------------------------------------ device-side views

    def prep_mem_view(self, dlist, mem_type: Optional[str] = None, backends: Sequence[str] = ()) -> int:
        """Prepare a device-side view. Remote lists (``nixlRemoteDList``) give peer pointers."""
        if not isinstance(dlist, (nixlBind.nixlRemoteDList, nixlBind.nixlXferDList)):
            dlist = self.get_xfer_descs(dlist, mem_type)
        return self.agent.prepMemView(dlist, self._handles(backends))

    def release_mem_view(self, mvh: int) -> None:
        self.agent.releaseMemView(mvh)

    # ------------------------------------------------------------------ notifications

    def get_new_notifs(self, backends: Sequence[str] = ()) -> dict[str, list[bytes]]:
        return self.agent.getNotifs({}, self._handles(backends))

    def update_notifs(self, backends: Sequence[str] = ()) -> dict[str, list[bytes]]:
        self.notifs = self.agent.getNotifs(self.notifs, self._handles(backends))
        return self.notifs

    def check_remote_xfer_done(
        self, remote_agent_name: str, lookup_tag: bytes, backends: Sequence[str] = (), tag_is_prefix: bool = True
    ) -> bool:
        """True (and the message is consumed) if a notification from the peer matches the tag."""
        self.update_notifs(backends)
        if isinstance(lookup_tag, str):
            lookup_tag = lookup_tag.encode()
        for msg in self.notifs.get(remote_agent_name, []):
            if (tag_is_prefix and msg.startswith(lookup_tag)) or (not tag_is_prefix and lookup_tag in msg):
                self.notifs[remote_agent_name].remove(msg)
                return True
        return False

    def send_notif(self, remote_agent_name: str, notif_msg: Union[bytes, str], backend: Optional[str] = None) -> None:
        self.agent.genNotif(remote_agent_name, notif_msg, [self.backends[backend]] if backend else [])

    # ------------------------------------------------------------------ metadata

    def get_agent_metadata(self) -> bytes:
        return self.agent.getLocalMD()

    def get_partial_agent_metadata(self, descs, inc_conn_info: bool, backends: Sequence[str]) -> bytes:
        return self.agent.getLocalPartialMD(descs, inc_conn_info, self._handles(backends))

    def add_remote_agent(self, metadata: bytes) -> str:
        """Load a peer's metadata; returns its agent name."""
        name = self.agent.loadRemoteMD(metadata)
        return name.decode() if isinstance(name, bytes) else name

    def remove_remote_agent(self, agent: str) -> None:
        self.agent.invalidateRemoteMD(agent)

    def send_local_metadata(self, ip_addr: str = "", port: int = DEFAULT_COMM_PORT, label: str = "") -> None:
        self.agent.sendLocalMD(ip_addr, port, label)

    def send_partial_agent_metadata(
        self, descs, inc_conn_info: bool, backends: Sequence[str], ip_addr: str = "", port: int = DEFAULT_COMM_PORT, label: str = ""
    ) -> None:
        self.agent.sendLocalPartialMD(descs, inc_conn_info, self._handles(backends), ip_addr, port, label)

    def fetch_remote_metadata(self, remote_agent: str, ip_addr: str = "", port: int = DEFAULT_COMM_PORT, label: str = "") -> None:
        self.agent.fetchRemoteMD(remote_agent, ip_addr, port, label)

    def invalidate_local_metadata(self, ip_addr: str = "", port: int = DEFAULT_COMM_PORT) -> None:
        self.agent.invalidateLocalMD(ip_addr, port)

    def check_remote_metadata(self, remote_agent: str, descs=None) -> bool:
        if descs is None:
            descs = nixlBind.nixlXferDList(nixlBind.DRAM_SEG)
        return self.agent.checkRemoteMD(remote_agent, descs)


def _error_for(status: int, what: str) -> Exception:
    table = {
        nixlBind.NIXL_ERR_NOT_POSTED: nixlBind.nixlNotPostedError,
        nixlBind.NIXL_ERR_INVALID_PARAM: nixlBind.nixlInvalidParamError,
        nixlBind.NIXL_ERR_BACKEND: nixlBind.nixlBackendError,
        nixlBind.NIXL_ERR_NOT_FOUND: nixlBind.nixlNotFoundError,
        nixlBind.NIXL_ERR_MISMATCH: nixlBind.nixlMismatchError,
        nixlBind.NIXL_ERR_NOT_ALLOWED: nixlBind.nixlNotAllowedError,
        nixlBind.NIXL_ERR_REPOST_ACTIVE: nixlBind.nixlRepostActiveError,
        nixlBind.NIXL_ERR_UNKNOWN: nixlBind.nixlUnknownError,
        nixlBind.NIXL_ERR_NOT_SUPPORTED: nixlBind.nixlNotSupportedError,
        nixlBind.NIXL_ERR_REMOTE_DISCONNECT: nixlBind.nixlRemoteDisconnectError,
        nixlBind.NIXL_ERR_CANCELED: nixlBind.nixlCancelledError,
        nixlBind.NIXL_ERR_NO_TELEMETRY: nixlBind.nixlNoTelemetryError,
    }
    return table.get(status, nixlBind.nixlError)(f"{what}: {nixlBind.status_str(status)}")
