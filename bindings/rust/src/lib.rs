//! Safe Rust wrappers over the C API of nixl_b200 (`csrc/include/nixl_capi.h`).
//!
//! Role of the reference's `src/bindings/rust` crate: an `Agent` that owns backends, registers
//! memory, exchanges metadata, builds and posts transfer requests and reads notifications.  The
//! C API is the same 1:1 surface the reference's `wrapper.h` declares, so the types below map
//! onto it directly: every handle type owns its C object and destroys it on drop.

pub mod sys;

use std::ffi::{CStr, CString};
use std::fmt;
use std::os::raw::{c_char, c_void};
use std::ptr;

/// Error codes of the C API (`nixl_capi_status_t` below zero).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum NixlError {
    InvalidParam,
    Backend,
    InvalidState,
    Exception,
    NoTelemetry,
    NotFound,
    /// A Rust string with an interior NUL could not be passed to C.
    BadString,
    Unknown(i32),
}

impl fmt::Display for NixlError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "{:?}", self)
    }
}

impl std::error::Error for NixlError {}

pub type Result<T> = std::result::Result<T, NixlError>;

/// State of a posted transfer.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum XferStatus {
    Done,
    InProgress,
}

fn check(status: sys::nixl_capi_status_t) -> Result<XferStatus> {
    match status {
        sys::NIXL_CAPI_SUCCESS => Ok(XferStatus::Done),
        sys::NIXL_CAPI_IN_PROG => Ok(XferStatus::InProgress),
        sys::NIXL_CAPI_ERROR_INVALID_PARAM => Err(NixlError::InvalidParam),
        sys::NIXL_CAPI_ERROR_BACKEND => Err(NixlError::Backend),
        sys::NIXL_CAPI_ERROR_INVALID_STATE => Err(NixlError::InvalidState),
        sys::NIXL_CAPI_ERROR_EXCEPTION => Err(NixlError::Exception),
        sys::NIXL_CAPI_ERROR_NO_TELEMETRY => Err(NixlError::NoTelemetry),
        sys::NIXL_CAPI_ERROR_NOT_FOUND => Err(NixlError::NotFound),
        other => Err(NixlError::Unknown(other)),
    }
}

fn cstring(s: &str) -> Result<CString> {
    CString::new(s).map_err(|_| NixlError::BadString)
}

/// Memory segment kinds (`nixl_mem_t`).
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum MemType {
    Dram = 0,
    Vram = 1,
    Block = 2,
    Object = 3,
    File = 4,
    Unknown = 5,
}

impl MemType {
    fn from_raw(v: i32) -> MemType {
        match v {
            0 => MemType::Dram,
            1 => MemType::Vram,
            2 => MemType::Block,
            3 => MemType::Object,
            4 => MemType::File,
            _ => MemType::Unknown,
        }
    }
}

/// Direction of a transfer.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum XferOp {
    Read = 0,
    Write = 1,
}

/// Thread synchronisation policy of an agent.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
#[repr(i32)]
pub enum ThreadSync {
    None = 0,
    Strict = 1,
    Rw = 2,
}

/// Agent configuration (`nixlAgentConfig`).
#[derive(Debug, Clone)]
pub struct AgentConfig {
    pub enable_prog_thread: bool,
    pub enable_listen_thread: bool,
    pub listen_port: i32,
    pub thread_sync: ThreadSync,
    pub num_workers: u32,
    pub pthr_delay_us: u64,
    pub lthr_delay_us: u64,
    pub capture_telemetry: bool,
}

impl Default for AgentConfig {
    fn default() -> Self {
        AgentConfig {
            enable_prog_thread: true,
            enable_listen_thread: false,
            listen_port: 0,
            thread_sync: ThreadSync::None,
            num_workers: 1,
            pthr_delay_us: 0,
            lthr_delay_us: 100_000,
            capture_telemetry: false,
        }
    }
}

/// Key/value parameters of a backend.
pub struct Params {
    raw: sys::nixl_capi_params_t,
}

impl Params {
    pub fn new() -> Result<Params> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_params(&mut raw) })?;
        Ok(Params { raw })
    }

    pub fn set(&mut self, key: &str, value: &str) -> Result<()> {
        let (k, v) = (cstring(key)?, cstring(value)?);
        check(unsafe { sys::nixl_capi_params_add(self.raw, k.as_ptr(), v.as_ptr()) }).map(|_| ())
    }

    pub fn is_empty(&self) -> Result<bool> {
        let mut empty = false;
        check(unsafe { sys::nixl_capi_params_is_empty(self.raw, &mut empty) })?;
        Ok(empty)
    }

    /// All pairs, in the C API's iteration order.
    pub fn to_vec(&self) -> Result<Vec<(String, String)>> {
        let mut out = Vec::new();
        if self.is_empty()? {
            return Ok(out);
        }
        let mut it = ptr::null_mut();
        check(unsafe { sys::nixl_capi_params_create_iterator(self.raw, &mut it) })?;
        loop {
            let (mut k, mut v): (*const c_char, *const c_char) = (ptr::null(), ptr::null());
            let mut more = false;
            let st = unsafe { sys::nixl_capi_params_iterator_next(it, &mut k, &mut v, &mut more) };
            if st != sys::NIXL_CAPI_SUCCESS || k.is_null() {
                break;
            }
            let key = unsafe { CStr::from_ptr(k) }.to_string_lossy().into_owned();
            let val = if v.is_null() { String::new() } else { unsafe { CStr::from_ptr(v) }.to_string_lossy().into_owned() };
            out.push((key, val));
            if !more {
                break;
            }
        }
        unsafe { sys::nixl_capi_params_destroy_iterator(it) };
        Ok(out)
    }
}

impl Drop for Params {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_destroy_params(self.raw) };
    }
}

/// A backend created on an agent.  Valid while its agent lives.
pub struct Backend {
    raw: sys::nixl_capi_backend_t,
}

impl Drop for Backend {
    fn drop(&mut self) {
        // Frees the handle object only; the engine belongs to the agent.
        unsafe { sys::nixl_capi_destroy_backend(self.raw) };
    }
}

/// Optional arguments of agent calls (`nixl_opt_args_t`).
pub struct OptArgs {
    raw: sys::nixl_capi_opt_args_t,
}

impl OptArgs {
    pub fn new() -> Result<OptArgs> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_opt_args(&mut raw) })?;
        Ok(OptArgs { raw })
    }

    pub fn add_backend(&mut self, backend: &Backend) -> Result<()> {
        check(unsafe { sys::nixl_capi_opt_args_add_backend(self.raw, backend.raw) }).map(|_| ())
    }

    /// Notification delivered to the target once the transfer is complete.
    pub fn set_notification(&mut self, msg: &[u8]) -> Result<()> {
        check(unsafe { sys::nixl_capi_opt_args_set_notif_msg(self.raw, msg.as_ptr() as *const c_void, msg.len()) })?;
        check(unsafe { sys::nixl_capi_opt_args_set_has_notif(self.raw, true) }).map(|_| ())
    }

    pub fn set_skip_desc_merge(&mut self, skip: bool) -> Result<()> {
        check(unsafe { sys::nixl_capi_opt_args_set_skip_desc_merge(self.raw, skip) }).map(|_| ())
    }

    /// Peer address for the socket metadata exchange.
    pub fn set_peer(&mut self, ip: &str, port: u16) -> Result<()> {
        let ip = cstring(ip)?;
        check(unsafe { sys::nixl_capi_opt_args_set_ip_addr(self.raw, ip.as_ptr()) })?;
        check(unsafe { sys::nixl_capi_opt_args_set_port(self.raw, port) }).map(|_| ())
    }
}

impl Drop for OptArgs {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_destroy_opt_args(self.raw) };
    }
}

fn opt_raw(o: Option<&OptArgs>) -> sys::nixl_capi_opt_args_t {
    o.map(|a| a.raw).unwrap_or(ptr::null_mut())
}

/// Descriptor list for registration: (address or offset, length, device id, metadata string).
pub struct RegDescList {
    raw: sys::nixl_capi_reg_dlist_t,
}

impl RegDescList {
    pub fn new(mem: MemType) -> Result<RegDescList> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_reg_dlist(mem as i32, &mut raw) })?;
        Ok(RegDescList { raw })
    }

    pub fn add(&mut self, addr: usize, len: usize, dev_id: u64, meta: &[u8]) -> Result<()> {
        check(unsafe { sys::nixl_capi_reg_dlist_add_desc(self.raw, addr, len, dev_id, meta.as_ptr() as *const c_void, meta.len()) }).map(|_| ())
    }

    /// Registers the bytes of a slice that the caller keeps alive (and in place) while registered.
    pub fn add_slice<T>(&mut self, data: &[T], dev_id: u64) -> Result<()> {
        self.add(data.as_ptr() as usize, std::mem::size_of_val(data), dev_id, &[])
    }

    pub fn len(&self) -> Result<usize> {
        let mut n = 0usize;
        check(unsafe { sys::nixl_capi_reg_dlist_desc_count(self.raw, &mut n) })?;
        Ok(n)
    }

    pub fn mem_type(&self) -> Result<MemType> {
        let mut t = 0i32;
        check(unsafe { sys::nixl_capi_reg_dlist_get_type(self.raw, &mut t) })?;
        Ok(MemType::from_raw(t))
    }

    pub fn clear(&mut self) -> Result<()> {
        check(unsafe { sys::nixl_capi_reg_dlist_clear(self.raw) }).map(|_| ())
    }
}

impl Drop for RegDescList {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_destroy_reg_dlist(self.raw) };
    }
}

/// Descriptor list of a transfer: (address or offset, length, device id).
pub struct XferDescList {
    raw: sys::nixl_capi_xfer_dlist_t,
}

impl XferDescList {
    pub fn new(mem: MemType) -> Result<XferDescList> {
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_xfer_dlist(mem as i32, &mut raw) })?;
        Ok(XferDescList { raw })
    }

    pub fn add(&mut self, addr: usize, len: usize, dev_id: u64) -> Result<()> {
        check(unsafe { sys::nixl_capi_xfer_dlist_add_desc(self.raw, addr, len, dev_id) }).map(|_| ())
    }

    pub fn add_slice<T>(&mut self, data: &[T], dev_id: u64) -> Result<()> {
        self.add(data.as_ptr() as usize, std::mem::size_of_val(data), dev_id)
    }

    pub fn len(&self) -> Result<usize> {
        let mut n = 0usize;
        check(unsafe { sys::nixl_capi_xfer_dlist_desc_count(self.raw, &mut n) })?;
        Ok(n)
    }

    /// Sum of the descriptors' lengths in bytes.
    pub fn total_bytes(&self) -> Result<usize> {
        let mut n = 0usize;
        check(unsafe { sys::nixl_capi_xfer_dlist_len(self.raw, &mut n) })?;
        Ok(n)
    }

    pub fn clear(&mut self) -> Result<()> {
        check(unsafe { sys::nixl_capi_xfer_dlist_clear(self.raw) }).map(|_| ())
    }
}

impl Drop for XferDescList {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_destroy_xfer_dlist(self.raw) };
    }
}

/// A descriptor list prepared on one side of a transfer (`prepXferDlist`).
pub struct PreparedDescList<'a> {
    agent: &'a Agent,
    raw: sys::nixl_capi_xfer_dlist_handle_t,
}

impl Drop for PreparedDescList<'_> {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_release_xfer_dlist_handle(self.agent.raw, self.raw) };
    }
}

/// A transfer request.  Released on drop (the agent aborts it first if it is still in flight).
pub struct XferRequest<'a> {
    agent: &'a Agent,
    raw: sys::nixl_capi_xfer_req_t,
}

/// Timings of one finished transfer (agents created with `capture_telemetry`).
#[derive(Debug, Clone, Copy, Default)]
pub struct XferTelemetry {
    pub start_time_us: u64,
    pub post_duration_us: u64,
    pub xfer_duration_us: u64,
    pub total_bytes: u64,
    pub desc_count: u64,
}

impl XferRequest<'_> {
    /// Posts (or re-posts) the request.
    pub fn post(&self, opt: Option<&OptArgs>) -> Result<XferStatus> {
        check(unsafe { sys::nixl_capi_post_xfer_req(self.agent.raw, self.raw, opt_raw(opt)) })
    }

    pub fn status(&self) -> Result<XferStatus> {
        check(unsafe { sys::nixl_capi_get_xfer_status(self.agent.raw, self.raw) })
    }

    /// Polls until the transfer is done or failed.
    pub fn wait(&self) -> Result<()> {
        loop {
            match self.status()? {
                XferStatus::Done => return Ok(()),
                XferStatus::InProgress => std::hint::spin_loop(),
            }
        }
    }

    /// The backend's estimate for this request: (duration, error margin) in microseconds.
    pub fn estimate_cost(&self, opt: Option<&OptArgs>) -> Result<(i64, i64)> {
        let (mut dur, mut err, mut method) = (0i64, 0i64, 0i32);
        check(unsafe { sys::nixl_capi_estimate_xfer_cost(self.agent.raw, self.raw, opt_raw(opt), &mut dur, &mut err, &mut method) })?;
        Ok((dur, err))
    }

    pub fn telemetry(&self) -> Result<XferTelemetry> {
        let mut t = sys::nixl_capi_xfer_telemetry_s::default();
        check(unsafe { sys::nixl_capi_get_xfer_telemetry(self.agent.raw, self.raw, &mut t) })?;
        Ok(XferTelemetry {
            start_time_us: t.start_time_us,
            post_duration_us: t.post_duration_us,
            xfer_duration_us: t.xfer_duration_us,
            total_bytes: t.total_bytes,
            desc_count: t.desc_count,
        })
    }
}

impl Drop for XferRequest<'_> {
    fn drop(&mut self) {
        unsafe {
            sys::nixl_capi_release_xfer_req(self.agent.raw, self.raw);
            sys::nixl_capi_destroy_xfer_req(self.raw);
        }
    }
}

/// Notifications received so far, per sending agent.
pub type Notifications = Vec<(String, Vec<Vec<u8>>)>;

/// A transfer agent (`nixlAgent`).
pub struct Agent {
    raw: sys::nixl_capi_agent_t,
    name: String,
}

// The C++ agent serialises its own state according to the configured thread-sync policy.
unsafe impl Send for Agent {}

impl Agent {
    pub fn new(name: &str) -> Result<Agent> {
        let cname = cstring(name)?;
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_agent(cname.as_ptr(), &mut raw) })?;
        Ok(Agent { raw, name: name.to_string() })
    }

    pub fn with_config(name: &str, cfg: &AgentConfig) -> Result<Agent> {
        let cname = cstring(name)?;
        let c = sys::nixl_capi_agent_config_t {
            enable_prog_thread: cfg.enable_prog_thread,
            enable_listen_thread: cfg.enable_listen_thread,
            listen_port: cfg.listen_port,
            thread_sync: cfg.thread_sync as i32,
            num_workers: cfg.num_workers,
            pthr_delay_us: cfg.pthr_delay_us,
            lthr_delay_us: cfg.lthr_delay_us,
            capture_telemetry: cfg.capture_telemetry,
        };
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_configured_agent(cname.as_ptr(), &c, &mut raw) })?;
        Ok(Agent { raw, name: name.to_string() })
    }

    pub fn name(&self) -> &str {
        &self.name
    }

    /// Names of the backend plug-ins that can be created.
    pub fn available_plugins(&self) -> Result<Vec<String>> {
        let mut list = ptr::null_mut();
        check(unsafe { sys::nixl_capi_get_available_plugins(self.raw, &mut list) })?;
        let mut n = 0usize;
        let mut out = Vec::new();
        if unsafe { sys::nixl_capi_string_list_size(list, &mut n) } == sys::NIXL_CAPI_SUCCESS {
            for i in 0..n {
                let mut s: *const c_char = ptr::null();
                if unsafe { sys::nixl_capi_string_list_get(list, i, &mut s) } == sys::NIXL_CAPI_SUCCESS && !s.is_null() {
                    out.push(unsafe { CStr::from_ptr(s) }.to_string_lossy().into_owned());
                }
            }
        }
        unsafe { sys::nixl_capi_destroy_string_list(list) };
        Ok(out)
    }

    /// Default parameters and supported memory kinds of a plug-in.
    pub fn plugin_params(&self, plugin: &str) -> Result<(Vec<MemType>, Params)> {
        let p = cstring(plugin)?;
        let (mut mems, mut params) = (ptr::null_mut(), ptr::null_mut());
        check(unsafe { sys::nixl_capi_get_plugin_params(self.raw, p.as_ptr(), &mut mems, &mut params) })?;
        Ok((take_mem_list(mems), Params { raw: params }))
    }

    pub fn create_backend(&self, plugin: &str, params: &Params) -> Result<Backend> {
        let p = cstring(plugin)?;
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_backend(self.raw, p.as_ptr(), params.raw, &mut raw) })?;
        Ok(Backend { raw })
    }

    pub fn backend_params(&self, backend: &Backend) -> Result<(Vec<MemType>, Params)> {
        let (mut mems, mut params) = (ptr::null_mut(), ptr::null_mut());
        check(unsafe { sys::nixl_capi_get_backend_params(self.raw, backend.raw, &mut mems, &mut params) })?;
        Ok((take_mem_list(mems), Params { raw: params }))
    }

    pub fn register_memory(&self, descs: &RegDescList, opt: Option<&OptArgs>) -> Result<()> {
        check(unsafe { sys::nixl_capi_register_mem(self.raw, descs.raw, opt_raw(opt)) }).map(|_| ())
    }

    pub fn deregister_memory(&self, descs: &RegDescList, opt: Option<&OptArgs>) -> Result<()> {
        check(unsafe { sys::nixl_capi_deregister_mem(self.raw, descs.raw, opt_raw(opt)) }).map(|_| ())
    }

    /// This agent's metadata blob, to be handed to peers.
    pub fn local_metadata(&self) -> Result<Vec<u8>> {
        let (mut data, mut len): (*mut c_void, usize) = (ptr::null_mut(), 0);
        check(unsafe { sys::nixl_capi_get_local_md(self.raw, &mut data, &mut len) })?;
        Ok(take_malloced(data, len))
    }

    /// Metadata restricted to `descs` (empty list: connection information only).
    pub fn local_partial_metadata(&self, descs: &RegDescList, opt: Option<&OptArgs>) -> Result<Vec<u8>> {
        let (mut data, mut len): (*mut c_void, usize) = (ptr::null_mut(), 0);
        check(unsafe { sys::nixl_capi_get_local_partial_md(self.raw, descs.raw, &mut data, &mut len, opt_raw(opt)) })?;
        Ok(take_malloced(data, len))
    }

    /// Loads a peer's metadata; returns the peer's name.
    pub fn load_remote_metadata(&self, blob: &[u8]) -> Result<String> {
        let mut name: *mut c_char = ptr::null_mut();
        check(unsafe { sys::nixl_capi_load_remote_md(self.raw, blob.as_ptr() as *const c_void, blob.len(), &mut name) })?;
        if name.is_null() {
            return Ok(String::new());
        }
        let out = unsafe { CStr::from_ptr(name) }.to_string_lossy().into_owned();
        unsafe { sys::free(name as *mut c_void) };
        Ok(out)
    }

    pub fn invalidate_remote_metadata(&self, remote: &str) -> Result<()> {
        let r = cstring(remote)?;
        check(unsafe { sys::nixl_capi_invalidate_remote_md(self.raw, r.as_ptr()) }).map(|_| ())
    }

    /// Publishes the metadata through the configured store, or to the peer named in `opt`.
    pub fn send_local_metadata(&self, opt: Option<&OptArgs>) -> Result<()> {
        check(unsafe { sys::nixl_capi_send_local_md(self.raw, opt_raw(opt)) }).map(|_| ())
    }

    pub fn fetch_remote_metadata(&self, remote: &str, opt: Option<&OptArgs>) -> Result<()> {
        let r = cstring(remote)?;
        check(unsafe { sys::nixl_capi_fetch_remote_md(self.raw, r.as_ptr(), opt_raw(opt)) }).map(|_| ())
    }

    pub fn invalidate_local_metadata(&self, opt: Option<&OptArgs>) -> Result<()> {
        check(unsafe { sys::nixl_capi_invalidate_local_md(self.raw, opt_raw(opt)) }).map(|_| ())
    }

    /// Whether `remote`'s metadata is loaded (and covers `descs` when given).
    pub fn check_remote_metadata(&self, remote: &str, descs: Option<&XferDescList>) -> bool {
        let r = match cstring(remote) {
            Ok(r) => r,
            Err(_) => return false,
        };
        let d = descs.map(|d| d.raw).unwrap_or(ptr::null_mut());
        unsafe { sys::nixl_capi_check_remote_md(self.raw, r.as_ptr(), d) == sys::NIXL_CAPI_SUCCESS }
    }

    pub fn make_connection(&self, remote: &str, opt: Option<&OptArgs>) -> Result<()> {
        let r = cstring(remote)?;
        check(unsafe { sys::nixl_capi_agent_make_connection(self.raw, r.as_ptr(), opt_raw(opt)) }).map(|_| ())
    }

    /// Prepares one side of future transfers; `agent_name` empty means this agent's own memory.
    pub fn prepare_desc_list<'a>(&'a self, agent_name: &str, descs: &XferDescList, opt: Option<&OptArgs>) -> Result<PreparedDescList<'a>> {
        let n = cstring(agent_name)?;
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_prep_xfer_dlist(self.raw, n.as_ptr(), descs.raw, &mut raw, opt_raw(opt)) })?;
        Ok(PreparedDescList { agent: self, raw })
    }

    /// Builds a request from index selections of two prepared lists.
    pub fn make_xfer_request<'a>(&'a self, op: XferOp, local: &PreparedDescList, local_idx: &[i32], remote: &PreparedDescList,
                                 remote_idx: &[i32], opt: Option<&OptArgs>) -> Result<XferRequest<'a>> {
        let mut raw = ptr::null_mut();
        check(unsafe {
            sys::nixl_capi_make_xfer_req(self.raw, op as i32, local.raw, local_idx.as_ptr(), local_idx.len(), remote.raw, remote_idx.as_ptr(),
                                         remote_idx.len(), &mut raw, opt_raw(opt))
        })?;
        Ok(XferRequest { agent: self, raw })
    }

    /// Builds a request from two descriptor lists of equal shape.
    pub fn create_xfer_request<'a>(&'a self, op: XferOp, local: &XferDescList, remote: &XferDescList, remote_agent: &str,
                                   opt: Option<&OptArgs>) -> Result<XferRequest<'a>> {
        let r = cstring(remote_agent)?;
        let mut raw = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_xfer_req(self.raw, op as i32, local.raw, remote.raw, r.as_ptr(), &mut raw, opt_raw(opt)) })?;
        Ok(XferRequest { agent: self, raw })
    }

    /// Sends a stand-alone notification.
    pub fn send_notification(&self, remote: &str, msg: &[u8], opt: Option<&OptArgs>) -> Result<()> {
        let r = cstring(remote)?;
        check(unsafe { sys::nixl_capi_gen_notif(self.raw, r.as_ptr(), msg.as_ptr() as *const c_void, msg.len(), opt_raw(opt)) }).map(|_| ())
    }

    /// Collects the notifications that arrived since the last call.
    pub fn notifications(&self, opt: Option<&OptArgs>) -> Result<Notifications> {
        let mut map = ptr::null_mut();
        check(unsafe { sys::nixl_capi_create_notif_map(&mut map) })?;
        let st = unsafe { sys::nixl_capi_get_notifs(self.raw, map, opt_raw(opt)) };
        let mut out = Notifications::new();
        if st == sys::NIXL_CAPI_SUCCESS {
            let mut agents = 0usize;
            unsafe { sys::nixl_capi_notif_map_size(map, &mut agents) };
            for i in 0..agents {
                let mut name: *const c_char = ptr::null();
                if unsafe { sys::nixl_capi_notif_map_get_agent_at(map, i, &mut name) } != sys::NIXL_CAPI_SUCCESS || name.is_null() {
                    continue;
                }
                let mut count = 0usize;
                unsafe { sys::nixl_capi_notif_map_get_notifs_size(map, name, &mut count) };
                let mut msgs = Vec::with_capacity(count);
                for j in 0..count {
                    let (mut data, mut len): (*const c_void, usize) = (ptr::null(), 0);
                    if unsafe { sys::nixl_capi_notif_map_get_notif(map, name, j, &mut data, &mut len) } == sys::NIXL_CAPI_SUCCESS {
                        let bytes = if data.is_null() || len == 0 { Vec::new() } else { unsafe { std::slice::from_raw_parts(data as *const u8, len) }.to_vec() };
                        msgs.push(bytes);
                    }
                }
                out.push((unsafe { CStr::from_ptr(name) }.to_string_lossy().into_owned(), msgs));
            }
        }
        unsafe { sys::nixl_capi_destroy_notif_map(map) };
        check(st).map(|_| out)
    }
}

impl Drop for Agent {
    fn drop(&mut self) {
        unsafe { sys::nixl_capi_destroy_agent(self.raw) };
    }
}

fn take_mem_list(list: sys::nixl_capi_mem_list_t) -> Vec<MemType> {
    let mut out = Vec::new();
    if list.is_null() {
        return out;
    }
    let mut n = 0usize;
    if unsafe { sys::nixl_capi_mem_list_size(list, &mut n) } == sys::NIXL_CAPI_SUCCESS {
        for i in 0..n {
            let mut t = 0i32;
            if unsafe { sys::nixl_capi_mem_list_get(list, i, &mut t) } == sys::NIXL_CAPI_SUCCESS {
                out.push(MemType::from_raw(t));
            }
        }
    }
    unsafe { sys::nixl_capi_destroy_mem_list(list) };
    out
}

fn take_malloced(data: *mut c_void, len: usize) -> Vec<u8> {
    if data.is_null() {
        return Vec::new();
    }
    let out = unsafe { std::slice::from_raw_parts(data as *const u8, len) }.to_vec();
    unsafe { sys::free(data) };
    out
}

#[cfg(test)]
mod tests {
    use super::*;

    // Needs libnixl_capi.so and the plug-in directory of an in-tree build (NIXL_PLUGIN_DIR).
    #[test]
    fn dram_write_between_two_agents() {
        let a = Agent::new("rust_a").unwrap();
        let b = Agent::new("rust_b").unwrap();
        let (_, params) = a.plugin_params("NVLINK").unwrap();
        let _ba = a.create_backend("NVLINK", &params).unwrap();
        let _bb = b.create_backend("NVLINK", &params).unwrap();
        let src: Vec<u8> = (0..4096u32).map(|i| (i * 7) as u8).collect();
        let mut dst = vec![0u8; 4096];
        let dst_ptr = dst.as_mut_ptr(); // the library writes through this address
        let mut ra = RegDescList::new(MemType::Dram).unwrap();
        ra.add_slice(&src, 0).unwrap();
        let mut rb = RegDescList::new(MemType::Dram).unwrap();
        rb.add(dst_ptr as usize, 4096, 0, &[]).unwrap();
        a.register_memory(&ra, None).unwrap();
        b.register_memory(&rb, None).unwrap();
        assert_eq!(a.load_remote_metadata(&b.local_metadata().unwrap()).unwrap(), "rust_b");
        let mut la = XferDescList::new(MemType::Dram).unwrap();
        la.add_slice(&src, 0).unwrap();
        let mut lb = XferDescList::new(MemType::Dram).unwrap();
        lb.add(dst_ptr as usize, 4096, 0).unwrap();
        let mut opt = OptArgs::new().unwrap();
        opt.set_notification(b"done").unwrap();
        let req = a.create_xfer_request(XferOp::Write, &la, &lb, "rust_b", Some(&opt)).unwrap();
        req.post(None).unwrap();
        req.wait().unwrap();
        std::sync::atomic::fence(std::sync::atomic::Ordering::SeqCst);
        assert_eq!(src, dst);
        let mut seen = false;
        for _ in 0..1000 {
            let n = b.notifications(None).unwrap();
            if n.iter().any(|(from, msgs)| from == "rust_a" && msgs.iter().any(|m| m == b"done")) {
                seen = true;
                break;
            }
        }
        assert!(seen);
    }
}
