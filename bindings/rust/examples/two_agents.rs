//! Two agents in one process: register host buffers, exchange metadata, WRITE with a notification.
//! Run from bindings/rust with NIXL_PLUGIN_DIR pointing at nixl_b200/lib/plugins of an in-tree build.
use nixl_b200::{Agent, MemType, OptArgs, RegDescList, XferDescList, XferOp};

fn main() -> Result<(), Box<dyn std::error::Error>> {
    let prefill = Agent::new("prefill")?;
    let decode = Agent::new("decode")?;
    println!("plug-ins: {:?}", prefill.available_plugins()?);
    let (mems, params) = prefill.plugin_params("NVLINK")?;
    println!("NVLINK serves {:?} with defaults {:?}", mems, params.to_vec()?);
    let _bp = prefill.create_backend("NVLINK", &params)?;
    let _bd = decode.create_backend("NVLINK", &params)?;

    let src: Vec<u32> = (0..1 << 16).collect();
    let mut dst = vec![0u32; 1 << 16];
    let bytes = src.len() * 4;
    let (src_addr, dst_addr) = (src.as_ptr() as usize, dst.as_mut_ptr() as usize);

    let mut reg_src = RegDescList::new(MemType::Dram)?;
    reg_src.add(src_addr, bytes, 0, &[])?;
    let mut reg_dst = RegDescList::new(MemType::Dram)?;
    reg_dst.add(dst_addr, bytes, 0, &[])?;
    prefill.register_memory(&reg_src, None)?;
    decode.register_memory(&reg_dst, None)?;

    let peer = prefill.load_remote_metadata(&decode.local_metadata()?)?;
    let mut local = XferDescList::new(MemType::Dram)?;
    local.add(src_addr, bytes, 0)?;
    let mut remote = XferDescList::new(MemType::Dram)?;
    remote.add(dst_addr, bytes, 0)?;
    let mut opt = OptArgs::new()?;
    opt.set_notification(b"kv-ready")?;
    let req = prefill.create_xfer_request(XferOp::Write, &local, &remote, &peer, Some(&opt))?;
    req.post(None)?;
    req.wait()?;
    loop {
        let got = decode.notifications(None)?;
        if got.iter().any(|(from, msgs)| from == "prefill" && msgs.iter().any(|m| m == b"kv-ready")) {
            break;
        }
    }
    std::sync::atomic::fence(std::sync::atomic::Ordering::SeqCst);
    assert_eq!(src, dst);
    println!("moved {} bytes, notification received", bytes);
    drop(req);
    prefill.deregister_memory(&reg_src, None)?;
    decode.deregister_memory(&reg_dst, None)?;
    Ok(())
}
