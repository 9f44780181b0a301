// Host hardware inventory from the PCI sysfs tree: what accelerators and fabric devices the box
// has, without loading CUDA or any NIC library (same purpose as the reference's
// src/utils/common/hw_info.h; here NVSwitch bridges are counted too, since the NVLINK backend's
// reach depends on them).
#ifndef NIXL_B200_HW_INFO_H
#define NIXL_B200_HW_INFO_H

#include <string>

namespace nixl {

struct hwInfo {
    unsigned numNvidiaGpus = 0;   // vendor 0x10de, display / 3-D controller class
    unsigned numNvSwitches = 0;   // vendor 0x10de, bridge class 0x0680
    unsigned numAmdGpus = 0;      // vendor 0x1002, display / 3-D controller / processing accelerator
    unsigned numIbDevices = 0;    // vendor 0x15b3, class 0x0207 (InfiniBand) or 0x0200 (RoCE NIC)
    unsigned numEfaDevices = 0;   // vendor 0x1d0f, device 0xefa0..0xefa3

    // Scans `root` (default: $NIXL_SYSFS_PCI_ROOT, else /sys/bus/pci/devices).  Missing tree: all zero.
    static hwInfo scan(const std::string &root = "");
    // Process-wide snapshot taken on first use.
    static const hwInfo &instance();
    std::string toString() const;
};

} // namespace nixl

#endif
