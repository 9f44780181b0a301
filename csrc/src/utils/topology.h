// Which network interfaces sit close to which GPU, from the PCI sysfs tree: every device's place in the tree (the chain
// of bridges above it), its NUMA node and, for network devices, the interface names the kernel gave it.  The TCP backend
// uses it to put the addresses of the nearest interfaces first; nothing here loads CUDA or a NIC library.
//
// Role parity: the reference's libfabric utilities discover the same relation with hwloc to give every GPU its rails
// (src/utils/libfabric/libfabric_topology.cpp); here the tree is read directly, and tests build it in a temporary
// directory.
#ifndef NIXL_B200_TOPOLOGY_H
#define NIXL_B200_TOPOLOGY_H

#include <cstdint>
#include <string>
#include <vector>

namespace nixl {

struct pciDevice {
    std::string bdf;                 // "0000:1b:00.0"
    std::vector<std::string> chain;  // the tree above it, outermost first: "pci0000:15", "0000:15:01.0", ..., the device itself
    int numaNode = -1;
    uint32_t vendor = 0, device = 0, classCode = 0; // class code as in sysfs (24 bits)
    std::vector<std::string> netInterfaces;         // network devices: "eth0", "ibp27s0", ...
    bool isGpu() const;
    bool isNic() const;
};

class pciTopology {
public:
    // Scans `root` (default: $NIXL_SYSFS_PCI_ROOT, else /sys/bus/pci/devices).  Missing tree: empty.
    static pciTopology scan(const std::string &root = "");

    const std::vector<pciDevice> &gpus() const { return gpus_; } // in bus order, which is CUDA's order under CUDA_DEVICE_ORDER=PCI_BUS_ID
    const std::vector<pciDevice> &nics() const { return nics_; }

    // How far apart two devices are: the bridges between them through their closest common ancestor; devices under
    // different root complexes cost 100 more, and 100 more again on different NUMA nodes.
    static int distance(const pciDevice &a, const pciDevice &b);
    // The network devices, nearest to that GPU first (ties in bus order).
    std::vector<const pciDevice *> nicsNearGpu(size_t gpu_index) const;
    // Interface names in that order, for all GPUs when gpu_index is out of range (then: bus order).
    std::vector<std::string> interfacesNearGpu(size_t gpu_index) const;
    std::string toString() const;

private:
    std::vector<pciDevice> gpus_, nics_;
};

} // namespace nixl

#endif
