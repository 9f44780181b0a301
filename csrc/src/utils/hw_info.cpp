#include "utils/hw_info.h"

#include <dirent.h>

#include <cstdlib>
#include <fstream>
#include <sstream>

namespace nixl {

namespace {
bool readHex(const std::string &path, unsigned long &out) {
    std::ifstream f(path);
    std::string s;
    if (!(f >> s)) return false;
    char *end = nullptr;
    out = std::strtoul(s.c_str(), &end, 16);
    return end != s.c_str();
}
} // namespace

hwInfo hwInfo::scan(const std::string &root_in) {
    hwInfo info;
    std::string root = root_in;
    if (root.empty()) {
        const char *env = std::getenv("NIXL_SYSFS_PCI_ROOT");
        root = env && *env ? env : "/sys/bus/pci/devices";
    }
    DIR *d = ::opendir(root.c_str());
    if (!d) return info;
    while (dirent *e = ::readdir(d)) {
        if (e->d_name[0] == '.') continue;
        const std::string dev = root + "/" + e->d_name;
        unsigned long vendor = 0, cls = 0, device = 0;
        if (!readHex(dev + "/vendor", vendor) || !readHex(dev + "/class", cls)) continue;
        readHex(dev + "/device", device);
        const unsigned long base = cls >> 8; // class + subclass, programming interface dropped
        switch (vendor) {
        case 0x10de:
            if (base == 0x0300 || base == 0x0302) ++info.numNvidiaGpus;
            else if (base == 0x0680) ++info.numNvSwitches;
            break;
        case 0x1002:
            if (base == 0x0300 || base == 0x0302 || base == 0x1200) ++info.numAmdGpus;
            break;
        case 0x15b3:
            if (base == 0x0207 || base == 0x0200) ++info.numIbDevices;
            break;
        case 0x1d0f:
            if (device >= 0xefa0 && device <= 0xefa3) ++info.numEfaDevices;
            break;
        default: break;
        }
    }
    ::closedir(d);
    return info;
}

const hwInfo &hwInfo::instance() {
    static const hwInfo info = scan();
    return info;
}

std::string hwInfo::toString() const {
    std::ostringstream os;
    os << "nvidia_gpus=" << numNvidiaGpus << " nvswitches=" << numNvSwitches << " amd_gpus=" << numAmdGpus << " ib_devices=" << numIbDevices
       << " efa_devices=" << numEfaDevices;
    return os.str();
}

} // namespace nixl
