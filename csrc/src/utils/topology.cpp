#include "utils/topology.h"

#include <dirent.h>
#include <limits.h>

#include <algorithm>
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

std::vector<std::string> listDir(const std::string &path) {
    std::vector<std::string> out;
    if (DIR *d = ::opendir(path.c_str())) {
        while (dirent *e = ::readdir(d))
            if (e->d_name[0] != '.') out.push_back(e->d_name);
        ::closedir(d);
    }
    std::sort(out.begin(), out.end());
    return out;
}

bool looksLikeBdf(const std::string &s) { // dddd:bb:dd.f
    return s.size() == 12 && s[4] == ':' && s[7] == ':' && s[10] == '.';
}
} // namespace

bool pciDevice::isGpu() const {
    const uint32_t base = classCode >> 8;
    return (vendor == 0x10de && (base == 0x0300 || base == 0x0302)) || (vendor == 0x1002 && (base == 0x0300 || base == 0x0302 || base == 0x1200));
}
bool pciDevice::isNic() const {
    const uint32_t base = classCode >> 8;
    return base == 0x0200 || base == 0x0207 || base == 0x0280; // Ethernet, InfiniBand, other network controller
}

pciTopology pciTopology::scan(const std::string &root_in) {
    pciTopology t;
    std::string root = root_in;
    if (root.empty()) {
        const char *env = std::getenv("NIXL_SYSFS_PCI_ROOT");
        root = env && *env ? env : "/sys/bus/pci/devices";
    }
    for (const std::string &name : listDir(root)) {
        const std::string dev = root + "/" + name;
        unsigned long vendor = 0, cls = 0, device = 0;
        if (!readHex(dev + "/vendor", vendor) || !readHex(dev + "/class", cls)) continue;
        readHex(dev + "/device", device);
        pciDevice d;
        d.bdf = name;
        d.vendor = static_cast<uint32_t>(vendor);
        d.device = static_cast<uint32_t>(device);
        d.classCode = static_cast<uint32_t>(cls);
        if (!d.isGpu() && !d.isNic()) continue;
        // The entry is a link into /sys/devices/pci<domain:bus>/<bridge>/.../<device>: the path is the tree.
        char real[PATH_MAX];
        std::string path = ::realpath(dev.c_str(), real) ? real : dev;
        size_t start = 0;
        bool in_tree = false;
        while (start <= path.size()) {
            size_t end = path.find('/', start);
            if (end == std::string::npos) end = path.size();
            const std::string piece = path.substr(start, end - start);
            if (piece.compare(0, 3, "pci") == 0 && piece.find(':') != std::string::npos) in_tree = true;
            if (in_tree && (looksLikeBdf(piece) || piece.compare(0, 3, "pci") == 0)) d.chain.push_back(piece);
            start = end + 1;
        }
        if (d.chain.empty() || d.chain.back() != name) d.chain.push_back(name); // a flat tree (no links): the device alone
        std::ifstream numa(dev + "/numa_node");
        if (!(numa >> d.numaNode)) d.numaNode = -1;
        if (d.isNic()) d.netInterfaces = listDir(dev + "/net");
        (d.isGpu() ? t.gpus_ : t.nics_).push_back(std::move(d));
    }
    return t;
}

int pciTopology::distance(const pciDevice &a, const pciDevice &b) {
    size_t common = 0;
    while (common < a.chain.size() && common < b.chain.size() && a.chain[common] == b.chain[common]) ++common;
    int d = static_cast<int>((a.chain.size() - common) + (b.chain.size() - common));
    if (common == 0) d += 100; // different root complexes: through the host
    if (a.numaNode >= 0 && b.numaNode >= 0 && a.numaNode != b.numaNode) d += 100; // and through the socket interconnect
    return d;
}

std::vector<const pciDevice *> pciTopology::nicsNearGpu(size_t gpu_index) const {
    std::vector<const pciDevice *> out;
    for (const auto &n : nics_) out.push_back(&n);
    if (gpu_index < gpus_.size()) {
        const pciDevice &g = gpus_[gpu_index];
        std::stable_sort(out.begin(), out.end(), [&](const pciDevice *x, const pciDevice *y) { return distance(g, *x) < distance(g, *y); });
    }
    return out;
}

std::vector<std::string> pciTopology::interfacesNearGpu(size_t gpu_index) const {
    std::vector<std::string> out;
    for (const pciDevice *n : nicsNearGpu(gpu_index))
        for (const auto &i : n->netInterfaces) out.push_back(i);
    return out;
}

std::string pciTopology::toString() const {
    std::ostringstream os;
    for (size_t g = 0; g < gpus_.size(); ++g) {
        os << "gpu" << g << " " << gpus_[g].bdf << " numa " << gpus_[g].numaNode << ":";
        for (const pciDevice *n : nicsNearGpu(g)) {
            os << " " << n->bdf << "(";
            for (size_t i = 0; i < n->netInterfaces.size(); ++i) os << (i ? "," : "") << n->netInterfaces[i];
            os << ";d=" << distance(gpus_[g], *n) << ")";
        }
        os << "\n";
    }
    return os.str();
}

} // namespace nixl
