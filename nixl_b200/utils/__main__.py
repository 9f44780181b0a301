"""``python -m nixl_b200.utils``: which network interfaces sit next to which GPU on this host."""
from . import pci_topology

if __name__ == "__main__":
    topo = pci_topology()
    print(topo["text"] or f"no GPUs in the PCI tree ({len(topo['nics'])} network device(s))")
