// Memory layout of a prepared memory view as it sits in device memory.  Shared between
// the backend that builds views (host code) and nixl_device.cuh (device code).
#ifndef NIXL_B200_DEVICE_LAYOUT_H
#define NIXL_B200_DEVICE_LAYOUT_H

#include <cstdint>

#define NIXL_MEMVIEW_MAGIC 0x4E584D5649455731ull /* "NXMVIEW1" */
#define NIXL_MEMVIEW_LOCAL 1u
#define NIXL_MEMVIEW_REMOTE 2u

struct nixlMemViewHeader {
    uint64_t magic;
    uint32_t count; // number of entries that follow
    uint32_t kind;  // NIXL_MEMVIEW_LOCAL or NIXL_MEMVIEW_REMOTE
};

// One registered range as the GPU sees it.  ptr == 0 marks a hole (an absent rank).
struct nixlMemViewEntry {
    uint64_t ptr;
    uint64_t len;
};

#endif
