// Helper types of the south-bound (backend plugin) interface.
//
// Parity: same roles and names as the reference's src/api/cpp/backend/backend_aux.h
// (notif_list_t :29, optional args :32, init params :46, request handle :60,
// backend metadata :67, meta descriptors :92/:119, stride descriptors :140-184).
#ifndef NIXL_B200_BACKEND_AUX_H
#define NIXL_B200_BACKEND_AUX_H

#include <cassert>
#include <string>
#include <utility>
#include <vector>
#include "nixl_descriptors.h"
#include "nixl_types.h"

// (sender agent, message) pairs drained from a backend.
using notif_list_t = std::vector<std::pair<std::string, std::string>>;

struct nixlBackendOptionalArgs {
    nixl_blob_t notifMsg;
    bool hasNotif = false;
    nixl_blob_t customParam;
};
using nixl_opt_b_args_t = nixlBackendOptionalArgs;

// What the agent hands a plugin when it instantiates an engine.
class nixlBackendInitParams {
public:
    std::string localAgent;
    nixl_backend_t type;
    nixl_b_params_t *customParams = nullptr;
    bool enableProgTh = false;
    uint64_t pthrDelay = 0; // microseconds
    nixl_thread_sync_t syncMode = nixl_thread_sync_t::NIXL_THREAD_SYNC_DEFAULT;
    bool enableTelemetry_ = false;
};

// Common base so the agent can own backend request state without knowing its type.
class nixlBackendReqH {
public:
    nixlBackendReqH() = default;
    virtual ~nixlBackendReqH() = default;
};

// Common base of per-registration backend metadata (private = local side,
// public = loaded from a remote blob).
class nixlBackendMD {
protected:
    bool isPrivateMD;

public:
    explicit nixlBackendMD(bool is_private) : isPrivateMD(is_private) {}
    virtual ~nixlBackendMD() = default;
    bool isPrivate() const { return isPrivateMD; }
};

// Descriptor resolved against a registration: range + that registration's backend metadata.
class nixlMetaDesc : public nixlBasicDesc {
public:
    nixlBackendMD *metadataP = nullptr;
    using nixlBasicDesc::nixlBasicDesc;
    nixlMetaDesc() = default;
    nixlMetaDesc(uintptr_t a, size_t l, uint64_t dev, nixlBackendMD *md) : nixlBasicDesc(a, l, dev), metadataP(md) {}
    friend bool operator==(const nixlMetaDesc &a, const nixlMetaDesc &b) {
        return static_cast<const nixlBasicDesc &>(a) == static_cast<const nixlBasicDesc &>(b) && a.metadataP == b.metadataP;
    }
};

struct nixlRemoteMetaDesc : public nixlMetaDesc {
    std::string remoteAgent;
    using nixlMetaDesc::nixlMetaDesc;
    nixlRemoteMetaDesc() = default;
    explicit nixlRemoteMetaDesc(const std::string &agent) : nixlMetaDesc(), remoteAgent(agent) {}
    friend bool operator==(const nixlRemoteMetaDesc &a, const nixlRemoteMetaDesc &b) {
        return static_cast<const nixlMetaDesc &>(a) == static_cast<const nixlMetaDesc &>(b) && a.remoteAgent == b.remoteAgent;
    }
};

using nixl_meta_dlist_t = nixlDescList<nixlMetaDesc>;
using nixl_remote_meta_dlist_t = nixlDescList<nixlRemoteMetaDesc>;

// Run-length form of a prepared list: `count` blocks of `len` bytes, `stride` bytes
// apart, the first of which has flat index `start_idx`.  A 64K-block KV cache that is
// laid out regularly collapses to a handful of these.
class nixlStrideDesc : public nixlMetaDesc {
public:
    size_t stride = 0;
    size_t count = 0;
    size_t start_idx = 0;

    nixlStrideDesc() = default;
    using nixlMetaDesc::nixlMetaDesc;
    nixlStrideDesc(uintptr_t a, size_t l, uint64_t dev, nixlBackendMD *md, size_t stride_, size_t count_)
        : nixlMetaDesc(a, l, dev, md), stride(stride_), count(count_) {}

    // Expand `size` consecutive blocks starting at flat index idx (dense runs only when size > 1).
    nixlMetaDesc getMetaDesc(size_t idx, size_t size) const noexcept {
        return nixlMetaDesc(addr + static_cast<uintptr_t>(idx - start_idx) * stride, len * size, devId, metadataP);
    }
};

class nixlStrideDescList : public nixlDescList<nixlStrideDesc> {
public:
    using nixlDescList<nixlStrideDesc>::nixlDescList;

    size_t flatSize() const { return descs.empty() ? 0 : descs.back().start_idx + descs.back().count; }

    // Run containing flat index `flat_idx` (must be < flatSize()).
    const nixlStrideDesc &find(size_t flat_idx, size_t /*run_size_hint*/ = 1) const noexcept {
        size_t lo = 0, hi = descs.size();
        while (hi - lo > 1) {
            const size_t mid = (lo + hi) / 2;
            if (descs[mid].start_idx <= flat_idx) lo = mid; else hi = mid;
        }
        return descs[lo];
    }
};
using nixl_stride_dlist_t = nixlStrideDescList;

#endif
