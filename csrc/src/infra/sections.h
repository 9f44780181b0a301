// Registered-memory bookkeeping.
//
// A *section* is the set of registrations one backend holds for one memory type, kept
// sorted by (device, address, length).  Transfer descriptors are resolved against a
// section to find the registration (and therefore the backend metadata: IPC mapping,
// file descriptor, ...) that covers them.
//
// Behavioural parity with the reference's src/infra/mem_section.h and
// src/infra/nixl_memory_section.cpp: overlapping registrations are legal; zero length
// on FILE/OBJ/BLK registrations means "unbounded"; the serialized form is
// `nixlSecElms` + per section `bknd` + an `nixlSDList` descriptor list
// (nixl_memory_section.cpp:333-363).  The lookup here differs: every list carries a
// running maximum of range ends, so a covering registration is found in O(log n) even
// when registrations nest or overlap.
#ifndef NIXL_B200_SECTIONS_H
#define NIXL_B200_SECTIONS_H

#include <array>
#include <atomic>
#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "backend/backend_engine.h"

// A registration as stored in a section: range, the user's meta blob (local side) or
// the backend's public blob (remote side), and the backend's metadata object.
class nixlSectionDesc : public nixlMetaDesc {
public:
    nixl_blob_t metaInfo;

    nixlSectionDesc() = default;
    nixlSectionDesc(const nixlBasicDesc &range, nixl_blob_t info, nixlBackendMD *md)
        : nixlMetaDesc(range.addr, range.len, range.devId, md), metaInfo(std::move(info)) {}
    nixl_blob_t serialize() const { return nixlBasicDesc::serialize() + metaInfo; }
};

class nixlSecDescList {
public:
    explicit nixlSecDescList(nixl_mem_t mem = DRAM_SEG) : mem_(mem) {}

    nixl_mem_t getType() const { return mem_; }
    int descCount() const { return static_cast<int>(items_.size()); }
    bool isEmpty() const { return items_.empty(); }
    const nixlSectionDesc &operator[](size_t i) const { return items_[i]; }
    nixlSectionDesc &operator[](size_t i) { return items_[i]; }
    std::vector<nixlSectionDesc>::const_iterator begin() const { return items_.begin(); }
    std::vector<nixlSectionDesc>::const_iterator end() const { return items_.end(); }

    // Sorted insert (after equal elements); returns the index used.
    int addDesc(const nixlSectionDesc &d);
    void remDesc(int index);
    void clear() { items_.clear(); maxEnd_.clear(); }

    // Exact {addr,len,devId} match or -1.
    int getIndex(const nixlBasicDesc &q) const;
    // Any registration covering q, or -1.  `hint` (a previous result) is tried first,
    // which makes resolving an ascending descriptor list linear overall.
    int getCoveringIndex(const nixlBasicDesc &q, int hint = -1) const;

    // Writes this list as an `nixlSDList`; `public_blob(i)` supplies the bytes that follow
    // the 24-byte range of element i.
    template<class F> nixl_status_t serialize(nixlSerDes *ser, F public_blob) const {
        ser->addStr("nixlDList", "nixlSDList");
        ser->addBuf("t", &mem_, sizeof(mem_));
        const size_t n = items_.size();
        ser->addBuf("n", &n, sizeof(n));
        for (size_t i = 0; i < n; ++i) {
            nixlBasicDesc wire = items_[i];
            if (unbounded() && wire.len == SIZE_MAX) wire.len = 0;
            ser->addStr("", wire.serialize() + public_blob(i));
        }
        return NIXL_SUCCESS;
    }

private:
    bool unbounded() const { return mem_ == BLK_SEG || mem_ == OBJ_SEG || mem_ == FILE_SEG; }
    nixlBasicDesc normalized(const nixlBasicDesc &q) const {
        return (unbounded() && q.len == 0) ? nixlBasicDesc(q.addr, SIZE_MAX, q.devId) : q;
    }
    static uint64_t endOf(const nixlBasicDesc &d) {
        return d.len > UINT64_MAX - d.addr ? UINT64_MAX : d.addr + d.len;
    }
    void rebuildMaxEnd(size_t from);

    nixl_mem_t mem_;
    std::vector<nixlSectionDesc> items_;
    // maxEnd_[i] = max range end over items_[first of this device .. i]
    std::vector<uint64_t> maxEnd_;
};

using section_key_t = std::pair<nixl_mem_t, nixlBackendEngine *>;
using backend_set_t = std::vector<nixlBackendEngine *>; // ordered by preference
using backend_map_t = std::unordered_map<nixl_backend_t, nixlBackendEngine *>;

class nixlMemSection {
public:
    virtual ~nixlMemSection() = default;

    // Engines that hold at least one registration of this memory type (preference order).
    const backend_set_t *queryBackends(nixl_mem_t mem) const;

    // Resolve every descriptor of `query` against `engine`'s section.
    nixl_status_t populate(const nixl_xfer_dlist_t &query, nixlBackendEngine *engine, nixl_meta_dlist_t &resp) const;
    // Same, run-length compressed (equal-length blocks at a constant stride inside one registration).
    nixl_status_t populate(const nixl_xfer_dlist_t &query, nixlBackendEngine *engine, nixl_stride_dlist_t &resp) const;

    const nixlSecDescList *find(nixl_mem_t mem, nixlBackendEngine *engine) const;

protected:
    nixlSecDescList &ensure(nixl_mem_t mem, nixlBackendEngine *engine);
    void dropIfEmpty(nixl_mem_t mem, nixlBackendEngine *engine);

    std::map<section_key_t, nixlSecDescList> sections_;
    std::array<backend_set_t, FILE_SEG + 1> byMem_;
};

class nixlLocalSection : public nixlMemSection {
public:
    ~nixlLocalSection() override;

    // Register every descriptor with `engine`; all-or-nothing.  On success the new
    // section entries are appended to `added` (used to mirror them into the agent's
    // own "remote" section for same-agent transfers).
    nixl_status_t addDescList(const nixl_reg_dlist_t &descs, nixlBackendEngine *engine,
                              std::vector<nixlSectionDesc> *added = nullptr);
    nixl_status_t remDescList(const nixl_reg_dlist_t &descs, nixlBackendEngine *engine);

    nixl_status_t serialize(nixlSerDes *ser) const;
    // Only the registrations named in `descs`, for the given engines.
    nixl_status_t serializePartial(nixlSerDes *ser, const backend_set_t &engines, const nixl_reg_dlist_t &descs) const;

private:
    nixl_status_t serializeSubset(nixlSerDes *ser, const std::map<section_key_t, std::vector<int>> *subset) const;
};

class nixlRemoteSection : public nixlMemSection {
public:
    explicit nixlRemoteSection(std::string agent);
    ~nixlRemoteSection() override;

    // Merge sections from a metadata blob.  Sections of backends we do not have are skipped.
    nixl_status_t loadRemoteData(nixlSerDes *des, const backend_map_t &engines);
    // Mirror a local registration (same-agent transfers).
    nixl_status_t loadLocalData(nixl_mem_t mem, const std::vector<nixlSectionDesc> &regs, nixlBackendEngine *engine);
    // Remove mirrored local registrations.
    nixl_status_t unloadLocalData(nixl_mem_t mem, const nixl_reg_dlist_t &descs, nixlBackendEngine *engine);

    const std::string &agent() const { return agent_; }
    // Unique id of this instance of the remote's metadata; prepared lists remember it
    // so that a reload is detected at post time.
    uint64_t generation() const { return generation_; }

private:
    std::string agent_;
    uint64_t generation_;
};

#endif
