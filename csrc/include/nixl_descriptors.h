// Descriptor model: a descriptor names a byte range {addr, len, devId}; lists of
// descriptors are typed by memory kind.
//
// API parity: class and method names follow the reference's
// src/api/cpp/nixl_descriptors.h (nixlBasicDesc :32, nixlBlobDesc :145,
// nixlRemoteDesc :205, nixlDescList<T> :262, aliases :466-477); the list wire
// format is the one of src/infra/nixl_descriptors.cpp:237-282.  The list template
// here is header-only so user code and CUDA translation units can instantiate it
// for their own descriptor types.
#ifndef NIXL_B200_DESCRIPTORS_H
#define NIXL_B200_DESCRIPTORS_H

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <sstream>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "nixl_types.h"
#include "serdes/serdes.h"

// 24-byte POD: the unit of the wire format.  Meaning of the fields per memory type:
//   DRAM: addr = host pointer, devId = NUMA hint (0 is fine)
//   VRAM: addr = device pointer, devId = CUDA device ordinal
//   FILE: addr = file offset, devId = file descriptor (or path-mode id)
class nixlBasicDesc {
public:
    uintptr_t addr = 0;
    size_t len = 0;
    uint64_t devId = 0;

    nixlBasicDesc() = default;
    nixlBasicDesc(const uintptr_t &a, const size_t &l, const uint64_t &dev) : addr(a), len(l), devId(dev) {}
    // Deserialize from exactly 24 raw bytes; anything else yields a zero descriptor.
    explicit nixlBasicDesc(const nixl_blob_t &raw) {
        if (raw.size() == sizeof(nixlBasicDesc)) std::memcpy(static_cast<void *>(this), raw.data(), sizeof(nixlBasicDesc));
    }

    // Total order: device, then address, then length.
    bool operator<(const nixlBasicDesc &o) const noexcept {
        if (devId != o.devId) return devId < o.devId;
        if (addr != o.addr) return addr < o.addr;
        return len < o.len;
    }
    friend bool operator==(const nixlBasicDesc &a, const nixlBasicDesc &b) {
        return a.addr == b.addr && a.len == b.len && a.devId == b.devId;
    }
    friend bool operator!=(const nixlBasicDesc &a, const nixlBasicDesc &b) { return !(a == b); }

    // True when `q` lies fully inside this range on the same device.
    bool covers(const nixlBasicDesc &q) const noexcept {
        return devId == q.devId && addr <= q.addr && addr + len >= q.addr + q.len;
    }
    bool overlaps(const nixlBasicDesc &q) const noexcept {
        return devId == q.devId && addr < q.addr + q.len && q.addr < addr + len;
    }

    nixl_blob_t serialize() const { return nixl_blob_t(reinterpret_cast<const char *>(this), sizeof(nixlBasicDesc)); }
    std::string to_string() const {
        std::ostringstream s;
        s << "(addr=0x" << std::hex << addr << std::dec << ", len=" << len << ", dev=" << devId << ")";
        return s.str();
    }
    void print(const std::string &suffix) const;
};
static_assert(sizeof(nixlBasicDesc) == 24, "descriptor wire size");

// Registration descriptor: range + opaque per-backend hint (file path/mode, bucket key, ...).
class nixlBlobDesc : public nixlBasicDesc {
public:
    nixl_blob_t metaInfo;

    nixlBlobDesc() = default;
    nixlBlobDesc(const uintptr_t &a, const size_t &l, const uint64_t &dev, const nixl_blob_t &meta = nixl_blob_t())
        : nixlBasicDesc(a, l, dev), metaInfo(meta) {}
    nixlBlobDesc(const nixlBasicDesc &d, const nixl_blob_t &meta) : nixlBasicDesc(d), metaInfo(meta) {}
    // Wire form: 24 raw bytes followed by metaInfo.
    explicit nixlBlobDesc(const nixl_blob_t &raw) {
        if (raw.size() >= sizeof(nixlBasicDesc)) {
            std::memcpy(static_cast<nixlBasicDesc *>(this), raw.data(), sizeof(nixlBasicDesc));
            metaInfo.assign(raw, sizeof(nixlBasicDesc), nixl_blob_t::npos);
        }
    }
    friend bool operator==(const nixlBlobDesc &a, const nixlBlobDesc &b) {
        return static_cast<const nixlBasicDesc &>(a) == static_cast<const nixlBasicDesc &>(b) && a.metaInfo == b.metaInfo;
    }
    nixl_blob_t serialize() const { return nixlBasicDesc::serialize() + metaInfo; }
    void print(const std::string &suffix) const;
};

// Range inside a named remote agent (used to build remote memory views).
class nixlRemoteDesc : public nixlBasicDesc {
public:
    std::string remoteAgent;

    nixlRemoteDesc() = default;
    nixlRemoteDesc(const uintptr_t a, const size_t l, const uint64_t dev, const std::string &agent)
        : nixlBasicDesc(a, l, dev), remoteAgent(agent) {}
    nixlRemoteDesc(const nixlBasicDesc &d, const std::string &agent) : nixlBasicDesc(d), remoteAgent(agent) {}
    explicit nixlRemoteDesc(const nixl_blob_t &raw) {
        if (raw.size() >= sizeof(nixlBasicDesc)) {
            std::memcpy(static_cast<nixlBasicDesc *>(this), raw.data(), sizeof(nixlBasicDesc));
            remoteAgent.assign(raw, sizeof(nixlBasicDesc), nixl_blob_t::npos);
        }
    }
    friend bool operator==(const nixlRemoteDesc &a, const nixlRemoteDesc &b) {
        return static_cast<const nixlBasicDesc &>(a) == static_cast<const nixlBasicDesc &>(b) && a.remoteAgent == b.remoteAgent;
    }
    nixl_blob_t serialize() const { return nixlBasicDesc::serialize() + remoteAgent; }
};

namespace nixl_detail {
void emitLine(const std::string &line); // writes one line to stdout (defined in the library)
// Which wire flavour a descriptor type uses: 'B' = packed 24-byte array, 'S' = one
// string per element, 0 = internal type that never goes on the wire.
template<class T> struct wire_kind { static constexpr char value = 0; };
template<> struct wire_kind<nixlBasicDesc> { static constexpr char value = 'B'; };
template<> struct wire_kind<nixlBlobDesc> { static constexpr char value = 'S'; };
template<> struct wire_kind<nixlRemoteDesc> { static constexpr char value = 'S'; };
} // namespace nixl_detail

template<class T> class nixlDescList {
    static_assert(std::is_base_of<nixlBasicDesc, T>::value, "descriptor lists hold nixlBasicDesc subclasses");

protected:
    nixl_mem_t type = DRAM_SEG;
    std::vector<T> descs;

public:
    using value_type = T;

    explicit nixlDescList(const nixl_mem_t &mem_type, const int &init_size = 0) : type(mem_type), descs(init_size) {}

    // Deserializing constructor.  On any framing error the list comes back empty
    // with descCount()==0 and (for callers that care) valid()==false.
    explicit nixlDescList(nixlSerDes *des) { ok_ = decode(des); if (!ok_) descs.clear(); }

    nixlDescList(const nixlDescList &) = default;
    nixlDescList(nixlDescList &&) noexcept = default;
    nixlDescList &operator=(const nixlDescList &) = default;
    nixlDescList &operator=(nixlDescList &&) noexcept = default;
    virtual ~nixlDescList() = default;

    nixl_mem_t getType() const { return type; }
    int descCount() const { return static_cast<int>(descs.size()); }
    bool isEmpty() const noexcept { return descs.empty(); }
    bool valid() const noexcept { return ok_; }

    const T &operator[](size_t i) const { return descs.at(i); }
    T &operator[](size_t i) { return descs.at(i); }
    typename std::vector<T>::const_iterator begin() const { return descs.begin(); }
    typename std::vector<T>::const_iterator end() const { return descs.end(); }
    typename std::vector<T>::iterator begin() { return descs.begin(); }
    typename std::vector<T>::iterator end() { return descs.end(); }
    const T *data() const { return descs.data(); }

    template<class Y> friend bool operator==(const nixlDescList<Y> &a, const nixlDescList<Y> &b);

    void resize(const size_t &n) { descs.resize(n); }
    void reserve(size_t n) { descs.reserve(n); }
    void clear() { descs.clear(); }
    void addDesc(const T &d) { descs.push_back(d); }
    template<class... Args> T &emplace(Args &&...args) { return descs.emplace_back(std::forward<Args>(args)...); }
    void remDesc(const int &index) {
        if (index < 0 || static_cast<size_t>(index) >= descs.size()) throw std::out_of_range("descriptor index out of range");
        descs.erase(descs.begin() + index);
    }

    // Drop everything but {addr,len,devId}.
    nixlDescList<nixlBasicDesc> trim() const {
        nixlDescList<nixlBasicDesc> out(type);
        out.reserve(descs.size());
        for (const auto &d : descs) out.addDesc(static_cast<const nixlBasicDesc &>(d));
        return out;
    }

    // Index of the first element equal (as a basic descriptor) to `q`, or NIXL_ERR_NOT_FOUND.
    int getIndex(const nixlBasicDesc &q) const {
        for (size_t i = 0; i < descs.size(); ++i)
            if (static_cast<const nixlBasicDesc &>(descs[i]) == q) return static_cast<int>(i);
        return NIXL_ERR_NOT_FOUND;
    }

    // Sum of lengths.
    size_t totalBytes() const {
        size_t s = 0;
        for (const auto &d : descs) s += d.len;
        return s;
    }

    nixl_status_t serialize(nixlSerDes *ser) const {
        constexpr char kind = nixl_detail::wire_kind<T>::value;
        if constexpr (kind == 0) {
            return NIXL_ERR_INVALID_PARAM;
        } else {
            ser->addStr("nixlDList", kind == 'B' ? "nixlBDList" : "nixlSDList");
            ser->addBuf("t", &type, sizeof(type));
            const size_t n = descs.size();
            ser->addBuf("n", &n, sizeof(n));
            if (n == 0) return NIXL_SUCCESS;
            if constexpr (kind == 'B') {
                ser->addStr("", std::string(reinterpret_cast<const char *>(descs.data()), n * sizeof(nixlBasicDesc)));
            } else {
                for (const auto &d : descs) ser->addStr("", d.serialize());
            }
            return NIXL_SUCCESS;
        }
    }

    std::string to_string(bool compact = false) const {
        std::ostringstream s;
        s << "DescList[" << nixlEnumStrings::memTypeStr(type) << ", n=" << descs.size() << "]";
        if (!compact)
            for (const auto &d : descs) s << "\n  " << d.to_string();
        return s.str();
    }
    void print() const { nixl_detail::emitLine(to_string()); }

private:
    bool ok_ = true;

    bool decode(nixlSerDes *des) {
        constexpr char kind = nixl_detail::wire_kind<T>::value;
        if constexpr (kind == 0) {
            return false;
        } else {
            const std::string flavour = des->getStr("nixlDList");
            if (flavour != (kind == 'B' ? "nixlBDList" : "nixlSDList")) return false;
            if (des->getBuf("t", &type, sizeof(type)) != NIXL_SUCCESS) return false;
            if (type < DRAM_SEG || type > FILE_SEG) return false;
            size_t n = 0;
            if (des->getBuf("n", &n, sizeof(n)) != NIXL_SUCCESS) return false;
            if (n == 0) return true;
            if constexpr (kind == 'B') {
                const std::string raw = des->getStr("");
                if (raw.size() != n * sizeof(nixlBasicDesc)) return false;
                descs.resize(n);
                std::memcpy(static_cast<void *>(descs.data()), raw.data(), raw.size());
            } else {
                if (n > des->remaining()) return false; // each element costs at least one byte
                descs.reserve(n);
                for (size_t i = 0; i < n; ++i) {
                    const std::string raw = des->getStr("");
                    if (raw.size() < sizeof(nixlBasicDesc)) return false;
                    descs.emplace_back(raw);
                }
            }
            return true;
        }
    }
};

template<class Y> bool operator==(const nixlDescList<Y> &a, const nixlDescList<Y> &b) {
    return a.type == b.type && a.descs == b.descs;
}

using nixl_xfer_dlist_t = nixlDescList<nixlBasicDesc>;
using nixl_reg_dlist_t = nixlDescList<nixlBlobDesc>;
using nixl_remote_dlist_t = nixlDescList<nixlRemoteDesc>;
using nixl_local_dlist_t = nixlDescList<nixlBasicDesc>;

#endif
