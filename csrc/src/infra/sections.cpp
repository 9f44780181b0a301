#include "infra/sections.h"

#include <algorithm>

#include "utils/log.h"

// ------------------------------------------------------------------ nixlSecDescList

void nixlSecDescList::rebuildMaxEnd(size_t from) {
    maxEnd_.resize(items_.size());
    for (size_t i = from; i < items_.size(); ++i) {
        const uint64_t e = endOf(items_[i]);
        const bool same_dev = i > 0 && items_[i - 1].devId == items_[i].devId;
        maxEnd_[i] = same_dev ? std::max(maxEnd_[i - 1], e) : e;
    }
}

int nixlSecDescList::addDesc(const nixlSectionDesc &d) {
    nixlSectionDesc n = d;
    static_cast<nixlBasicDesc &>(n) = normalized(d);
    auto pos = std::upper_bound(items_.begin(), items_.end(), n,
                                [](const nixlSectionDesc &a, const nixlSectionDesc &b) {
                                    return static_cast<const nixlBasicDesc &>(a) < static_cast<const nixlBasicDesc &>(b);
                                });
    const size_t idx = static_cast<size_t>(pos - items_.begin());
    items_.insert(pos, std::move(n));
    rebuildMaxEnd(idx);
    return static_cast<int>(idx);
}

void nixlSecDescList::remDesc(int index) {
    if (index < 0 || static_cast<size_t>(index) >= items_.size()) return;
    items_.erase(items_.begin() + index);
    rebuildMaxEnd(static_cast<size_t>(index));
}

int nixlSecDescList::getIndex(const nixlBasicDesc &query) const {
    const nixlBasicDesc q = normalized(query);
    auto pos = std::lower_bound(items_.begin(), items_.end(), q,
                                [](const nixlSectionDesc &a, const nixlBasicDesc &b) {
                                    return static_cast<const nixlBasicDesc &>(a) < b;
                                });
    if (pos == items_.end() || !(static_cast<const nixlBasicDesc &>(*pos) == q)) return -1;
    return static_cast<int>(pos - items_.begin());
}

int nixlSecDescList::getCoveringIndex(const nixlBasicDesc &query, int hint) const {
    const nixlBasicDesc q = normalized(query);
    if (hint >= 0 && static_cast<size_t>(hint) < items_.size()) {
        if (items_[hint].covers(q)) return hint;
        if (static_cast<size_t>(hint) + 1 < items_.size() && items_[hint + 1].covers(q)) return hint + 1;
    }
    // Last registration on q's device that starts at or before q.addr.
    auto pos = std::upper_bound(items_.begin(), items_.end(), q, [](const nixlBasicDesc &b, const nixlSectionDesc &a) {
        if (b.devId != a.devId) return b.devId < a.devId;
        return b.addr < a.addr;
    });
    if (pos == items_.begin()) return -1;
    int i = static_cast<int>(pos - items_.begin()) - 1;
    if (items_[i].devId != q.devId) return -1;
    const uint64_t need = endOf(q);
    if (maxEnd_[i] < need) return -1; // nobody that starts early enough reaches far enough
    for (; i >= 0 && items_[i].devId == q.devId; --i)
        if (endOf(items_[i]) >= need) return i;
    return -1;
}

// ------------------------------------------------------------------ nixlMemSection

const backend_set_t *nixlMemSection::queryBackends(nixl_mem_t mem) const {
    if (mem < DRAM_SEG || mem > FILE_SEG) return nullptr;
    return &byMem_[mem];
}

const nixlSecDescList *nixlMemSection::find(nixl_mem_t mem, nixlBackendEngine *engine) const {
    auto it = sections_.find({mem, engine});
    return it == sections_.end() ? nullptr : &it->second;
}

nixlSecDescList &nixlMemSection::ensure(nixl_mem_t mem, nixlBackendEngine *engine) {
    auto it = sections_.find({mem, engine});
    if (it != sections_.end()) return it->second;
    auto &set = byMem_[mem];
    if (std::find(set.begin(), set.end(), engine) == set.end()) set.push_back(engine);
    return sections_.emplace(section_key_t{mem, engine}, nixlSecDescList(mem)).first->second;
}

void nixlMemSection::dropIfEmpty(nixl_mem_t mem, nixlBackendEngine *engine) {
    auto it = sections_.find({mem, engine});
    if (it == sections_.end() || !it->second.isEmpty()) return;
    sections_.erase(it);
    auto &set = byMem_[mem];
    set.erase(std::remove(set.begin(), set.end(), engine), set.end());
}

nixl_status_t nixlMemSection::populate(const nixl_xfer_dlist_t &query, nixlBackendEngine *engine,
                                       nixl_meta_dlist_t &resp) const {
    if (query.getType() != resp.getType() || query.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixlSecDescList *base = find(query.getType(), engine);
    if (!base) return NIXL_ERR_NOT_FOUND;
    resp.clear();
    resp.reserve(query.descCount());
    int at = -1;
    for (const auto &q : query) {
        at = base->getCoveringIndex(q, at);
        if (at < 0) {
            resp.clear();
            return NIXL_ERR_UNKNOWN;
        }
        resp.emplace(q.addr, q.len, q.devId, (*base)[at].metadataP);
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlMemSection::populate(const nixl_xfer_dlist_t &query, nixlBackendEngine *engine,
                                       nixl_stride_dlist_t &resp) const {
    if (query.getType() != resp.getType() || query.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixlSecDescList *base = find(query.getType(), engine);
    if (!base) return NIXL_ERR_NOT_FOUND;
    resp.clear();
    int at = -1;
    size_t flat = 0;
    nixlStrideDesc run;
    bool open = false;
    uintptr_t last_addr = 0;
    for (const auto &q : query) {
        at = base->getCoveringIndex(q, at);
        if (at < 0) {
            resp.clear();
            return NIXL_ERR_UNKNOWN;
        }
        nixlBackendMD *md = (*base)[at].metadataP;
        bool extended = false;
        if (open && q.len == run.len && q.devId == run.devId && md == run.metadataP && q.addr > last_addr) {
            const size_t step = q.addr - last_addr;
            if (run.count == 1) {
                run.stride = step;
                extended = true;
            } else if (step == run.stride) extended = true;
        }
        if (extended) {
            ++run.count;
        } else {
            if (open) resp.addDesc(run);
            run = nixlStrideDesc(q.addr, q.len, q.devId, md, q.len, 1);
            run.start_idx = flat;
            open = true;
        }
        last_addr = q.addr;
        ++flat;
    }
    if (open) resp.addDesc(run);
    return NIXL_SUCCESS;
}

// ------------------------------------------------------------------ nixlLocalSection

nixl_status_t nixlLocalSection::addDescList(const nixl_reg_dlist_t &descs, nixlBackendEngine *engine,
                                            std::vector<nixlSectionDesc> *added) {
    if (!engine || descs.isEmpty()) return NIXL_ERR_INVALID_PARAM;
    const nixl_mem_t mem = descs.getType();
    const auto mems = engine->getSupportedMems();
    if (std::find(mems.begin(), mems.end(), mem) == mems.end()) return NIXL_ERR_NOT_SUPPORTED;

    std::vector<nixlSectionDesc> fresh;
    fresh.reserve(descs.descCount());
    nixl_status_t st = NIXL_SUCCESS;
    for (const auto &d : descs) {
        nixlBackendMD *md = nullptr;
        st = engine->registerMem(d, mem, md);
        if (st != NIXL_SUCCESS) break;
        fresh.emplace_back(d, d.metaInfo, md);
    }
    if (st != NIXL_SUCCESS) { // undo what this call registered
        for (auto &f : fresh) engine->deregisterMem(f.metadataP);
        return st;
    }
    nixlSecDescList &sec = ensure(mem, engine);
    for (auto &f : fresh) sec.addDesc(f);
    if (added) added->insert(added->end(), fresh.begin(), fresh.end());
    return NIXL_SUCCESS;
}

nixl_status_t nixlLocalSection::remDescList(const nixl_reg_dlist_t &descs, nixlBackendEngine *engine) {
    const nixl_mem_t mem = descs.getType();
    auto it = sections_.find({mem, engine});
    if (it == sections_.end()) return NIXL_ERR_NOT_FOUND;
    nixlSecDescList &sec = it->second;
    // Validate first so a bad list changes nothing.
    for (const auto &d : descs)
        if (sec.getIndex(d) < 0) return NIXL_ERR_NOT_FOUND;
    for (const auto &d : descs) {
        const int idx = sec.getIndex(d);
        if (idx < 0) continue; // duplicate entry in the list
        engine->deregisterMem(sec[idx].metadataP);
        sec.remDesc(idx);
    }
    dropIfEmpty(mem, engine);
    return NIXL_SUCCESS;
}

nixl_status_t nixlLocalSection::serializeSubset(nixlSerDes *ser,
                                                const std::map<section_key_t, std::vector<int>> *subset) const {
    size_t count = 0;
    if (subset) {
        for (auto &kv : *subset) count += kv.first.second->supportsRemote() ? 1 : 0;
    } else {
        for (auto &kv : sections_) count += kv.first.second->supportsRemote() ? 1 : 0;
    }
    ser->addBuf("nixlSecElms", &count, sizeof(count));

    auto emit = [&](const section_key_t &key, const nixlSecDescList &sec, const std::vector<int> *pick) -> nixl_status_t {
        nixlBackendEngine *engine = key.second;
        if (!engine->supportsRemote()) return NIXL_SUCCESS;
        ser->addStr("bknd", engine->getType());
        nixlSecDescList out(sec.getType());
        const nixlSecDescList *src = &sec;
        if (pick) {
            for (int i : *pick) out.addDesc(sec[i]);
            src = &out;
        }
        nixl_status_t inner = NIXL_SUCCESS;
        src->serialize(ser, [&](size_t i) {
            std::string pub;
            if (engine->getPublicData((*src)[i].metadataP, pub) != NIXL_SUCCESS) inner = NIXL_ERR_BACKEND;
            return pub;
        });
        return inner;
    };

    if (subset) {
        for (auto &kv : *subset) {
            auto it = sections_.find(kv.first);
            if (it == sections_.end()) return NIXL_ERR_NOT_FOUND;
            if (auto st = emit(kv.first, it->second, &kv.second); st != NIXL_SUCCESS) return st;
        }
    } else {
        for (auto &kv : sections_)
            if (auto st = emit(kv.first, kv.second, nullptr); st != NIXL_SUCCESS) return st;
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlLocalSection::serialize(nixlSerDes *ser) const { return serializeSubset(ser, nullptr); }

nixl_status_t nixlLocalSection::serializePartial(nixlSerDes *ser, const backend_set_t &engines,
                                                 const nixl_reg_dlist_t &descs) const {
    std::map<section_key_t, std::vector<int>> subset;
    if (!descs.isEmpty()) {
        for (nixlBackendEngine *engine : engines) {
            auto it = sections_.find({descs.getType(), engine});
            if (it == sections_.end()) continue;
            std::vector<int> pick;
            for (const auto &d : descs) {
                const int idx = it->second.getIndex(d);
                if (idx < 0) return NIXL_ERR_NOT_FOUND;
                pick.push_back(idx);
            }
            subset.emplace(it->first, std::move(pick));
        }
    }
    return serializeSubset(ser, &subset);
}

nixlLocalSection::~nixlLocalSection() {
    for (auto &kv : sections_)
        for (const auto &d : kv.second) kv.first.second->deregisterMem(d.metadataP);
}

// ------------------------------------------------------------------ nixlRemoteSection

namespace {
std::atomic<uint64_t> g_generation{1};
}

nixlRemoteSection::nixlRemoteSection(std::string agent) : agent_(std::move(agent)), generation_(g_generation.fetch_add(1)) {}

nixl_status_t nixlRemoteSection::loadRemoteData(nixlSerDes *des, const backend_map_t &engines) {
    size_t count = 0;
    if (des->getBuf("nixlSecElms", &count, sizeof(count)) != NIXL_SUCCESS) return NIXL_ERR_MISMATCH;
    if (count > des->remaining()) return NIXL_ERR_MISMATCH;
    for (size_t s = 0; s < count; ++s) {
        const std::string backend = des->getStr("bknd");
        if (backend.empty()) return NIXL_ERR_MISMATCH;
        nixl_reg_dlist_t wire(des);
        if (!wire.valid()) return NIXL_ERR_MISMATCH;
        auto eit = engines.find(backend);
        if (eit == engines.end()) continue; // a backend we do not run: ignore its registrations
        nixlBackendEngine *engine = eit->second;
        const nixl_mem_t mem = wire.getType();
        nixlSecDescList &sec = ensure(mem, engine);
        for (const auto &d : wire) {
            if (sec.getIndex(d) >= 0) continue; // already known (partial metadata re-sent)
            nixlBackendMD *md = nullptr;
            const nixl_status_t st = engine->loadRemoteMD(d, mem, agent_, md);
            if (st != NIXL_SUCCESS) {
                NIXL_ERROR << "backend " << backend << " rejected remote registration of agent " << agent_;
                dropIfEmpty(mem, engine);
                return st;
            }
            sec.addDesc(nixlSectionDesc(d, d.metaInfo, md));
        }
        dropIfEmpty(mem, engine);
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlRemoteSection::loadLocalData(nixl_mem_t mem, const std::vector<nixlSectionDesc> &regs,
                                               nixlBackendEngine *engine) {
    if (regs.empty()) return NIXL_ERR_INVALID_PARAM;
    nixlSecDescList &sec = ensure(mem, engine);
    for (const auto &r : regs) {
        nixlBackendMD *md = nullptr;
        const nixl_status_t st = engine->loadLocalMD(r.metadataP, md);
        if (st != NIXL_SUCCESS) return st;
        sec.addDesc(nixlSectionDesc(r, r.metaInfo, md));
    }
    return NIXL_SUCCESS;
}

nixl_status_t nixlRemoteSection::unloadLocalData(nixl_mem_t mem, const nixl_reg_dlist_t &descs, nixlBackendEngine *engine) {
    auto it = sections_.find({mem, engine});
    if (it == sections_.end()) return NIXL_ERR_NOT_FOUND;
    for (const auto &d : descs) {
        const int idx = it->second.getIndex(d);
        if (idx < 0) continue;
        engine->unloadMD(it->second[idx].metadataP);
        it->second.remDesc(idx);
    }
    dropIfEmpty(mem, engine);
    return NIXL_SUCCESS;
}

nixlRemoteSection::~nixlRemoteSection() {
    for (auto &kv : sections_)
        for (const auto &d : kv.second) kv.first.second->unloadMD(d.metadataP);
}
