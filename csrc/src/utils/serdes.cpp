// Implementation of the tagged serializer; see serdes/serdes.h for the wire format.
#include "serdes/serdes.h"

#include <cstring>

#include "utils/log.h"

namespace {
constexpr char kMagic[] = "nixlSerDes|";
constexpr size_t kMagicLen = sizeof(kMagic) - 1;
} // namespace

nixlSerDes::nixlSerDes() : data_(kMagic), cursor_(kMagicLen) {}

std::string nixlSerDes::_bytesToString(const void *buf, ssize_t size) {
    return std::string(static_cast<const char *>(buf), static_cast<size_t>(size));
}

void nixlSerDes::_stringToBytes(void *fill_buf, const std::string &s, ssize_t size) {
    std::memcpy(fill_buf, s.data(), std::min(static_cast<size_t>(size), s.size()));
}

nixl_status_t nixlSerDes::addBuf(const std::string &tag, const void *buf, ssize_t len) {
    if (len < 0) return NIXL_ERR_INVALID_PARAM;
    const size_t n = static_cast<size_t>(len);
    data_.reserve(data_.size() + tag.size() + sizeof(n) + n + 1);
    data_.append(tag);
    data_.append(reinterpret_cast<const char *>(&n), sizeof(n));
    if (n) data_.append(static_cast<const char *>(buf), n);
    data_.push_back('|');
    return NIXL_SUCCESS;
}

nixl_status_t nixlSerDes::addStr(const std::string &tag, const std::string &str) {
    return addBuf(tag, str.data(), static_cast<ssize_t>(str.size()));
}

// Checks that the next field starts with `tag` and is fully present; yields its length.
bool nixlSerDes::headerOk(const std::string &tag, size_t &len) const {
    const size_t hdr = tag.size() + sizeof(size_t);
    if (data_.size() < cursor_ + hdr) {
        NIXL_ERROR << "serdes: truncated header while reading tag '" << tag << "'";
        return false;
    }
    if (std::memcmp(data_.data() + cursor_, tag.data(), tag.size()) != 0) {
        NIXL_ERROR << "serdes: expected tag '" << tag << "'";
        return false;
    }
    std::memcpy(&len, data_.data() + cursor_ + tag.size(), sizeof(len));
    // payload + trailing '|' must fit (written to avoid overflow on hostile lengths)
    const size_t avail = data_.size() - cursor_ - hdr;
    if (avail == 0 || len > avail - 1) {
        NIXL_ERROR << "serdes: truncated payload for tag '" << tag << "'";
        return false;
    }
    return true;
}

std::string nixlSerDes::getStr(const std::string &tag) {
    size_t len = 0;
    if (!headerOk(tag, len)) return "";
    const size_t start = cursor_ + tag.size() + sizeof(size_t);
    std::string out = data_.substr(start, len);
    cursor_ = start + len + 1;
    if (out.empty() && tag != "msg") NIXL_ERROR << "serdes: empty payload for tag '" << tag << "'";
    return out;
}

ssize_t nixlSerDes::getBufLen(const std::string &tag) const {
    size_t len = 0;
    if (!headerOk(tag, len)) return -1;
    return static_cast<ssize_t>(len);
}

nixl_status_t nixlSerDes::getBuf(const std::string &tag, void *buf, ssize_t len) {
    size_t stored = 0;
    if (!headerOk(tag, stored)) return NIXL_ERR_MISMATCH;
    if (len < 0 || stored != static_cast<size_t>(len)) {
        NIXL_ERROR << "serdes: length mismatch for tag '" << tag << "' (stored " << stored << ", asked " << len << ")";
        return NIXL_ERR_MISMATCH;
    }
    const size_t start = cursor_ + tag.size() + sizeof(size_t);
    if (stored) std::memcpy(buf, data_.data() + start, stored);
    cursor_ = start + stored + 1;
    return NIXL_SUCCESS;
}

std::string nixlSerDes::exportStr() const { return data_; }

nixl_status_t nixlSerDes::importStr(const std::string &blob) {
    if (blob.compare(0, kMagicLen, kMagic) != 0) {
        NIXL_ERROR << "serdes: blob does not start with the nixlSerDes magic";
        return NIXL_ERR_MISMATCH;
    }
    data_ = blob;
    cursor_ = kMagicLen;
    return NIXL_SUCCESS;
}
