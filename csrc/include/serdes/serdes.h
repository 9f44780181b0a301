// Tagged, length-prefixed byte serializer used for every metadata blob.
//
// Wire format (byte-compatible with the reference's src/utils/serdes/serdes.cpp:22-47):
//   "nixlSerDes|"  then repeated fields  <tag bytes><u64 length, host endian><payload>'|'
// Tags are not self-describing: the reader must ask for the tags in the order
// the writer added them.
#ifndef NIXL_B200_SERDES_H
#define NIXL_B200_SERDES_H

#include <string>
#include <sys/types.h>
#include "nixl_types.h"

class nixlSerDes {
public:
    nixlSerDes();

    // Append a string / raw buffer field.
    nixl_status_t addStr(const std::string &tag, const std::string &str);
    nixl_status_t addBuf(const std::string &tag, const void *buf, ssize_t len);

    // Read the next field, which must carry `tag`.  getStr returns "" on any
    // framing error (an empty payload is only legal for tag "msg").
    std::string getStr(const std::string &tag);
    // Length of the next field without consuming it, or -1.
    ssize_t getBufLen(const std::string &tag) const;
    // Read the next field into buf; `len` must equal the stored length.
    nixl_status_t getBuf(const std::string &tag, void *buf, ssize_t len);

    std::string exportStr() const;
    nixl_status_t importStr(const std::string &blob);

    // Bytes not yet consumed by the reader.
    size_t remaining() const { return data_.size() - cursor_; }

    // Helpers for shipping arbitrary bytes through text-only channels.
    static std::string _bytesToString(const void *buf, ssize_t size);
    static void _stringToBytes(void *fill_buf, const std::string &s, ssize_t size);

private:
    bool headerOk(const std::string &tag, size_t &len) const;
    std::string data_;
    size_t cursor_;
};

#endif
