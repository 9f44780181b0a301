// File helpers shared by storage backends.
//
// Path-mode registration string (behavioural parity with the reference's
// src/utils/file/file_path_mode.cpp:34-81):  "<ro|rw>[,direct][,sync][,noatime][,create]:<path>"
// A registration whose metaInfo parses as such makes the backend open the file itself; any
// other metaInfo means the descriptor's devId already is an open file descriptor.
#ifndef NIXL_B200_FILE_UTILS_H
#define NIXL_B200_FILE_UTILS_H

#include <optional>
#include <string>
#include <sys/types.h>
#include <vector>

#include "nixl_types.h"

namespace nixl {

struct PathSpec {
    std::string path;
    int flags = 0;
    mode_t mode = 0;
};

std::optional<PathSpec> parsePathMeta(const std::string &meta);

// Owns an fd only when it opened it (path mode).
class FileFd {
public:
    FileFd() = default;
    // Path mode when `meta` parses; otherwise adopts `fallback_fd` without owning it.
    // Throws std::system_error if the open fails.
    FileFd(int fallback_fd, const std::string &meta);
    FileFd(FileFd &&o) noexcept;
    FileFd &operator=(FileFd &&o) noexcept;
    FileFd(const FileFd &) = delete;
    FileFd &operator=(const FileFd &) = delete;
    ~FileFd();
    int fd() const { return fd_; }
    bool owned() const { return owned_; }
    const std::string &path() const { return path_; }

private:
    int fd_ = -1;
    bool owned_ = false;
    std::string path_;
};

// stat() results as strings: size, mode, mtime; nullopt when the file does not exist.
// Accepts a plain path or a path-mode string.
nixl_query_resp_t queryFileInfo(const std::string &name_or_meta);
nixl_status_t queryFileInfoList(const std::vector<std::string> &names, std::vector<nixl_query_resp_t> &resp);

} // namespace nixl

#endif
