#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include "utils/file/file_utils.h"

#include <cerrno>
#include <fcntl.h>
#include <sstream>
#include <sys/stat.h>
#include <system_error>
#include <unistd.h>

#include "utils/log.h"

namespace nixl {

std::optional<PathSpec> parsePathMeta(const std::string &meta) {
    const size_t colon = meta.find(':');
    if (colon == std::string::npos) return std::nullopt;
    std::vector<std::string> tokens;
    {
        std::istringstream in(meta.substr(0, colon));
        std::string t;
        while (std::getline(in, t, ',')) tokens.push_back(t);
    }
    if (tokens.empty()) return std::nullopt;
    PathSpec spec;
    if (tokens[0] == "ro") spec.flags = O_RDONLY;
    else if (tokens[0] == "rw") spec.flags = O_RDWR;
    else return std::nullopt;
    spec.path = meta.substr(colon + 1);
    if (spec.path.empty()) {
        NIXL_DEBUG << "path-mode string without a path: '" << meta << "'";
        return std::nullopt;
    }
    for (size_t i = 1; i < tokens.size(); ++i) {
        if (tokens[i] == "direct") spec.flags |= O_DIRECT;
        else if (tokens[i] == "sync") spec.flags |= O_SYNC;
        else if (tokens[i] == "noatime") spec.flags |= O_NOATIME;
        else if (tokens[i] == "create") {
            spec.flags |= O_CREAT;
            spec.mode = 0644;
        } else {
            NIXL_DEBUG << "path-mode string with unknown flag '" << tokens[i] << "'";
            return std::nullopt;
        }
    }
    return spec;
}

FileFd::FileFd(int fallback_fd, const std::string &meta) {
    auto spec = parsePathMeta(meta);
    if (!spec) {
        fd_ = fallback_fd;
        return;
    }
    const int fd = ::open(spec->path.c_str(), spec->flags | O_CLOEXEC, spec->mode);
    if (fd < 0) throw std::system_error(errno, std::generic_category(), "open(" + spec->path + ")");
    fd_ = fd;
    owned_ = true;
    path_ = spec->path;
}

FileFd::FileFd(FileFd &&o) noexcept : fd_(o.fd_), owned_(o.owned_), path_(std::move(o.path_)) {
    o.fd_ = -1;
    o.owned_ = false;
}

FileFd &FileFd::operator=(FileFd &&o) noexcept {
    if (this != &o) {
        if (owned_ && fd_ >= 0) ::close(fd_);
        fd_ = o.fd_;
        owned_ = o.owned_;
        path_ = std::move(o.path_);
        o.fd_ = -1;
        o.owned_ = false;
    }
    return *this;
}

FileFd::~FileFd() {
    if (owned_ && fd_ >= 0) ::close(fd_);
}

nixl_query_resp_t queryFileInfo(const std::string &name_or_meta) {
    std::string path = name_or_meta;
    if (auto spec = parsePathMeta(name_or_meta)) path = spec->path;
    if (path.empty()) return std::nullopt;
    struct stat st;
    if (::stat(path.c_str(), &st) != 0) return std::nullopt;
    nixl_b_params_t info;
    info["size"] = std::to_string(st.st_size);
    info["mode"] = std::to_string(st.st_mode);
    info["mtime"] = std::to_string(st.st_mtime);
    return info;
}

nixl_status_t queryFileInfoList(const std::vector<std::string> &names, std::vector<nixl_query_resp_t> &resp) {
    resp.clear();
    resp.reserve(names.size());
    for (const auto &n : names) resp.push_back(queryFileInfo(n));
    return NIXL_SUCCESS;
}

} // namespace nixl
