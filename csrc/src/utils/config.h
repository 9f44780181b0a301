// Configuration lookup: environment variable first, then a TOML-style file.
//
// Behavioural parity with the reference's src/utils/common/configuration.cpp:44-84:
// the file is the first that exists of $NIXL_CONFIG_FILE, $HOME/.nixl.cfg, /etc/nixl.cfg.
// A key NIXL_FOO_BAR is looked up in the file as top-level "NIXL_FOO_BAR" and, failing
// that, as lower-case "foo_bar" (optionally under a [nixl] table).  Only the scalar
// subset of TOML is read: strings, integers, floats, booleans, `#` comments, [tables].
#ifndef NIXL_B200_CONFIG_H
#define NIXL_B200_CONFIG_H

#include <optional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace nixl::config {

// Raw string value or nullopt.
std::optional<std::string> lookup(const std::string &env_name);
// Drop the cached file contents (tests change NIXL_CONFIG_FILE between cases).
void reload();

template<class T> std::optional<T> convert(const std::string &raw) {
    if constexpr (std::is_same_v<T, std::string>) {
        return raw;
    } else if constexpr (std::is_same_v<T, bool>) {
        std::string s;
        for (char c : raw) s.push_back(static_cast<char>(std::tolower(static_cast<unsigned char>(c))));
        if (s == "1" || s == "y" || s == "yes" || s == "on" || s == "true") return true;
        if (s == "0" || s == "n" || s == "no" || s == "off" || s == "false") return false;
        return std::nullopt;
    } else {
        std::istringstream in(raw);
        T v{};
        in >> v;
        if (in.fail()) return std::nullopt;
        in >> std::ws;
        if (!in.eof()) return std::nullopt;
        return v;
    }
}

// Value if set and well-formed; nullopt if unset; throws std::runtime_error if malformed.
template<class T> std::optional<T> getValueOptional(const std::string &env_name) {
    auto raw = lookup(env_name);
    if (!raw) return std::nullopt;
    auto v = convert<T>(*raw);
    if (!v) throw std::runtime_error("configuration value of " + env_name + " is malformed: '" + *raw + "'");
    return v;
}
template<class T> T getValue(const std::string &env_name) {
    auto v = getValueOptional<T>(env_name);
    if (!v) throw std::runtime_error("configuration value " + env_name + " is not set");
    return *v;
}
template<class T> T getValueDefaulted(const std::string &env_name, const T &fallback) {
    try {
        auto v = getValueOptional<T>(env_name);
        return v ? *v : fallback;
    } catch (const std::exception &) {
        return fallback;
    }
}
} // namespace nixl::config

#endif
