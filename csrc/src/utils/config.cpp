#include "utils/config.h"

#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sys/stat.h>

#include "utils/log.h"

namespace nixl::config {
namespace {
std::mutex g_mu;
bool g_loaded = false;
std::map<std::string, std::string> g_file; // flattened "table.key" -> value

std::string strip(const std::string &s) {
    const size_t b = s.find_first_not_of(" \t\r\n");
    if (b == std::string::npos) return "";
    const size_t e = s.find_last_not_of(" \t\r\n");
    return s.substr(b, e - b + 1);
}

// Remove a trailing comment that is not inside quotes.
std::string dropComment(const std::string &line) {
    char quote = 0;
    for (size_t i = 0; i < line.size(); ++i) {
        const char c = line[i];
        if (quote) {
            if (c == '\\' && quote == '"') ++i;
            else if (c == quote) quote = 0;
        } else if (c == '"' || c == '\'') quote = c;
        else if (c == '#') return line.substr(0, i);
    }
    return line;
}

std::string unquote(const std::string &v) {
    if (v.size() >= 2 && ((v.front() == '"' && v.back() == '"') || (v.front() == '\'' && v.back() == '\''))) {
        const bool basic = v.front() == '"';
        std::string out;
        for (size_t i = 1; i + 1 < v.size(); ++i) {
            if (basic && v[i] == '\\' && i + 2 < v.size()) {
                const char n = v[++i];
                out.push_back(n == 'n' ? '\n' : n == 't' ? '\t' : n);
            } else out.push_back(v[i]);
        }
        return out;
    }
    return v;
}

bool fileExists(const std::string &p) {
    struct stat st;
    return !p.empty() && ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

std::string locate() {
    if (const char *e = std::getenv("NIXL_CONFIG_FILE"); e && *e) {
        if (fileExists(e)) return e;
        NIXL_WARN << "NIXL_CONFIG_FILE=" << e << " does not name a readable file";
        return "";
    }
    if (const char *h = std::getenv("HOME"); h && *h) {
        const std::string p = std::string(h) + "/.nixl.cfg";
        if (fileExists(p)) return p;
    }
    return fileExists("/etc/nixl.cfg") ? "/etc/nixl.cfg" : "";
}

void loadLocked() {
    g_loaded = true;
    g_file.clear();
    const std::string path = locate();
    if (path.empty()) return;
    std::ifstream in(path);
    std::string line, table;
    int lineno = 0;
    while (std::getline(in, line)) {
        ++lineno;
        line = strip(dropComment(line));
        if (line.empty()) continue;
        if (line.front() == '[') {
            if (line.back() != ']') {
                NIXL_WARN << path << ":" << lineno << ": malformed table header";
                continue;
            }
            table = strip(line.substr(1, line.size() - 2));
            continue;
        }
        const size_t eq = line.find('=');
        if (eq == std::string::npos) {
            NIXL_WARN << path << ":" << lineno << ": expected key = value";
            continue;
        }
        const std::string key = unquote(strip(line.substr(0, eq)));
        const std::string val = unquote(strip(line.substr(eq + 1)));
        g_file[table.empty() ? key : table + "." + key] = val;
    }
}

std::string lower(std::string s) {
    for (auto &c : s) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
    return s;
}
} // namespace

void reload() {
    std::lock_guard<std::mutex> g(g_mu);
    g_loaded = false;
}

std::optional<std::string> lookup(const std::string &env_name) {
    if (const char *e = std::getenv(env_name.c_str())) return std::string(e);
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_loaded) loadLocked();
    if (g_file.empty()) return std::nullopt;
    std::string shortName = lower(env_name);
    if (shortName.rfind("nixl_", 0) == 0) shortName = shortName.substr(5);
    for (const std::string &k : {env_name, shortName, "nixl." + shortName, "nixl." + env_name}) {
        auto it = g_file.find(k);
        if (it != g_file.end()) return it->second;
    }
    return std::nullopt;
}
} // namespace nixl::config
