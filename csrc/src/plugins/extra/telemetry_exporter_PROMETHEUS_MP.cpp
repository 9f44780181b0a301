// PROMETHEUS_MP telemetry exporter: one scrape endpoint for many processes of a node.
//
// Every exporter (one per agent, any number per process) keeps its metrics in a small file of its
// own, mapped shared, under NIXL_TELEMETRY_MULTIPROC_DIR (default /tmp/nixl_prometheus_mp).
// Whoever holds the advisory lock on <dir>/owner.lock serves http://<addr>:<port>/metrics and
// renders all files it finds there; the others keep trying for the lock once a second, so the
// endpoint survives the death of its owner.  Files of processes that no longer exist are removed
// by the owner.  Same port and bind variables as the single-process exporter
// (NIXL_TELEMETRY_PROMETHEUS_PORT, NIXL_TELEMETRY_PROMETHEUS_LOCAL).
//
// Role parity with the reference's src/plugins/telemetry/prometheus_mp (mmap store, flock owner
// election, scrape endpoint); the file format and the HTTP responder are this build's own.
#include <arpa/inet.h>
#include <dirent.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <poll.h>
#include <signal.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <sstream>
#include <thread>
#include <vector>

#include "core/telemetry/telemetry.h"
#include "telemetry/telemetry_plugin.h"
#include "utils/config.h"

namespace {

constexpr uint64_t kMagic = 0x31504d504c58494eull; // "NIXLPMP1"
constexpr size_t kTypes = nixl_telemetry_event_type_count;
constexpr size_t kMaxBuckets = 32;

// One exporter's metrics.  The writer bumps `seq` to odd, updates, bumps to even; readers retry on change.
struct Store {
    uint64_t magic;
    std::atomic<uint64_t> seq;
    int64_t pid;
    char agent[96];
    uint64_t nbuckets;
    uint64_t buckets[kMaxBuckets];
    uint64_t total[kTypes], last[kTypes], count[kTypes];
    uint64_t hist[kTypes][kMaxBuckets + 1];
};

bool isTime(size_t t) {
    return t == static_cast<size_t>(nixl_telemetry_event_type_t::AGENT_XFER_TIME) || t == static_cast<size_t>(nixl_telemetry_event_type_t::AGENT_XFER_POST_TIME);
}
bool isError(size_t t) { return t >= 8 && t <= 19; }

void renderOne(std::ostringstream &o, const Store &s) {
    const std::string label = std::string("{agent=\"") + s.agent + "\",pid=\"" + std::to_string(s.pid) + "\"";
    for (size_t t = 8; t <= 19 && t < kTypes; ++t) {
        const std::string name(nixlEnumStrings::telemetryEventTypeStr(static_cast<nixl_telemetry_event_type_t>(t)));
        o << "agent_errors_total" << label << ",status=\"" << name.substr(10) << "\"} " << s.total[t] << "\n";
    }
    for (size_t t = 0; t < kTypes; ++t) {
        if (isError(t)) continue;
        const std::string name(nixlEnumStrings::telemetryEventTypeStr(static_cast<nixl_telemetry_event_type_t>(t)));
        if (isTime(t)) {
            uint64_t cum = 0;
            for (size_t b = 0; b < s.nbuckets; ++b) {
                cum += s.hist[t][b];
                o << name << "_us_bucket" << label << ",le=\"" << s.buckets[b] << "\"} " << cum << "\n";
            }
            cum += s.hist[t][s.nbuckets];
            o << name << "_us_bucket" << label << ",le=\"+Inf\"} " << cum << "\n";
            o << name << "_us_sum" << label << "} " << s.total[t] << "\n" << name << "_us_count" << label << "} " << s.count[t] << "\n";
        } else {
            o << name << "_total" << label << "} " << s.total[t] << "\n";
            o << name << "_last" << label << "} " << s.last[t] << "\n";
        }
    }
}

class PrometheusMpExporter final : public nixlTelemetryExporter {
public:
    explicit PrometheusMpExporter(const nixlTelemetryExporterInitParams &p) : nixlTelemetryExporter(p) {
        // NIXL_TELEMETRY_MULTIPROC_DIR is the reference's name for the directory; the longer name is accepted too.
        dir_ = nixl::config::getValueDefaulted<std::string>(
            "NIXL_TELEMETRY_MULTIPROC_DIR", nixl::config::getValueDefaulted<std::string>("NIXL_TELEMETRY_PROMETHEUS_MP_DIR", "/tmp/nixl_prometheus_mp"));
        port_ = nixl::config::getValueDefaulted<int>("NIXL_TELEMETRY_PROMETHEUS_PORT", 9090);
        local_ = nixl::config::getValueDefaulted<bool>("NIXL_TELEMETRY_PROMETHEUS_LOCAL", false);
        ::mkdir(dir_.c_str(), 0777);
        static std::atomic<unsigned> serial{0};
        path_ = dir_ + "/" + std::to_string(::getpid()) + "_" + std::to_string(serial++) + ".prom";
        const int fd = ::open(path_.c_str(), O_RDWR | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
        if (fd < 0 || ::ftruncate(fd, sizeof(Store)) != 0) {
            if (fd >= 0) ::close(fd);
            throw nixlTelemetryBindFailed("prometheus_mp exporter cannot create " + path_);
        }
        void *m = ::mmap(nullptr, sizeof(Store), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        ::close(fd);
        if (m == MAP_FAILED) throw nixlTelemetryBindFailed("prometheus_mp exporter cannot map " + path_);
        store_ = new (m) Store();
        const auto buckets = nixlTelemetryHistogramBucketsUs();
        store_->nbuckets = std::min(buckets.size(), kMaxBuckets);
        for (size_t b = 0; b < store_->nbuckets; ++b) store_->buckets[b] = buckets[b];
        store_->pid = ::getpid();
        std::strncpy(store_->agent, p.agentName.c_str(), sizeof(store_->agent) - 1);
        store_->seq.store(0, std::memory_order_release);
        store_->magic = kMagic;
        lockFd_ = ::open((dir_ + "/owner.lock").c_str(), O_RDWR | O_CREAT | O_CLOEXEC, 0666);
        th_ = std::thread([this] { run(); });
    }
    ~PrometheusMpExporter() override {
        stop_ = true;
        if (th_.joinable()) th_.join();
        if (listenFd_ >= 0) ::close(listenFd_);
        if (lockFd_ >= 0) ::close(lockFd_); // releases the lock if we held it
        if (store_) ::munmap(store_, sizeof(Store));
        ::unlink(path_.c_str());
    }

    nixl_status_t exportEvent(const nixlTelemetryEvent &e) override {
        const auto t = static_cast<size_t>(e.eventType_);
        if (t >= kTypes) return NIXL_ERR_INVALID_PARAM;
        store_->seq.fetch_add(1, std::memory_order_acq_rel);
        store_->total[t] += e.value_;
        store_->last[t] = e.value_;
        ++store_->count[t];
        if (isTime(t)) {
            size_t b = 0;
            while (b < store_->nbuckets && e.value_ > store_->buckets[b]) ++b;
            ++store_->hist[t][b];
        }
        store_->seq.fetch_add(1, std::memory_order_acq_rel);
        return NIXL_SUCCESS;
    }

private:
    // A consistent copy of another exporter's file; false if it is not (yet) a valid store.
    static bool snapshot(const std::string &path, Store &out) {
        const int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
        if (fd < 0) return false;
        struct stat st {};
        if (::fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(Store)) {
            ::close(fd);
            return false;
        }
        void *m = ::mmap(nullptr, sizeof(Store), PROT_READ, MAP_SHARED, fd, 0);
        ::close(fd);
        if (m == MAP_FAILED) return false;
        const Store *s = static_cast<const Store *>(m);
        bool ok = false;
        for (int tries = 0; tries < 100 && !ok; ++tries) {
            const uint64_t a = s->seq.load(std::memory_order_acquire);
            if (a & 1) continue;
            std::memcpy(static_cast<void *>(&out), s, sizeof(Store));
            ok = s->seq.load(std::memory_order_acquire) == a && out.magic == kMagic;
        }
        ::munmap(m, sizeof(Store));
        return ok;
    }

    std::string render() const {
        std::ostringstream o;
        o << "# metrics of every NIXL exporter under " << dir_ << "\n";
        DIR *d = ::opendir(dir_.c_str());
        if (!d) return o.str();
        while (dirent *e = ::readdir(d)) {
            const std::string name = e->d_name;
            if (name.size() < 6 || name.compare(name.size() - 5, 5, ".prom") != 0) continue;
            const std::string path = dir_ + "/" + name;
            Store s;
            if (!snapshot(path, s)) continue;
            if (::kill(static_cast<pid_t>(s.pid), 0) != 0 && errno == ESRCH) {
                ::unlink(path.c_str()); // its process is gone
                continue;
            }
            s.agent[sizeof(s.agent) - 1] = 0;
            s.nbuckets = std::min<uint64_t>(s.nbuckets, kMaxBuckets);
            renderOne(o, s);
        }
        ::closedir(d);
        return o.str();
    }

    bool becomeOwner() {
        if (lockFd_ < 0 || ::flock(lockFd_, LOCK_EX | LOCK_NB) != 0) return false;
        const int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
        int one = 1;
        setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_addr.s_addr = htonl(local_ ? INADDR_LOOPBACK : INADDR_ANY);
        a.sin_port = htons(static_cast<uint16_t>(port_));
        if (fd < 0 || ::bind(fd, reinterpret_cast<sockaddr *>(&a), sizeof(a)) != 0 || ::listen(fd, 16) != 0) {
            if (fd >= 0) ::close(fd);
            ::flock(lockFd_, LOCK_UN); // somebody outside this scheme has the port: let another process try later
            return false;
        }
        listenFd_ = fd;
        return true;
    }

    void run() {
        auto next_try = std::chrono::steady_clock::now();
        while (!stop_) {
            if (listenFd_ < 0) {
                if (std::chrono::steady_clock::now() >= next_try) {
                    becomeOwner();
                    next_try = std::chrono::steady_clock::now() + std::chrono::seconds(1);
                }
                if (listenFd_ < 0) {
                    std::this_thread::sleep_for(std::chrono::milliseconds(50));
                    continue;
                }
            }
            pollfd pf{listenFd_, POLLIN, 0};
            if (::poll(&pf, 1, 100) <= 0) continue;
            const int c = ::accept(listenFd_, nullptr, nullptr);
            if (c < 0) continue;
            char req[2048];
            pollfd cp{c, POLLIN, 0};
            if (::poll(&cp, 1, 500) > 0) (void)!::recv(c, req, sizeof(req), 0);
            const std::string body = render();
            std::ostringstream o;
            o << "HTTP/1.1 200 OK\r\nContent-Type: text/plain; version=0.0.4\r\nContent-Length: " << body.size() << "\r\nConnection: close\r\n\r\n" << body;
            const std::string resp = o.str();
            size_t off = 0;
            while (off < resp.size()) {
                const ssize_t w = ::send(c, resp.data() + off, resp.size() - off, MSG_NOSIGNAL);
                if (w <= 0) break;
                off += static_cast<size_t>(w);
            }
            ::close(c);
        }
    }

    std::string dir_, path_;
    int port_ = 9090;
    bool local_ = false;
    Store *store_ = nullptr;
    int lockFd_ = -1, listenFd_ = -1;
    std::atomic<bool> stop_{false};
    std::thread th_;
};

nixlTelemetryPlugin g_table = {NIXL_TELEMETRY_PLUGIN_API_VERSION,
                               [](const nixlTelemetryExporterInitParams *p) -> nixlTelemetryExporter * {
                                   try {
                                       return new PrometheusMpExporter(*p);
                                   } catch (const std::exception &) {
                                       return nullptr;
                                   }
                               },
                               [](nixlTelemetryExporter *e) { delete e; }, [] { return "PROMETHEUS_MP"; }, [] { return "1.0.0"; }};
} // namespace

extern "C" __attribute__((visibility("default"))) nixlTelemetryPlugin *nixl_telemetry_plugin_init() { return &g_table; }
extern "C" __attribute__((visibility("default"))) void nixl_telemetry_plugin_fini() {}
