// PROMETHEUS telemetry exporter: keeps counters / gauges / histograms per event type and serves
// them in the text exposition format on http://<addr>:<port>/metrics.
//
// Behavioural parity with the reference's src/plugins/telemetry/prometheus (port from
// NIXL_TELEMETRY_PROMETHEUS_PORT, default 9090; NIXL_TELEMETRY_PROMETHEUS_LOCAL=y binds loopback
// only; error events share the family agent_errors_total with a `status` label; time events are
// histograms with the default buckets 10 us .. 10 s).  The reference links prometheus-cpp; this
// one carries its own minimal HTTP responder.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <array>
#include <atomic>
#include <cstring>
#include <mutex>
#include <sstream>
#include <thread>
#include <vector>

#include "core/telemetry/telemetry.h"
#include "telemetry/telemetry_plugin.h"
#include "utils/config.h"

namespace {

class PrometheusExporter final : public nixlTelemetryExporter {
public:
    explicit PrometheusExporter(const nixlTelemetryExporterInitParams &p) : nixlTelemetryExporter(p), buckets_(nixlTelemetryHistogramBucketsUs()) {
        for (auto &h : hist_) h.assign(buckets_.size() + 1, 0);
        const int port = nixl::config::getValueDefaulted<int>("NIXL_TELEMETRY_PROMETHEUS_PORT", 9090);
        const bool local = nixl::config::getValueDefaulted<bool>("NIXL_TELEMETRY_PROMETHEUS_LOCAL", false);
        fd_ = ::socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK, 0);
        int one = 1;
        setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in a{};
        a.sin_family = AF_INET;
        a.sin_addr.s_addr = htonl(local ? INADDR_LOOPBACK : INADDR_ANY);
        a.sin_port = htons(static_cast<uint16_t>(port));
        if (fd_ < 0 || ::bind(fd_, reinterpret_cast<sockaddr *>(&a), sizeof(a)) != 0 || ::listen(fd_, 16) != 0) {
            if (fd_ >= 0) ::close(fd_);
            throw nixlTelemetryBindFailed("prometheus exporter cannot bind port " + std::to_string(port));
        }
        th_ = std::thread([this] { serve(); });
    }
    ~PrometheusExporter() override {
        stop_ = true;
        if (th_.joinable()) th_.join();
        ::close(fd_);
    }

    nixl_status_t exportEvent(const nixlTelemetryEvent &e) override {
        const auto t = static_cast<size_t>(e.eventType_);
        if (t >= nixl_telemetry_event_type_count) return NIXL_ERR_INVALID_PARAM;
        std::lock_guard<std::mutex> g(mu_);
        total_[t] += e.value_;
        last_[t] = e.value_;
        ++count_[t];
        if (isTime(e.eventType_)) {
            size_t b = 0;
            while (b < buckets_.size() && e.value_ > buckets_[b]) ++b;
            ++hist_[t][b];
        }
        return NIXL_SUCCESS;
    }

private:
    static bool isTime(nixl_telemetry_event_type_t t) {
        return t == nixl_telemetry_event_type_t::AGENT_XFER_TIME || t == nixl_telemetry_event_type_t::AGENT_XFER_POST_TIME;
    }
    static bool isError(size_t t) { return t >= 8 && t <= 19; }

    std::string render() {
        std::lock_guard<std::mutex> g(mu_);
        std::ostringstream o;
        const std::string label = "{agent=\"" + agentName() + "\"";
        o << "# HELP agent_errors_total Cumulative error count by status\n# TYPE agent_errors_total counter\n";
        for (size_t t = 8; t <= 19; ++t) {
            const std::string name(nixlEnumStrings::telemetryEventTypeStr(static_cast<nixl_telemetry_event_type_t>(t)));
            o << "agent_errors_total" << label << ",status=\"" << name.substr(10) << "\"} " << total_[t] << "\n";
        }
        for (size_t t = 0; t < nixl_telemetry_event_type_count; ++t) {
            if (isError(t)) continue;
            const auto type = static_cast<nixl_telemetry_event_type_t>(t);
            const std::string name(nixlEnumStrings::telemetryEventTypeStr(type));
            if (isTime(type)) {
                o << "# TYPE " << name << "_us histogram\n";
                uint64_t cum = 0;
                for (size_t b = 0; b < buckets_.size(); ++b) {
                    cum += hist_[t][b];
                    o << name << "_us_bucket" << label << ",le=\"" << buckets_[b] << "\"} " << cum << "\n";
                }
                cum += hist_[t][buckets_.size()];
                o << name << "_us_bucket" << label << ",le=\"+Inf\"} " << cum << "\n";
                o << name << "_us_sum" << label << "} " << total_[t] << "\n" << name << "_us_count" << label << "} " << count_[t] << "\n";
            } else {
                o << "# TYPE " << name << "_total counter\n" << name << "_total" << label << "} " << total_[t] << "\n";
                o << "# TYPE " << name << "_last gauge\n" << name << "_last" << label << "} " << last_[t] << "\n";
            }
        }
        return o.str();
    }

    void serve() {
        while (!stop_) {
            pollfd pf{fd_, POLLIN, 0};
            if (::poll(&pf, 1, 100) <= 0) continue;
            const int c = ::accept(fd_, nullptr, nullptr);
            if (c < 0) continue;
            char req[2048];
            pollfd cp{c, POLLIN, 0};
            if (::poll(&cp, 1, 500) > 0) (void)!::recv(c, req, sizeof(req), 0);
            const std::string body = render();
            std::ostringstream o;
            o << "HTTP/1.1 200 OK\r\nContent-Type: text/plain; version=0.0.4\r\nContent-Length: " << body.size()
              << "\r\nConnection: close\r\n\r\n"
              << body;
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

    std::vector<uint64_t> buckets_;
    std::mutex mu_;
    std::array<uint64_t, nixl_telemetry_event_type_count> total_{}, last_{}, count_{};
    std::array<std::vector<uint64_t>, nixl_telemetry_event_type_count> hist_;
    int fd_ = -1;
    std::atomic<bool> stop_{false};
    std::thread th_;
};

nixlTelemetryPlugin g_table = {NIXL_TELEMETRY_PLUGIN_API_VERSION,
                               [](const nixlTelemetryExporterInitParams *p) -> nixlTelemetryExporter * {
                                   try {
                                       return new PrometheusExporter(*p);
                                   } catch (const std::exception &) {
                                       return nullptr;
                                   }
                               },
                               [](nixlTelemetryExporter *e) { delete e; }, [] { return "PROMETHEUS"; }, [] { return "1.0.0"; }};
} // namespace

extern "C" __attribute__((visibility("default"))) nixlTelemetryPlugin *nixl_telemetry_plugin_init() { return &g_table; }
extern "C" __attribute__((visibility("default"))) void nixl_telemetry_plugin_fini() {}
