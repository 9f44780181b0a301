// NVTX trace backend: spans become NVTX ranges in a per-agent domain, coloured by kind, with
// the correlation id as payload; marks become NVTX marks.  Header-only NVTX3: without a
// profiler attached every call is a no-op.  Parity: the reference's src/plugins/tracing/nvtx.
#include <nvtx3/nvToolsExt.h>

#include <string>

#include "core/tracing/trace.h"

namespace {
using namespace nixl::trace;

uint32_t colourOf(Kind k) {
    static const uint32_t c[] = {0xFF4C9AFF, 0xFF36B37E, 0xFFFFAB00, 0xFFFF5630, 0xFF6554C0, 0xFF00B8D9, 0xFF8777D9, 0xFF97A0AF, 0xFF505F79};
    const auto i = static_cast<uint32_t>(k);
    return c[i < 9 ? i : 8];
}

class NvtxBackend final : public Backend {
public:
    explicit NvtxBackend(const char *agent) : domain_(nvtxDomainCreateA((std::string("nixl.") + agent).c_str())) {}
    ~NvtxBackend() override { nvtxDomainDestroy(domain_); }
    const char *name() const override { return "nvtx"; }
    void spanBegin(const std::string &, Kind kind, const char *what, uint64_t corr) override {
        nvtxEventAttributes_t a = attrs(kind, what, corr);
        nvtxDomainRangePushEx(domain_, &a);
    }
    void spanEnd(const std::string &, Kind, const char *, uint64_t) override { nvtxDomainRangePop(domain_); }
    void mark(const std::string &, Kind kind, const char *what, uint64_t corr) override {
        nvtxEventAttributes_t a = attrs(kind, what, corr);
        nvtxDomainMarkEx(domain_, &a);
    }

private:
    static nvtxEventAttributes_t attrs(Kind kind, const char *what, uint64_t corr) {
        nvtxEventAttributes_t a{};
        a.version = NVTX_VERSION;
        a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
        a.colorType = NVTX_COLOR_ARGB;
        a.color = colourOf(kind);
        a.messageType = NVTX_MESSAGE_TYPE_ASCII;
        a.message.ascii = what;
        a.payloadType = NVTX_PAYLOAD_TYPE_UNSIGNED_INT64;
        a.payload.ullValue = corr;
        a.category = static_cast<uint32_t>(kind);
        return a;
    }
    nvtxDomainHandle_t domain_;
};

TracePlugin g_table = {NIXL_TRACE_PLUGIN_API_VERSION, [](const char *agent) -> Backend * { return new NvtxBackend(agent); },
                       [](Backend *b) { delete b; }, [] { return "nvtx"; }};
} // namespace

extern "C" __attribute__((visibility("default"))) void *nixl_trace_plugin_init() { return &g_table; }
