// Drains the telemetry ring an agent writes when NIXL_TELEMETRY_ENABLE=1 and
// NIXL_TELEMETRY_DIR=<dir> are set (BUFFER exporter: one file <dir>/<agent name>) and prints the
// events.  Counterpart of the reference's examples/cpp/telemetry_reader.cpp.  The file is a
// single-producer / single-consumer ring: a 64-byte header (magic 'NXRB', format version, record
// size, capacity, head, tail, dropped) followed by the records (timestamp in microseconds, event
// type, value); the reader consumes by advancing `tail`.
//
//   g++ -std=c++20 -I csrc/include examples/cpp/telemetry_reader.cpp -o telemetry_reader
//   ./telemetry_reader <dir>/<agent> [--follow]
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

#include "telemetry/telemetry_event.h"

namespace {

struct RingHeader {
    uint32_t magic, version, record_size, capacity;
    std::atomic<uint64_t> head, tail, dropped;
    uint8_t pad[24];
};
static_assert(sizeof(RingHeader) == 64, "ring header is 64 bytes");

struct Record {
    uint64_t timestamp_us;
    uint32_t type;
    uint32_t pad;
    uint64_t value;
};

const char *eventName(uint32_t t) {
    static const char *names[] = {"agent_tx_bytes", "agent_rx_bytes", "agent_tx_requests_num", "agent_rx_requests_num",
                                  "agent_memory_registered", "agent_memory_deregistered", "agent_xfer_time", "agent_xfer_post_time",
                                  "agent_err_not_posted", "agent_err_invalid_param", "agent_err_backend", "agent_err_not_found",
                                  "agent_err_mismatch", "agent_err_not_allowed", "agent_err_repost_active", "agent_err_unknown",
                                  "agent_err_not_supported", "agent_err_remote_disconnect", "agent_err_canceled", "agent_err_no_telemetry",
                                  "agent_telemetry_events_dropped"};
    return t < sizeof(names) / sizeof(names[0]) ? names[t] : "event";
}

} // namespace

int main(int argc, char **argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s <NIXL_TELEMETRY_DIR>/<agent> [--follow]\n", argv[0]);
        return 2;
    }
    const bool follow = argc > 2 && std::strcmp(argv[2], "--follow") == 0;
    const int fd = ::open(argv[1], O_RDWR);
    struct stat st;
    if (fd < 0 || ::fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(RingHeader)) {
        std::fprintf(stderr, "cannot open %s as a telemetry ring\n", argv[1]);
        return 1;
    }
    void *map = ::mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (map == MAP_FAILED) return 1;
    auto *hdr = static_cast<RingHeader *>(map);
    if (hdr->magic != 0x4E585242u || hdr->record_size < sizeof(Record)) {
        std::fprintf(stderr, "%s is not a telemetry ring\n", argv[1]);
        return 1;
    }
    std::printf("# format version %u, %u slots of %u bytes\n", hdr->version, hdr->capacity, hdr->record_size);
    const char *records = static_cast<const char *>(map) + sizeof(RingHeader);
    uint64_t seen = 0;
    for (;;) {
        uint64_t tail = hdr->tail.load(std::memory_order_relaxed);
        const uint64_t head = hdr->head.load(std::memory_order_acquire);
        for (; tail < head; ++tail, ++seen) {
            Record r;
            std::memcpy(&r, records + (tail % hdr->capacity) * hdr->record_size, sizeof(r));
            std::printf("%.6f %s %llu\n", static_cast<double>(r.timestamp_us) / 1e6, eventName(r.type), static_cast<unsigned long long>(r.value));
        }
        hdr->tail.store(tail, std::memory_order_release); // consumed: the writer may reuse the slots
        if (!follow) break;
        std::fflush(stdout);
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    if (const uint64_t dropped = hdr->dropped.load()) std::printf("# %llu events were dropped because the ring was full\n", static_cast<unsigned long long>(dropped));
    std::printf("# %llu events\n", static_cast<unsigned long long>(seen));
    ::munmap(map, static_cast<size_t>(st.st_size));
    ::close(fd);
    return 0;
}
