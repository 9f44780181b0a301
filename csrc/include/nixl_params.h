// Agent-wide configuration.
//
// API parity: field names and defaults follow the reference's
// src/api/cpp/nixl_params.h:29-108 (progress thread, listener thread and port,
// sync mode, telemetry capture, thread delays, etcd watch timeout).
#ifndef NIXL_B200_PARAMS_H
#define NIXL_B200_PARAMS_H

#include <chrono>
#include <cstdint>
#include "nixl_types.h"

class nixlAgentConfig {
public:
    static constexpr bool kDefaultUseProgThread = false;
    static constexpr bool kDefaultUseListenThread = false;
    static constexpr uint16_t kDefaultListenPort = 0;
    static constexpr nixl_thread_sync_t kDefaultSyncMode = nixl_thread_sync_t::NIXL_THREAD_SYNC_DEFAULT;
    static constexpr bool kDefaultCaptureTelemetry = false;
    static constexpr uint64_t kDefaultPthrDelayUs = 0;
    static constexpr uint64_t kDefaultLthrDelayUs = 100000;
    static constexpr std::chrono::microseconds kDefaultEtcdWatchTimeout{5000000};

    // Backends may run a progress thread that completes transfers and delivers
    // notifications without the user polling.
    bool useProgThread = kDefaultUseProgThread;
    // A TCP listener thread that serves peer-to-peer metadata requests.
    bool useListenThread = kDefaultUseListenThread;
    uint16_t listenPort = kDefaultListenPort;
    nixl_thread_sync_t syncMode = kDefaultSyncMode;
    bool captureTelemetry = kDefaultCaptureTelemetry;
    uint64_t pthrDelay = kDefaultPthrDelayUs; // progress thread sleep, microseconds
    uint64_t lthrDelay = kDefaultLthrDelayUs; // listener thread sleep, microseconds
    std::chrono::microseconds etcdWatchTimeout = kDefaultEtcdWatchTimeout;

    nixlAgentConfig() = default;

    explicit nixlAgentConfig(bool use_prog_thread,
                             bool use_listen_thread = kDefaultUseListenThread,
                             uint16_t port = kDefaultListenPort,
                             nixl_thread_sync_t sync_mode = kDefaultSyncMode,
                             unsigned int /*num_workers*/ = 1,
                             uint64_t pthr_delay_us = kDefaultPthrDelayUs,
                             uint64_t lthr_delay_us = kDefaultLthrDelayUs,
                             bool capture_telemetry = kDefaultCaptureTelemetry,
                             std::chrono::microseconds etcd_watch_timeout = kDefaultEtcdWatchTimeout) noexcept
        : useProgThread(use_prog_thread), useListenThread(use_listen_thread), listenPort(port),
          syncMode(sync_mode), captureTelemetry(capture_telemetry), pthrDelay(pthr_delay_us),
          lthrDelay(lthr_delay_us), etcdWatchTimeout(etcd_watch_timeout) {}
};

#endif
