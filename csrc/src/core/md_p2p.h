// Peer-to-peer metadata exchange over TCP.
//
// Wire protocol (parity with the reference's src/core/nixl_p2p_metadata_backend.cpp
// :46-50,:262-308,:393-412): each message is a frame `u64 size | body`; a body is one
// command: "NIXLCOMM:LOAD" + metadata blob (load this), "NIXLCOMM:SEND" (reply on this
// connection with a LOAD of your metadata), "NIXLCOMM:INVL" + agent name (forget that
// agent).  Frames above 1 GiB are rejected; a body must arrive within 5 s of its size.
#ifndef NIXL_B200_MD_P2P_H
#define NIXL_B200_MD_P2P_H

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "core/md_manager.h"

namespace nixl_p2p {
constexpr size_t kMaxFrame = 1ull << 30;
constexpr int kBodyTimeoutMs = 5000;

// Blocking helpers on a connected socket; false on error/timeout.
bool sendFrame(int fd, const std::string &body);
bool recvFrame(int fd, std::string &body, int timeout_ms);
// Connect with a timeout; -1 on failure.
int dial(const std::string &ip, int port, int timeout_ms);
} // namespace nixl_p2p

// Accepts connections and serves LOAD / SEND / INVL on a background thread.
class nixlP2PListener {
public:
    nixlP2PListener(nixlMetadataContext &ctx, uint16_t port, uint64_t poll_delay_us);
    ~nixlP2PListener();
    bool ok() const { return listenFd_ >= 0; }
    uint16_t port() const { return port_; }
    void start();
    void stop();

private:
    // One accepted connection and the frame that is arriving on it.  Frames are put together as their bytes come in, so
    // a connection that announces much and sends little keeps nobody else waiting and holds no more memory than it sent.
    struct Client {
        int fd = -1;
        std::string buf;       // the length word, then the body, as far as received
        uint64_t frameLen = 0; // valid once buf holds the length word
        int64_t startedMs = 0; // when the first byte of the current frame came (0: between frames)
    };
    void loop();
    bool advance(Client &c);                           // reads what is there; false: drop the connection
    bool handle(Client &c, const std::string &frame);  // one complete frame; false: drop the connection

    nixlMetadataContext &ctx_;
    int listenFd_ = -1;
    uint16_t port_ = 0;
    uint64_t delayUs_;
    std::atomic<bool> stop_{false};
    std::thread th_;
    std::vector<Client> clients_;
};

#endif
