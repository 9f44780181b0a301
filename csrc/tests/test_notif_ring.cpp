// The shared-memory notification ring of the NVLINK backend (src/plugins/nvlink/notif_ring.h), without a GPU:
// the host plays the part of the copy kernel's tail (one store to the slot's sequence word).
#include <sched.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "harness.h"
#include "plugins/nvlink/notif_ring.h"

using namespace nixl_nvlink;
using NotifList = std::vector<std::pair<std::string, std::string>>;

static std::string ringName(const char *tag) { return std::string("/nixl_b200.test.") + tag + "." + std::to_string(::getpid()); }

TEST_CASE(a_slot_is_delivered_only_once_its_sequence_word_is_stored) {
    NotifRingOwner owner;
    CHECK(owner.create(ringName("a")));
    auto w = NotifRingWriter::open(owner.name());
    CHECK(w != nullptr);
    CHECK(NotifRingWriter::open(owner.name()) == w); // one mapping per process
    uint64_t *word = nullptr, seq = 0;
    CHECK(w->claim("prefill", std::string("kv\0ready", 8), &word, &seq));
    CHECK(seq == 1);
    NotifList got;
    owner.poll(got);
    CHECK(got.empty()); // claimed, data not complete
    CHECK(owner.outstanding() == 1);
    NotifRingWriter::complete(word, seq, true);
    owner.poll(got);
    CHECK(got.size() == 1);
    CHECK(got[0].first == "prefill");
    CHECK(got[0].second == std::string("kv\0ready", 8)); // binary-safe
    CHECK(owner.outstanding() == 0);
    owner.poll(got);
    CHECK(got.size() == 1); // delivered once
}

TEST_CASE(later_slots_are_delivered_while_an_earlier_one_is_still_in_flight) {
    NotifRingOwner owner;
    CHECK(owner.create(ringName("b")));
    auto w = NotifRingWriter::open(owner.name());
    CHECK(w != nullptr);
    uint64_t *w0 = nullptr, *w1 = nullptr, *w2 = nullptr, s0 = 0, s1 = 0, s2 = 0;
    CHECK(w->claim("a", "long", &w0, &s0));
    CHECK(w->claim("a", "short1", &w1, &s1));
    CHECK(w->claim("a", "short2", &w2, &s2));
    NotifRingWriter::complete(w2, s2, true);
    NotifRingWriter::complete(w1, s1, true);
    NotifList got;
    owner.poll(got);
    CHECK(got.size() == 2);
    CHECK(got[0].second == "short1" && got[1].second == "short2");
    CHECK(owner.outstanding() == 3); // the tail waits for the first claim
    NotifRingWriter::complete(w0, s0, true);
    owner.poll(got);
    CHECK(got.size() == 3 && got[2].second == "long");
    CHECK(owner.outstanding() == 0);
}

TEST_CASE(a_voided_slot_is_consumed_without_a_notification) {
    NotifRingOwner owner;
    CHECK(owner.create(ringName("c")));
    auto w = NotifRingWriter::open(owner.name());
    uint64_t *word = nullptr, seq = 0;
    CHECK(w->claim("a", "never sent", &word, &seq));
    NotifRingWriter::complete(word, seq, false);
    NotifList got;
    owner.poll(got);
    CHECK(got.empty());
    CHECK(owner.outstanding() == 0);
}

TEST_CASE(a_full_ring_and_an_oversized_message_are_refused) {
    NotifRingOwner owner;
    CHECK(owner.create(ringName("d")));
    auto w = NotifRingWriter::open(owner.name());
    std::vector<std::pair<uint64_t *, uint64_t>> claims;
    uint64_t *word = nullptr, seq = 0;
    for (uint32_t i = 0; i < kNotifSlots; ++i) {
        CHECK(w->claim("a", std::to_string(i), &word, &seq));
        claims.emplace_back(word, seq);
    }
    CHECK(!w->claim("a", "one too many", &word, &seq));
    CHECK(!w->claim("a", std::string(kNotifPayloadMax, 'x'), &word, &seq)); // name + message exceed the slot
    for (auto &c : claims) NotifRingWriter::complete(c.first, c.second, true);
    NotifList got;
    owner.poll(got);
    CHECK(got.size() == kNotifSlots);
    CHECK(got.front().second == "0" && got.back().second == std::to_string(kNotifSlots - 1));
    // the ring wraps: slot 0 is reused under a new sequence number
    CHECK(w->claim("a", "wrapped", &word, &seq));
    CHECK(seq == kNotifSlots + 1);
    got.clear();
    owner.poll(got);
    CHECK(got.empty()); // the old sequence word of that slot does not count
    NotifRingWriter::complete(word, seq, true);
    owner.poll(got);
    CHECK(got.size() == 1 && got[0].second == "wrapped");
}

TEST_CASE(another_process_writes_and_a_claimant_that_died_does_not_hold_the_ring) {
    NotifRingOwner owner;
    CHECK(owner.create(ringName("e")));
    const std::string name = owner.name();
    const pid_t child = ::fork();
    if (child == 0) {
        auto w = NotifRingWriter::open(name);
        if (!w) ::_exit(2);
        uint64_t *word = nullptr, seq = 0;
        if (!w->claim("child", "left hanging", &word, &seq)) ::_exit(3); // its "kernel" never finishes
        if (!w->claim("child", "delivered", &word, &seq)) ::_exit(4);
        NotifRingWriter::complete(word, seq, true);
        ::_exit(0);
    }
    int status = 0;
    CHECK(::waitpid(child, &status, 0) == child);
    CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    NotifList got;
    owner.poll(got);
    CHECK(got.size() == 1 && got[0].first == "child" && got[0].second == "delivered");
    CHECK(owner.outstanding() == 2); // the dead claimant's first slot holds the tail for now
    for (int i = 0; i < 30 && owner.outstanding() != 0; ++i) { // skipped once the claim is older than a second
        std::this_thread::sleep_for(std::chrono::milliseconds(110));
        owner.poll(got);
    }
    CHECK(owner.outstanding() == 0);
    CHECK(got.size() == 1);
}

TEST_CASE(several_writers_and_one_reader_deliver_every_message_exactly_once) {
    // Every writer is a process of its own: what orders two writers that use the same slot one lap apart is the
    // reader in between, and a race detector sees neither another process nor a second mapping of the ring in this one.
    NotifRingOwner owner;
    CHECK(owner.create(ringName("g")));
    const std::string name = owner.name();
    constexpr int kWriters = 4, kEach = 3000; // 12000 messages through 1024 slots: the ring wraps many times
    std::vector<pid_t> children;
    for (int t = 0; t < kWriters; ++t) {
        const pid_t child = ::fork();
        if (child == 0) {
            auto w = NotifRingWriter::open(name);
            if (!w) ::_exit(2);
            for (int i = 0; i < kEach; ++i) {
                uint64_t *word = nullptr, seq = 0;
                const std::string msg = std::to_string(t) + ":" + std::to_string(i);
                while (!w->claim("writer" + std::to_string(t), msg, &word, &seq)) ::sched_yield(); // full: the reader is behind
                if (i % 7 == 3) ::sched_yield(); // some claims complete late, out of order with the other writers'
                NotifRingWriter::complete(word, seq, i % 11 != 5); // and some are voided
            }
            ::_exit(0);
        }
        children.push_back(child);
    }
    std::vector<std::vector<int>> seen(kWriters);
    size_t total = 0, expected = 0;
    for (int i = 0; i < kEach; ++i) expected += i % 11 != 5;
    expected *= kWriters;
    const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(60);
    while (total < expected && std::chrono::steady_clock::now() < end) {
        NotifList got;
        owner.poll(got);
        for (auto &n : got) {
            const int t = n.first.back() - '0';
            CHECK(t >= 0 && t < kWriters && n.first == "writer" + std::to_string(t));
            const size_t colon = n.second.find(':');
            CHECK(colon != std::string::npos && std::stoi(n.second.substr(0, colon)) == t);
            seen[t].push_back(std::stoi(n.second.substr(colon + 1)));
            ++total;
        }
    }
    for (pid_t child : children) {
        int status = 0;
        CHECK(::waitpid(child, &status, 0) == child);
        CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    }
    NotifList rest;
    owner.poll(rest);
    CHECK(rest.empty());
    CHECK_EQ(total, expected);
    CHECK_EQ(owner.outstanding(), uint64_t(0));
    for (int t = 0; t < kWriters; ++t) {
        std::sort(seen[t].begin(), seen[t].end());
        CHECK(std::adjacent_find(seen[t].begin(), seen[t].end()) == seen[t].end()); // no duplicates
        size_t at = 0;
        for (int i = 0; i < kEach; ++i)
            if (i % 11 != 5) CHECK(seen[t][at++] == i);
    }
}

TEST_CASE(rings_left_by_dead_processes_are_removed_by_the_next_owner) {
    const pid_t child = ::fork();
    if (child == 0) { // dies without running the owner's destructor
        auto *leaked = new NotifRingOwner();
        ::_exit(leaked->create("/nixl_b200_reap." + std::to_string(::getpid()) + ".leak") ? 0 : 2);
    }
    int status = 0;
    CHECK(::waitpid(child, &status, 0) == child);
    CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    const std::string stale = "/nixl_b200_reap." + std::to_string(child) + ".leak";
    CHECK(NotifRingWriter::open(stale) != nullptr); // still there ...
    NotifRingOwner next;
    CHECK(next.create("/nixl_b200_reap." + std::to_string(::getpid()) + ".next"));
    CHECK(::access(("/dev/shm" + stale).c_str(), F_OK) != 0); // ... until the next owner of the family comes
}

TEST_CASE(a_ring_that_is_gone_cannot_be_opened) {
    std::string name;
    {
        NotifRingOwner owner;
        CHECK(owner.create(ringName("f")));
        name = owner.name();
    }
    CHECK(NotifRingWriter::open(name) == nullptr);
    CHECK(NotifRingWriter::open("/nixl_b200.test.never.created") == nullptr);
}

TEST_MAIN()
