// The descriptor hand-off of the NVLINK backend's VMM sharing (src/plugins/nvlink/vmm_share.h), without a GPU:
// file descriptors of ordinary files stand in for exported memory handles.
#include <fcntl.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>

#include "harness.h"
#include "plugins/nvlink/vmm_share.h"

using namespace nixl_nvlink;

static std::string uniqueName(const char *tag) { return std::string("nixl_b200.test.") + tag + "." + std::to_string(::getpid()); }

TEST_CASE(descriptors_cross_to_another_process_and_name_the_same_file) {
    char path[] = "/tmp/nixl_vmm_share_XXXXXX";
    const int fd = ::mkstemp(path);
    CHECK(fd >= 0);
    ::unlink(path);
    const int other = ::open("/dev/null", O_RDONLY);
    VmmFdServer server;
    const std::string name = uniqueName("fd");
    CHECK(server.start(name));
    CHECK(server.start(name)); // idempotent
    server.allow(fd);
    server.allow(other);
    const pid_t child = ::fork();
    if (child == 0) { // importer: fetch both descriptors, write through the first
        const std::vector<int> got = vmmFetchFds(name, {fd, other}, 3000);
        if (got.size() != 2) ::_exit(2);
        if (::pwrite(got[0], "through the socket", 18, 0) != 18) ::_exit(3);
        ::_exit(0);
    }
    int status = 0;
    CHECK(::waitpid(child, &status, 0) == child);
    CHECK(WIFEXITED(status) && WEXITSTATUS(status) == 0);
    char buf[32] = {0};
    CHECK(::pread(fd, buf, 18, 0) == 18);
    CHECK(std::strcmp(buf, "through the socket") == 0);
    ::close(fd);
    ::close(other);
}

TEST_CASE(a_number_that_was_not_exported_is_refused) {
    VmmFdServer server;
    const std::string name = uniqueName("refuse");
    CHECK(server.start(name));
    const int fd = ::open("/dev/null", O_RDONLY);
    server.allow(fd);
    CHECK(vmmFetchFds(name, {fd}, 2000).size() == 1);
    CHECK(vmmFetchFds(name, {fd, 0}, 2000).empty()); // stdin was never exported
    server.revoke(fd);
    CHECK(vmmFetchFds(name, {fd}, 2000).empty());
    CHECK(vmmFetchFds(uniqueName("nobody"), {fd}, 200).empty()); // no such server
    ::close(fd);
}

TEST_CASE(many_descriptors_travel_in_several_messages) {
    VmmFdServer server;
    const std::string name = uniqueName("many");
    CHECK(server.start(name));
    std::vector<int> mine;
    for (int i = 0; i < 300; ++i) {
        mine.push_back(::open("/dev/null", O_RDONLY));
        CHECK(mine.back() >= 0);
        server.allow(mine.back());
    }
    std::vector<int> got = vmmFetchFds(name, mine, 3000);
    CHECK(got.size() == mine.size());
    for (int f : got) ::close(f);
    for (int f : mine) ::close(f);
}

TEST_CASE(host_memory_is_not_vmm_memory) {
    // Without a GPU (or for an address CUDA does not know) the export simply says no.
    std::vector<VmmChunk> chunks;
    static char buf[4096];
    CHECK(!vmmExportRange(reinterpret_cast<uintptr_t>(buf), sizeof(buf), chunks));
    CHECK(chunks.empty());
}

TEST_MAIN()
