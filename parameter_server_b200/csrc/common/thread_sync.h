// Cross-thread request coalescing primitives.
//
// Parity: ThreadReduce / ThreadBcast of pico-ps/common/ThreadSync.h:19-92. Up to GROUP_SIZE (32)
// threads register in a group; each announces that its request data is ready with reduce(); the thread
// that observes "enough are ready, or nobody is still preparing" claims every ready slot and sends ONE
// merged request for them, the others get an empty claim and sleep on their eventfd until the owner
// broadcasts the shared status. The flag word packs running (high 32 bits) and finished (low 32 bits)
// bitmaps so that claim decisions are one compare-and-swap.
#pragma once
#include <sys/eventfd.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <stdexcept>

namespace psb {

constexpr int kThreadGroupSize = 32;

class ThreadReduce {
public:
    // Thread `tid` (0..31) starts preparing a request.
    void add(int tid) { flags_.fetch_or(1ull << (32 + tid), std::memory_order_acq_rel); }

    // Thread `tid` finished preparing. Returns the bitmap of slots THIS thread must send (possibly
    // including others'), or 0 when another thread will send this one.
    uint32_t reduce(int tid, int sync_num) {
        const uint64_t run_bit = 1ull << (32 + tid), fin_bit = 1ull << tid;
        uint64_t cur = flags_.load(std::memory_order_acquire);
        for (;;) {
            uint64_t next = (cur & ~run_bit) | fin_bit;
            const uint32_t running = (uint32_t)(next >> 32), finished = (uint32_t)next;
            const bool claim = __builtin_popcount(finished) >= sync_num || running == 0;
            if (claim) next &= ~(uint64_t)finished;  // take every finished slot
            if (flags_.compare_exchange_weak(cur, next, std::memory_order_acq_rel)) return claim ? finished : 0u;
        }
    }

private:
    std::atomic<uint64_t> flags_{0};
};

class ThreadBcast {
public:
    ThreadBcast() {
        for (auto& fd : fds_) {
            fd = ::eventfd(0, EFD_SEMAPHORE);
            if (fd < 0) throw std::runtime_error("eventfd failed");
        }
    }
    ~ThreadBcast() {
        for (int fd : fds_) ::close(fd);
    }
    // Owner: wake every thread in `tids` except itself.
    void notify(uint32_t tids, int self) {
        for (int t = 0; t < kThreadGroupSize; ++t)
            if (((tids >> t) & 1u) && t != self) {
                uint64_t one = 1;
                ssize_t r = ::write(fds_[t], &one, 8);
                (void)r;
            }
    }
    // Merged thread: sleep until the owner notified.
    void wait(int tid) {
        uint64_t v;
        ssize_t r = ::read(fds_[tid], &v, 8);
        (void)r;
    }

private:
    int fds_[kThreadGroupSize];
};

}  // namespace psb
