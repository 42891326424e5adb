// Pinned host memory in fixed-size units, carved from large arenas that a background thread allocates, places
// (NUMA policy) and pins, so that nobody on the serving path ever waits for a page-locking call of hundreds of
// milliseconds: callers `reserve` ahead of need, `get` a unit (blocking only if the reserve ran dry, with the wait
// accounted), and `put` it back; arenas that become empty beyond the standing reserve are released off-thread.
// Pinning is mlock plus, when the CUDA runtime is loaded in the process, cudaHostRegister (portable + mapped), looked
// up with dlsym so that this header builds and runs without CUDA.
// (Role of the reference's src/engine/pinned_pool.{hpp,cpp} and the NUMA placement of src/engine/spill.cpp:64-164.)
#pragma once
#include <dlfcn.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "common.hpp"

namespace qwh {

// ---- NUMA placement without libnuma
enum class NumaPolicy { Process = 0, Bind = 1, Preferred = 2, Interleave = 3 };

inline int numa_nodes() {
    int n = 0;
    for (; n < 64; ++n) {
        const std::string p = "/sys/devices/system/node/node" + std::to_string(n);
        if (access(p.c_str(), F_OK) != 0) break;
    }
    return n > 0 ? n : 1;
}
// Applies a policy to [p, p + bytes) before the pages are touched.  Returns false when the kernel refuses (the
// memory then follows the process policy; callers log it and go on).
inline bool numa_place(void *p, size_t bytes, NumaPolicy pol, int node) {
    if (pol == NumaPolicy::Process) return true;
    const int nodes = numa_nodes();
    unsigned long mask = 0;
    if (pol == NumaPolicy::Interleave) mask = nodes >= 64 ? ~0ul : ((1ul << nodes) - 1);
    else mask = 1ul << (node < 0 || node >= nodes ? 0 : node);
    const int mode = pol == NumaPolicy::Bind ? 2 /*MPOL_BIND*/ : pol == NumaPolicy::Preferred ? 1 /*MPOL_PREFERRED*/ : 3 /*MPOL_INTERLEAVE*/;
#ifdef SYS_mbind
    return syscall(SYS_mbind, p, bytes, mode, &mask, sizeof(mask) * 8 + 1, 0) == 0;
#else
    (void)p; (void)bytes; (void)mode;
    return false;
#endif
}
// The node a touched page lives on, or -1.
inline int numa_node_of(void *p) {
#ifdef SYS_move_pages
    void *pages[1] = {p};
    int status[1] = {-1};
    if (syscall(SYS_move_pages, 0, 1ul, pages, nullptr, status, 0) == 0) return status[0];
#endif
    return -1;
}

struct PoolStats {
    int64_t arenas, units_total, units_free, gets, waits;
    double wait_seconds, pin_seconds;
    int32_t cuda_registered, numa_node;
};

class PinnedPool {
public:
    PinnedPool(size_t unit_bytes, size_t arena_bytes, int standing_units, bool use_cuda, NumaPolicy pol = NumaPolicy::Process,
               int node = -1)
        : unit_((unit_bytes + 4095) & ~size_t(4095)), per_arena_(std::max<size_t>(1, arena_bytes / std::max<size_t>(unit_, 1))),
          standing_(standing_units), pol_(pol), node_(node) {
        if (use_cuda) {
            reg_ = reinterpret_cast<RegFn>(dlsym(RTLD_DEFAULT, "cudaHostRegister"));
            unreg_ = reinterpret_cast<UnregFn>(dlsym(RTLD_DEFAULT, "cudaHostUnregister"));
        }
        worker_ = std::thread([this] { run(); });
        reserve(standing_);
    }
    ~PinnedPool() {
        {
            std::lock_guard<std::mutex> l(m_);
            stop_ = true;
        }
        cv_work_.notify_all();
        worker_.join();
        for (auto &a : arenas_) release(a);
    }
    size_t unit_bytes() const { return unit_; }

    // Make sure `n` units are free or being prepared (returns at once).
    void reserve(int n) {
        std::lock_guard<std::mutex> l(m_);
        want_free_ = std::max(want_free_, n);
        cv_work_.notify_one();
    }
    // A pinned unit; blocks while none is free (the worker is asked again each time, so a lost wake-up cannot strand us).
    void *get() {
        std::unique_lock<std::mutex> l(m_);
        ++gets_;
        if (free_.empty()) {
            ++waits_;
            const auto t0 = std::chrono::steady_clock::now();
            while (free_.empty()) {
                want_free_ = std::max(want_free_, 1);
                cv_work_.notify_one();
                cv_free_.wait_for(l, std::chrono::milliseconds(50));
            }
            wait_s_ += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        }
        void *p = free_.back();
        free_.pop_back();
        arena_of(p)->used++;
        if (int(free_.size()) < standing_) {          // keep the standing reserve topped up
            want_free_ = std::max(want_free_, standing_);
            cv_work_.notify_one();
        }
        return p;
    }
    void put(void *p) {
        std::lock_guard<std::mutex> l(m_);
        Arena *a = arena_of(p);
        QWH_CHECK(a && a->used > 0, "pinned pool: put of a foreign or free unit");
        a->used--;
        free_.push_back(p);
        want_free_ = 0;
        cv_free_.notify_one();
        cv_work_.notify_one();                         // maybe an arena can be retired
    }
    PoolStats stats() {
        std::lock_guard<std::mutex> l(m_);
        return PoolStats{int64_t(arenas_.size()), int64_t(arenas_.size() * per_arena_), int64_t(free_.size()), gets_, waits_, wait_s_,
                         pin_s_, int32_t(reg_ != nullptr && registered_), last_node_};
    }

private:
    using RegFn = int (*)(void *, size_t, unsigned);
    using UnregFn = int (*)(void *);
    struct Arena { char *base = nullptr; size_t bytes = 0; int used = 0; bool registered = false; };

    Arena *arena_of(void *p) {
        for (auto &a : arenas_)
            if (p >= a.base && p < a.base + a.bytes) return &a;
        return nullptr;
    }
    Arena make() {            // outside the lock: allocation, placement, touching and pinning are the slow part
        Arena a;
        a.bytes = unit_ * per_arena_;
        a.base = static_cast<char *>(mmap(nullptr, a.bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0));
        QWH_CHECK(a.base != MAP_FAILED, "pinned pool: mmap failed");
        numa_place(a.base, a.bytes, pol_, node_);
        for (size_t o = 0; o < a.bytes; o += 4096) a.base[o] = 0;          // fault the pages in where the policy puts them
        mlock(a.base, a.bytes);                                           // best effort (RLIMIT_MEMLOCK may refuse)
        if (reg_ && reg_(a.base, a.bytes, 3u /* portable | mapped */) == 0) a.registered = true;
        return a;
    }
    void release(Arena &a) {
        if (a.registered && unreg_) unreg_(a.base);
        munlock(a.base, a.bytes);
        munmap(a.base, a.bytes);
    }
    void run() {
        std::unique_lock<std::mutex> l(m_);
        for (;;) {
            cv_work_.wait(l, [this] { return stop_ || int(free_.size()) < want_free_ || retire_candidate() >= 0; });
            if (stop_) return;
            if (int(free_.size()) < want_free_) {
                l.unlock();
                const auto t0 = std::chrono::steady_clock::now();
                Arena a = make();
                const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                const int node = numa_node_of(a.base);
                l.lock();
                pin_s_ += dt;
                last_node_ = node;
                registered_ = registered_ || a.registered;
                arenas_.push_back(a);
                for (size_t i = 0; i < per_arena_; ++i) free_.push_back(a.base + i * unit_);
                cv_free_.notify_all();
                continue;
            }
            const int r = retire_candidate();
            if (r >= 0) {
                Arena a = arenas_[size_t(r)];
                arenas_.erase(arenas_.begin() + r);
                free_.erase(std::remove_if(free_.begin(), free_.end(), [&](void *p) { return p >= a.base && p < a.base + a.bytes; }),
                            free_.end());
                l.unlock();
                release(a);
                l.lock();
            }
        }
    }
    // An arena with no unit in use whose removal still leaves the standing reserve free; -1 if none.
    int retire_candidate() const {
        if (int(free_.size()) - int(per_arena_) < std::max(standing_, want_free_)) return -1;
        for (size_t i = 0; i < arenas_.size(); ++i)
            if (arenas_[i].used == 0) return int(i);
        return -1;
    }

    const size_t unit_, per_arena_;
    const int standing_;
    const NumaPolicy pol_;
    const int node_;
    RegFn reg_ = nullptr;
    UnregFn unreg_ = nullptr;
    std::mutex m_;
    std::condition_variable cv_work_, cv_free_;
    std::vector<Arena> arenas_;
    std::vector<void *> free_;
    int want_free_ = 0;
    bool stop_ = false, registered_ = false;
    int64_t gets_ = 0, waits_ = 0;
    double wait_s_ = 0, pin_s_ = 0;
    int32_t last_node_ = -1;
    std::thread worker_;
};

}  // namespace qwh
