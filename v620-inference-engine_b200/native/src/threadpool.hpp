// Worker pool for data-parallel loops on the host (the PLE gather, the fp32 oracle's matrix products).
//
// parallel_for(n, grain, fn) splits [0, n) into pieces of at least `grain` items and returns when fn has run on all of
// them; the calling thread works too.  Pieces are claimed with one atomic increment, so the mutex is only taken to
// publish a loop and to sleep.  A loop lives in a shared_ptr that every woken worker copies: a worker that wakes late,
// after the caller has already returned, finds nothing left to claim and lets go of it - no counting of who is still
// inside.  (Role of the reference's src/core/threadpool.hpp:14-113.)
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "common.hpp"

namespace qwh {

class ThreadPool {
public:
    using Body = std::function<void(int64_t, int64_t)>;

    explicit ThreadPool(int threads) {
        for (int i = 1; i < threads; ++i) helpers_.emplace_back(&ThreadPool::helper_main, this);
    }
    ThreadPool(const ThreadPool &) = delete;
    ThreadPool &operator=(const ThreadPool &) = delete;
    ~ThreadPool() {
        {
            std::lock_guard<std::mutex> g(m_);
            quitting_ = true;
        }
        wake_.notify_all();
        for (std::thread &t : helpers_) t.join();
    }

    int size() const { return 1 + int(helpers_.size()); }

    void parallel_for(int64_t n, int64_t grain, const Body &fn) {
        if (n <= 0) return;
        const int64_t min_piece = grain > 0 ? grain : 1;
        int64_t pieces = (n + min_piece - 1) / min_piece;
        const int64_t most = int64_t(size()) * 4;               // a few pieces per thread evens out uneven ones
        if (pieces > most) pieces = most;
        if (pieces < 2 || helpers_.empty()) {
            fn(0, n);
            return;
        }
        auto loop = std::make_shared<Loop>();
        loop->body = &fn;
        loop->total = n;
        loop->piece = (n + pieces - 1) / pieces;
        loop->count = (n + loop->piece - 1) / loop->piece;
        loop->unfinished.store(loop->count, std::memory_order_relaxed);
        {
            std::lock_guard<std::mutex> g(m_);
            current_ = loop;
            ++generation_;
        }
        wake_.notify_all();
        work_on(*loop);
        std::unique_lock<std::mutex> g(m_);
        finished_.wait(g, [&] { return loop->unfinished.load(std::memory_order_acquire) == 0; });
        if (current_ == loop) current_.reset();
    }

private:
    struct Loop {
        const Body *body = nullptr;
        int64_t total = 0, piece = 0, count = 0;
        std::atomic<int64_t> claimed{0};
        std::atomic<int64_t> unfinished{0};
    };

    void work_on(Loop &loop) {
        for (;;) {
            const int64_t i = loop.claimed.fetch_add(1, std::memory_order_relaxed);
            if (i >= loop.count) return;
            const int64_t lo = i * loop.piece;
            const int64_t hi = lo + loop.piece < loop.total ? lo + loop.piece : loop.total;
            (*loop.body)(lo, hi);
            if (loop.unfinished.fetch_sub(1, std::memory_order_acq_rel) == 1) {
                std::lock_guard<std::mutex> g(m_);              // the waiter checks under this lock: no lost wake-up
                finished_.notify_all();
            }
        }
    }

    void helper_main() {
        uint64_t seen = 0;
        for (;;) {
            std::shared_ptr<Loop> loop;
            {
                std::unique_lock<std::mutex> g(m_);
                wake_.wait(g, [&] { return quitting_ || generation_ != seen; });
                if (quitting_) return;
                seen = generation_;
                loop = current_;
            }
            if (loop) work_on(*loop);
        }
    }

    std::vector<std::thread> helpers_;
    std::mutex m_;
    std::condition_variable wake_, finished_;
    std::shared_ptr<Loop> current_;
    uint64_t generation_ = 0;
    bool quitting_ = false;
};

}  // namespace qwh
