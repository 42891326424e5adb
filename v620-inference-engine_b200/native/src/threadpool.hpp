// Persistent worker pool with a blocking, chunked parallel_for.
#pragma once
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "common.hpp"

namespace qwh {

class ThreadPool {
public:
    explicit ThreadPool(int n) {
        if (n < 1) n = 1;
        for (int i = 0; i < n - 1; ++i) workers_.emplace_back([this] { loop(); });
    }
    ~ThreadPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto &t : workers_) t.join();
    }
    int size() const { return int(workers_.size()) + 1; }

    // fn(begin, end) over [0, n) in chunks of at least `grain`; returns when all chunks ran.
    void parallel_for(int64_t n, int64_t grain, const std::function<void(int64_t, int64_t)> &fn) {
        if (n <= 0) return;
        if (grain < 1) grain = 1;
        const int64_t chunks = std::min<int64_t>((n + grain - 1) / grain, size() * 4);
        if (chunks <= 1 || workers_.empty()) { fn(0, n); return; }
        Job job{&fn, n, (n + chunks - 1) / chunks, 0, 0, chunks, 0};
        {
            std::lock_guard<std::mutex> lk(mu_);
            job_ = &job;
            ++epoch_;
        }
        cv_.notify_all();
        run(job);
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [&] { return job.finished == job.chunks && job.active == 0; });
        job_ = nullptr;
    }

private:
    struct Job {
        const std::function<void(int64_t, int64_t)> *fn;
        int64_t n, step, next, finished, chunks;
        int active = 0;      // workers currently inside run(): the job must outlive them
    };
    void run(Job &job) {
        for (;;) {
            int64_t c;
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (job.next >= job.chunks) return;
                c = job.next++;
            }
            const int64_t b = c * job.step, e = std::min(job.n, b + job.step);
            if (b < e) (*job.fn)(b, e);
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (++job.finished == job.chunks) done_.notify_all();
            }
        }
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            Job *job;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || (job_ && epoch_ != seen); });
                if (stop_) return;
                seen = epoch_;
                job = job_;
                if (job) ++job->active;
            }
            if (job) {
                run(*job);
                std::lock_guard<std::mutex> lk(mu_);
                --job->active;
                done_.notify_all();
            }
        }
    }
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_, done_;
    Job *job_ = nullptr;
    uint64_t epoch_ = 0;
    bool stop_ = false;
};

}  // namespace qwh
