// TEST INFRASTRUCTURE (oracle build only). Linux stand-in for the two Grand Central Dispatch
// names the Ingot CPU path uses (src/ops.h:16-19): dispatch_apply_f and DISPATCH_APPLY_AUTO.
// Real libdispatch is not available on Linux images without network access, so this header
// provides a blocking parallel-for with the same contract: work(ctx, i) is called exactly
// once for every i in [0, n), possibly concurrently, and the call returns when all are done.
// Iterations are handed out through an atomic counter, as GCD hands out iterations to its
// worker threads, so uneven items (24 heads on 8 cores) balance the same way. Workers are
// persistent (GCD's are too); the pool size is hardware_concurrency() or INGOT_REF_THREADS.
#pragma once

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <cstdlib>
#include <mutex>
#include <thread>
#include <vector>

#define DISPATCH_APPLY_AUTO nullptr

namespace ingot_dispatch_shim {

class Pool {
public:
    static Pool& get() {
        static Pool p;
        return p;
    }
    unsigned size() const { return n_threads_; }

    void apply(size_t n, void* ctx, void (*work)(void*, size_t)) {
        if (n == 0) return;
        if (n_threads_ <= 1 || n == 1 || busy_.exchange(true)) {
            // Single thread, single item, or a nested/concurrent call: run inline.
            for (size_t i = 0; i < n; i++) work(ctx, i);
            return;
        }
        {
            std::lock_guard<std::mutex> lk(mu_);
            n_ = n; ctx_ = ctx; work_ = work;
            next_.store(0, std::memory_order_relaxed);
            pending_ = unsigned(workers_.size());
            generation_++;
        }
        cv_start_.notify_all();
        drain();
        std::unique_lock<std::mutex> lk(mu_);
        cv_done_.wait(lk, [&] { return pending_ == 0; });
        busy_.store(false);
    }

private:
    Pool() {
        unsigned n = 0;
        if (const char* e = std::getenv("INGOT_REF_THREADS")) n = unsigned(std::max(0, std::atoi(e)));
        if (n == 0) n = std::thread::hardware_concurrency();
        n_threads_ = n ? n : 1;
        for (unsigned t = 1; t < n_threads_; t++) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
            generation_++;
        }
        cv_start_.notify_all();
        for (auto& w : workers_) w.join();
    }
    void drain() {
        for (;;) {
            size_t i = next_.fetch_add(1, std::memory_order_relaxed);
            if (i >= n_) return;
            work_(ctx_, i);
        }
    }
    void loop() {
        unsigned long seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_start_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (stop_) return;
            }
            drain();
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (--pending_ == 0) cv_done_.notify_one();
            }
        }
    }

    unsigned n_threads_ = 1;
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable cv_start_, cv_done_;
    unsigned long generation_ = 0;
    unsigned pending_ = 0;
    bool stop_ = false;
    std::atomic<bool> busy_{false};
    std::atomic<size_t> next_{0};
    size_t n_ = 0;
    void* ctx_ = nullptr;
    void (*work_)(void*, size_t) = nullptr;
};

}  // namespace ingot_dispatch_shim

inline void dispatch_apply_f(size_t n, void* /*queue*/, void* ctx, void (*work)(void*, size_t)) {
    ingot_dispatch_shim::Pool::get().apply(n, ctx, work);
}
