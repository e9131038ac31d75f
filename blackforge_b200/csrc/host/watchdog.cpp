#include "watchdog.hpp"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <vector>

namespace bfb200 {

WatchdogOutcome waitWithDeadline(const WatchdogHooks& hooks, std::int64_t timeoutMs) {
    using clock = std::chrono::steady_clock;
    const auto deadline = clock::now() + std::chrono::milliseconds(std::max<std::int64_t>(timeoutMs, 0));
    auto pause = std::chrono::microseconds(50);
    WatchdogOutcome outcome = WatchdogOutcome::TimedOut;
    while (true) {
        const int q = hooks.query ? hooks.query() : 0;
        if (q == 0) return WatchdogOutcome::Completed;
        if (q != 1) {
            outcome = WatchdogOutcome::QueryError;
            break;
        }
        if (hooks.asyncError && hooks.asyncError() != 0) {
            outcome = WatchdogOutcome::AsyncError;
            break;
        }
        if (clock::now() >= deadline) break;
        std::this_thread::sleep_for(pause);
        pause = std::min(pause * 2, std::chrono::microseconds(1000));
    }
    if (hooks.abort) hooks.abort();
    return outcome;
}

int watchdogSelfTest(int ranks, int skipRank, std::int64_t timeoutMs, bool* sumOk) {
    ranks = std::max(1, std::min(ranks, 16));
    struct Rendezvous {
        std::mutex mu;
        int contributed = 0;
        double sum = 0.0;
        std::atomic<bool> aborted{false};
    } rv;
    std::vector<int> timedOut(static_cast<std::size_t>(ranks), 0);
    std::vector<double> seen(static_cast<std::size_t>(ranks), 0.0);
    std::vector<std::thread> threads;
    for (int r = 0; r < ranks; ++r) {
        threads.emplace_back([&, r] {
            if (r == skipRank) return;   // this rank never joins the collective
            {
                std::lock_guard<std::mutex> lock(rv.mu);
                rv.sum += static_cast<double>(r + 1);
                ++rv.contributed;
            }
            WatchdogHooks hooks;
            hooks.query = [&] {
                std::lock_guard<std::mutex> lock(rv.mu);
                return rv.contributed == ranks ? 0 : 1;
            };
            hooks.asyncError = [&] { return rv.aborted.load() ? 1 : 0; };   // a peer's abort reaches the others
            hooks.abort = [&] { rv.aborted.store(true); };
            const WatchdogOutcome o = waitWithDeadline(hooks, timeoutMs);
            if (o == WatchdogOutcome::Completed) {
                std::lock_guard<std::mutex> lock(rv.mu);
                seen[static_cast<std::size_t>(r)] = rv.sum;
            } else {
                timedOut[static_cast<std::size_t>(r)] = 1;
            }
        });
    }
    for (std::thread& t : threads) t.join();
    bool ok = true;
    const double want = 0.5 * ranks * (ranks + 1);
    int count = 0;
    for (int r = 0; r < ranks; ++r) {
        if (r == skipRank) continue;
        if (timedOut[static_cast<std::size_t>(r)]) ++count;
        else ok = ok && seen[static_cast<std::size_t>(r)] == want;
    }
    if (sumOk != nullptr) *sumOk = ok;
    return count;
}

}  // namespace bfb200
