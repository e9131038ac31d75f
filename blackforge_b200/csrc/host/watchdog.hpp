// A deadline around work that completes asynchronously on a stream and may never complete: a collective whose
// peer died, left or skipped the call. The waiting side polls instead of blocking in a synchronize, looks for an
// asynchronous error of the communicator, and when the deadline passes aborts the communicator so that nothing is
// left spinning on the device. Written over three callables so that the same code runs against CUDA + NCCL in
// production and against host-only stand-ins in the tests (no GPU is made to hang to test it).
#pragma once

#include <cstdint>
#include <functional>

namespace bfb200 {

enum class WatchdogOutcome { Completed = 0, TimedOut = 1, AsyncError = 2, QueryError = 3 };

struct WatchdogHooks {
    std::function<int()> query;        // 0: the work has completed, 1: not yet, anything else: the query itself failed
    std::function<int()> asyncError;   // 0: the communicator is healthy, anything else: it reported an error
    std::function<void()> abort;       // called once on TimedOut / AsyncError / QueryError; must not block for long
};

// Polls until completion, an error or `timeoutMs` (sleeping between polls, from 50 us up to 1 ms).
WatchdogOutcome waitWithDeadline(const WatchdogHooks& hooks, std::int64_t timeoutMs);

// Host-only exercise of the above with threads as ranks: `ranks` threads sum a host buffer through a shared
// rendezvous (the stand-in for an all-reduce: it completes when every rank has contributed); rank `skipRank` never
// contributes (-1: everyone does). Every other rank waits with `timeoutMs`. Returns how many ranks timed out and
// aborted; `sumOk` tells whether the ranks that completed saw the right sum.
int watchdogSelfTest(int ranks, int skipRank, std::int64_t timeoutMs, bool* sumOk);

}  // namespace bfb200
