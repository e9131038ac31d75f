"""Failure detection on the host, with no device involved: the watchdog that guards the tensor-parallel step (poll
the stream, look for an asynchronous error of the communicator, abort at the deadline) run against stand-ins, with
threads as ranks exchanging host values. One rank that never joins the collective must not block the others."""
import ctypes as C
import time


def run(bfb, ranks, skip, timeout_ms):
    timed_out, sum_ok = C.c_int32(-1), C.c_int32(-1)
    t0 = time.time()
    bfb.check(bfb.lib().bfb_selftest_collective_watchdog(ranks, skip, timeout_ms, C.byref(timed_out), C.byref(sum_ok)))
    return timed_out.value, sum_ok.value, time.time() - t0


def test_all_ranks_join_and_see_the_sum(bfb):
    for ranks in (1, 2, 8):
        timed_out, sum_ok, seconds = run(bfb, ranks, -1, 5000)
        assert timed_out == 0 and sum_ok == 1 and seconds < 4.0


def test_a_rank_that_skips_the_collective_times_the_others_out(bfb):
    # rank 1 of 4 never contributes: the other three give up after the deadline and abort; nothing blocks for ever
    timed_out, _sum_ok, seconds = run(bfb, 4, 1, 200)
    assert timed_out == 3
    assert 0.15 <= seconds < 3.0


def test_an_abort_by_one_rank_reaches_the_others_as_an_asynchronous_error(bfb):
    # with a zero deadline the first rank to poll aborts at once; the others learn of it through the communicator's
    # error state on their next poll instead of waiting out a deadline of their own
    timed_out, _sum_ok, seconds = run(bfb, 8, 0, 0)
    assert timed_out == 7 and seconds < 2.0


def test_bad_arguments_are_refused(bfb):
    lib = bfb.lib()
    assert lib.bfb_selftest_collective_watchdog(0, -1, 10, None, None) == bfb.INVALID_ARGUMENT
    assert lib.bfb_selftest_collective_watchdog(4, 4, 10, None, None) == bfb.INVALID_ARGUMENT
    assert lib.bfb_selftest_bounded_wait(10, None, None) in (bfb.INVALID_ARGUMENT, bfb.CUDA_ERROR)   # limit below 1 us
