"""Timing model of the cross-GPU protocol of the fused reduce kernel
(csrc/comm/rs_adam.cu): per call a start barrier (every rank publishes "my kernel
has started" and waits, bounded, for the same word of all peers), the work, and an
end barrier (the rank publishes "I read your buffers no more" and waits, bounded,
for the peers' words).  Ranks issue the calls from one stream while their compute
runs ahead by at most two calls (two gradient buffers).

What the model is for: one rank that is late by more than the wait budget must cost
a bounded number of time-outs, after which all ranks run in step again.  With the
earlier behaviour of the kernel (a CTA that timed out at the start left at once,
without sending the rank's done word) the peers lose one budget per call at the end
barrier, arrive late to the next call and make the first rank time out again: the
time-outs never stop.  Both behaviours are modelled; the test pins the difference.
"""
import heapq

BUDGET = 10.0       # bounded wait, in the time unit of the model
COMPUTE = 1.0       # compute between two calls of a rank
WORK = 0.2          # duration of the reduction itself


def run(world, calls, late_rank=None, late_call=None, late_by=0.0, leave_on_start_timeout=False):
    """Returns (finish time of the last call, list of (rank, call, kind) time-outs)."""
    start_word = [[None] * calls for _ in range(world)]      # time rank r published its start of call k
    done_word = [[None] * calls for _ in range(world)]
    finish = [[None] * calls for _ in range(world)]
    timeouts = []
    events = []                                              # (time, order, fn)
    order = [0]

    def at(t, fn):
        order[0] += 1
        heapq.heappush(events, (t, order[0], fn))

    def launch(r, k, compute_done):
        # the call is issued when the compute before it is done and the previous call of the
        # stream has finished; compute runs at most two calls ahead of the reductions
        def try_start(t):
            start_word[r][k] = t
            wait_start(r, k, t, t)
        prev = finish[r][k - 1] if k > 0 else 0.0
        at(max(compute_done, prev), lambda t: try_start(t))

    def peers_have(words, r, k):
        return all(words[p][k] is not None for p in range(world) if p != r)

    def wait_start(r, k, began, now):
        if peers_have(start_word, r, k):
            at(now + WORK, lambda t: end_barrier(r, k, t, ran=True))
        elif now - began >= BUDGET:
            timeouts.append((r, k, "start"))
            if leave_on_start_timeout:
                finished(r, k, now)                          # old kernel: gone, no done word
            else:
                end_barrier(r, k, now, ran=False)
        else:
            at(now + 0.05, lambda t: wait_start(r, k, began, t))

    def end_barrier(r, k, now, ran):
        done_word[r][k] = now
        if not ran:
            finished(r, k, now)                              # read nothing: nothing to wait for
        else:
            wait_done(r, k, now, now)

    def wait_done(r, k, began, now):
        if peers_have(done_word, r, k):
            finished(r, k, now)
        elif now - began >= BUDGET:
            timeouts.append((r, k, "end"))
            finished(r, k, now)
        else:
            at(now + 0.05, lambda t: wait_done(r, k, began, t))

    compute_at = [[None] * calls for _ in range(world)]

    def finished(r, k, now):
        finish[r][k] = now
        if k + 1 < calls:
            schedule(r, k + 1)

    def schedule(r, k):
        # compute of call k starts after the compute of k-1 and after call k-2 released its buffer
        base = compute_at[r][k - 1] if k > 0 else 0.0
        if k >= 2:
            base = max(base, finish[r][k - 2])
        extra = late_by if (r == late_rank and k == late_call) else 0.0
        compute_at[r][k] = base + COMPUTE + extra
        launch(r, k, compute_at[r][k])

    for r in range(world):
        schedule(r, 0)
    while events:
        t, _, fn = heapq.heappop(events)
        fn(t)
    return max(finish[r][calls - 1] for r in range(world)), timeouts


def test_ranks_in_step_never_time_out():
    end, timeouts = run(world=8, calls=40)
    assert timeouts == []
    assert end < 40 * (COMPUTE + WORK) + 1.0


def test_a_short_delay_is_absorbed_by_the_waits():
    end, timeouts = run(world=8, calls=40, late_rank=3, late_call=5, late_by=0.8 * BUDGET)
    assert timeouts == []


def test_one_long_delay_costs_a_bounded_number_of_timeouts():
    delay = 2.5 * BUDGET
    end, timeouts = run(world=8, calls=60, late_rank=0, late_call=4, late_by=delay)
    assert timeouts, "a delay beyond the budget has to show"
    last_bad = max(k for _, k, _ in timeouts)
    assert last_bad <= 4 + 6, f"time-outs go on until call {last_bad}"
    # afterwards the run proceeds at full speed again
    assert end < 60 * (COMPUTE + WORK) + delay + 4 * BUDGET


def test_leaving_at_the_start_timeout_never_recovers():
    """The behaviour the kernel had before: kept here so that the property above is known
    to distinguish the two."""
    delay = 2.5 * BUDGET
    end, timeouts = run(world=8, calls=60, late_rank=0, late_call=4, late_by=delay,
                        leave_on_start_timeout=True)
    last_bad = max(k for _, k, _ in timeouts)
    assert last_bad >= 50
    assert end > 40 * BUDGET
