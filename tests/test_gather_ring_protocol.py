"""Host restatement of the copy ring of ``gather_role_w`` (csrc/kernels/gemm2_kernel.cuh), the
copy warp of the all-gather GEMM: one thread streams chunks peer HBM -> shared memory (bulk
load, mbarrier per stage) -> local HBM (bulk store, one commit group per chunk) through NSTAGE
stages.  The kernel uses the lagged form (a chunk is announced LAG groups after its store was
issued; a stage is reloaded as soon as the previous store has READ it); the one-store-at-a-time
form is replayed as well, as the simpler protocol the lagged one must be equivalent to.

Replayed with asynchronous loads and stores that finish after random delays, stores finishing
their read of shared memory before their write to global memory, and the semantics of
``cp.async.bulk.wait_group N`` (at most N groups not yet complete) and ``wait_group.read N``
(at most N groups still reading).  A stage must not be overwritten while a store still reads
it, and a chunk must not be announced before its bytes are in local memory.
"""
import random

import pytest


def simulate(n, nstage, lagged, seed):
    rng = random.Random(seed)
    now = [0]
    stage_version = [None] * nstage          # chunk whose bytes the stage holds (after the load landed)
    loads = {}                               # chunk -> landing time
    stores = []                              # per group: dict(chunk, read_done, done)
    announced = []

    def advance(t):
        now[0] = max(now[0], t)

    def issue_load(q):
        s = q % nstage
        # the stage's previous store must have finished reading by the time the load may land
        for g in stores:
            if g["stage"] == s:
                assert g["read_done"] <= now[0], f"chunk {q} loaded into stage {s} while chunk {g['chunk']} is still read"
        loads[q] = now[0] + rng.randint(1, 50)

    def wait_load(q):
        advance(loads[q])
        stage_version[q % nstage] = q

    def issue_store(q):
        s = q % nstage
        assert stage_version[s] == q
        read_done = now[0] + rng.randint(1, 20)
        stores.append({"chunk": q, "stage": s, "read_done": read_done, "done": read_done + rng.randint(1, 60)})

    def wait_group(k, read=False):
        # groups complete in order of issue as far as the waiting thread is concerned: wait until at most
        # k of the most recent groups are outstanding
        if len(stores) > k:
            upto = stores[:len(stores) - k]
            advance(max(g["read_done" if read else "done"] for g in upto))

    def announce(q):
        g = next(g for g in stores if g["chunk"] == q)
        assert g["done"] <= now[0], f"chunk {q} announced before its store completed"
        announced.append(q)

    for q in range(min(n, nstage - 1)):
        issue_load(q)
    if lagged:
        lag = nstage - 1
        for q in range(n):
            wait_load(q)
            issue_store(q)
            wait_group(lag)
            if q >= lag:
                announce(q - lag)
            nq = q + nstage - 1
            if nq < n:
                wait_group(1, read=True)
                issue_load(nq)
        wait_group(0)
        for q in range(max(0, n - lag), n):
            announce(q)
    else:
        prev = None
        for q in range(n):
            wait_load(q)
            issue_store(q)
            wait_group(1)
            if q >= 1:
                announce(prev)
            prev = q
            nq = q + nstage - 1
            if nq < n:
                issue_load(nq)
        wait_group(0)
        if prev is not None:
            announce(prev)
    assert announced == list(range(n))
    return True


@pytest.mark.parametrize("lagged", [True, False])
@pytest.mark.parametrize("nstage", [3, 4])
@pytest.mark.parametrize("n", [0, 1, 2, 3, 4, 5, 9, 40])
def test_ring_never_overwrites_a_stage_in_use_nor_announces_early(n, nstage, lagged):
    for seed in range(50):
        assert simulate(n, nstage, lagged, seed)
