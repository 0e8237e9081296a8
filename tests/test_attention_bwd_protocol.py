"""Host restatement of the attention backward's synchronisation (csrc/kernels/attention_bwd.cuh).

One CTA walks `iters` (head, query block) steps with K and V resident.  Per step:

  loader     waits do_empty -> loads dO -> do_full;  waits q_empty -> loads Q -> q_full
  issuer     waits q_full, s_free, do_full -> S (into the S columns), commit s_full -> dP, commit
             dp_full -> waits p_full -> dV, commit do_empty -> waits ds_full -> dK, commit q_empty
             -> dQ (into the S columns again), commit dq_full
  softmax    waits s_full -> reads S, writes the P tile, arrives p_full -> waits dp_full and
             shared_free of the previous step -> writes the dS tile, arrives ds_full -> waits
             dq_full -> reads dQ, arrives s_free -> waits own_free of the previous step -> writes
             the dQ slabs (two in memory of their own, two inside the dS tile), arrives dqs_full
  reducer    waits dqs_full -> reduce-adds the slabs inside the dS tile, arrives shared_free ->
             reduce-adds the own slabs, arrives own_free

Replayed with phase-parity barriers, an in-order tensor pipe whose commits arrive when everything
issued before them has run, and random delays for loads, products, the reduce-adds and the
softmax warps (two groups that finish at different times).  Checked: every product finds the
operands of its own step, no tile or tensor-memory column is overwritten while something still
reads it, and the walk ends for any number of steps.  Dropping one of the waits must be noticed.
"""
import random

import pytest


class Barrier:
    def __init__(self, count=1):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self, n=1):
        self.arrived += n
        if self.arrived >= self.count:
            self.arrived, self.completed = 0, self.completed + 1

    def passed(self, parity):
        return (self.completed & 1) != parity


GROUPS = 2      # softmax warps modelled as two groups with independent timing


def simulate(iters, seed, drop=None):
    rng = random.Random(seed)
    names = ["q_full", "do_full", "q_empty", "do_empty", "s_full", "dp_full", "dq_full", "shared_free",
             "own_free"]
    bars = {n: Barrier() for n in names}
    for n in ("p_full", "ds_full", "s_free", "dqs_full"):
        bars[n] = Barrier(GROUPS)
    # what each resource holds: (kind, step); readers still outstanding are counted per resource
    holds = {"sQ": None, "sdO": None, "sP": None, "sdS": None, "tmS": None, "tmdP": None, "own": None}
    pending_reads = {k: 0 for k in holds}
    pipe, inflight, tick = [], [], [0]

    def write(res, what):
        assert pending_reads[res] == 0, f"{res} overwritten with {what} while {holds[res]} is still being read"
        holds[res] = what

    def loader():
        for it in range(iters):
            yield ("wait", "do_empty", (it & 1) ^ 1)

            def landed_do(it=it):
                write("sdO", ("dO", it))
                bars["do_full"].arrive()
            inflight.append((tick[0] + rng.randint(1, 40), landed_do))
            yield ("wait", "q_empty", (it & 1) ^ 1)

            def landed_q(it=it):
                write("sQ", ("Q", it))
                bars["q_full"].arrive()
            inflight.append((tick[0] + rng.randint(1, 40), landed_q))

    def issue(kind, it, reads, writes, commits):
        for r in reads:
            pending_reads[r] += 1                     # operand bound at issue, released when it ran
        pipe.append(("mma", kind, it, reads, writes))
        for c in commits:
            pipe.append(("commit", c))

    def issuer():
        for it in range(iters):
            ph = it & 1
            yield ("wait", "q_full", ph)
            if drop != "s_free":
                yield ("wait", "s_free", ph ^ 1)
            yield ("wait", "do_full", ph)
            issue("S", it, ["sQ"], ["tmS"], ["s_full"])
            issue("dP", it, ["sdO"], ["tmdP"], ["dp_full"])
            yield ("wait", "p_full", ph)
            issue("dV", it, ["sP", "sdO"], [], ["do_empty"])
            yield ("wait", "ds_full", ph)
            issue("dK", it, ["sdS", "sQ"], [], ["q_empty"])
            issue("dQ", it, ["sdS"], ["tmS"], ["dq_full"])

    expect = {"S": {"sQ": "Q"}, "dP": {"sdO": "dO"}, "dV": {"sP": "P", "sdO": "dO"},
              "dK": {"sdS": "dS", "sQ": "Q"}, "dQ": {"sdS": "dS"}}

    # The two softmax groups share the tiles; the model lets the first group to reach a write do
    # the hazard check and the write of the whole tile.
    written = {}

    def tile_write(res, what):
        if written.get(res) != what:
            write(res, what)
            written[res] = what

    def softmax(g):
        for it in range(iters):
            ph = it & 1
            yield ("wait", "s_full", ph)
            assert holds["tmS"] == ("S", it), f"softmax of step {it} found {holds['tmS']} in the S columns"
            yield ("work",)
            tile_write("sP", ("P", it))
            bars["p_full"].arrive()
            yield ("wait", "dp_full", ph)
            if it > 0 and drop != "shared_free":
                yield ("wait", "shared_free", (it - 1) & 1)
            assert holds["tmdP"] == ("dP", it)
            yield ("work",)
            tile_write("sdS", ("dS", it))
            bars["ds_full"].arrive()
            yield ("wait", "dq_full", ph)
            assert holds["tmS"] == ("dQ", it), f"dQ of step {it} expected in the S columns, found {holds['tmS']}"
            yield ("work",)
            bars["s_free"].arrive()
            if it > 0 and drop != "own_free":
                yield ("wait", "own_free", (it - 1) & 1)
            tile_write("own", ("dQ-own", it))
            tile_write("sdS", ("dQ-shared", it))      # the slabs that live inside the dS tile
            bars["dqs_full"].arrive()

    def reducer():
        for it in range(iters):
            yield ("wait", "dqs_full", it & 1)
            assert holds["sdS"] == ("dQ-shared", it) and holds["own"] == ("dQ-own", it)
            pending_reads["sdS"] += 1
            pending_reads["own"] += 1

            def read_shared():
                pending_reads["sdS"] -= 1
                bars["shared_free"].arrive()
            t_shared = tick[0] + rng.randint(1, 60)
            inflight.append((t_shared, read_shared))

            def read_own():
                pending_reads["own"] -= 1
                bars["own_free"].arrive()
            inflight.append((t_shared + rng.randint(1, 60), read_own))

    roles = {"loader": loader(), "issuer": issuer(), "reducer": reducer()}
    for g in range(GROUPS):
        roles[f"softmax{g}"] = softmax(g)
    blocked, busy_until = {}, 0
    for _ in range(400000):
        tick[0] += 1
        for x in sorted([x for x in inflight if x[0] <= tick[0]], key=lambda x: x[0]):
            inflight.remove(x)
            x[1]()
        if pipe and tick[0] >= busy_until:
            op = pipe.pop(0)
            if op[0] == "commit":
                bars[op[1]].arrive()
            else:
                _, kind, it, reads, writes = op
                for r in reads:
                    assert holds[r] == (expect[kind][r], it), \
                        f"{kind} of step {it} found {holds[r]} in {r}"
                    pending_reads[r] -= 1
                for w in writes:
                    write(w, (kind, it))
                busy_until = tick[0] + rng.randint(1, 8)
        if not roles and not pipe and not inflight:
            return True
        if rng.random() < 0.4:
            continue
        order = list(roles)
        rng.shuffle(order)
        for name in order:
            if name in blocked:
                _, bar, parity = blocked[name]
                if not bars[bar].passed(parity):
                    continue
                del blocked[name]
            try:
                ev = next(roles[name])
            except StopIteration:
                del roles[name]
                break
            if ev[0] == "wait" and not bars[ev[1]].passed(ev[2]):
                blocked[name] = ev
            break
    raise AssertionError(f"no progress: blocked {blocked}")


@pytest.mark.parametrize("iters", [1, 2, 3, 8, 33])
def test_protocol_neither_deadlocks_nor_races(iters):
    for seed in range(40):
        assert simulate(iters, seed)


@pytest.mark.parametrize("drop", ["s_free", "shared_free", "own_free"])
def test_the_checker_sees_a_missing_wait(drop):
    with pytest.raises(AssertionError):
        for seed in range(300):
            simulate(12, seed, drop=drop)
