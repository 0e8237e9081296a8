"""Host restatement of the barrier protocol of the second-generation attention
backward (csrc/kernels/attention_bwd2.cuh): the four roles of a CTA are replayed as
coroutines over mbarrier objects with the hardware's phase-parity semantics, the
tensor pipe executes the issued products in order, TMA loads and products complete
after random delays, and every shared-memory / tensor-memory buffer carries the
version it holds.  Over many random schedules the run must never dead-lock, every
read must see the version it expects, and no buffer may be overwritten before every
reader of its current contents is done.

Each role below follows the statement order of the kernel; a change there must be
repeated here.
"""
import random

import pytest


class Barrier:
    def __init__(self, count):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self):
        self.arrived += 1
        if self.arrived == self.count:
            self.arrived, self.completed = 0, self.completed + 1

    def passed(self, parity):
        # try_wait.parity(q) succeeds once the phase with parity q is over, i.e. when the
        # barrier's current phase bit differs from q (a fresh barrier passes q = 1)
        return (self.completed & 1) != parity


class Buffers:
    """Version held by every buffer plus the readers that still have to see it."""
    READERS = {"q": ("S", "dK"), "do": ("dP", "dV"), "tm_s": ("ldS",), "tm_dp:dp": ("lddP",),
               "tm_dp:dq": ("lddQ",), "sP:p": ("dV",), "sdS:ds": ("dK", "dQ"), "stage": ("store",)}

    def __init__(self):
        self.version, self.pending = {}, {}

    def write(self, buf, kind, it):
        left = self.pending.get(buf)
        assert not left, f"{buf} overwritten with {kind}{it} while {left} still have to read {self.version[buf]}"
        self.version[buf] = (kind, it)
        self.pending[buf] = set(self.READERS[kind])

    def read(self, buf, kind, it, reader):
        assert self.version.get(buf) == (kind, it), \
            f"{reader} expected {kind}{it} in {buf}, found {self.version.get(buf)}"
        self.pending[buf].discard(reader)


def simulate(iters, seed):
    rng = random.Random(seed)
    names1 = ["kv_full", "do_full", "do_empty", "s_full", "dp_full", "dq_full", "stage_free", "acc_full",
              "q_full0", "q_full1", "q_empty0", "q_empty1"]
    bars = {n: Barrier(1) for n in names1}
    # 256 softmax threads arrive together here: one arrival stands for all of them
    for n in ("s_free", "dp_free", "p_full", "ds_full", "dqs_full"):
        bars[n] = Barrier(1)
    buf = Buffers()
    pipe = []          # tensor pipe: products and commits in issue order
    inflight = []      # (ready_tick, action) for TMA completions
    tick = [0]

    def tma(action):
        inflight.append((tick[0] + rng.randint(1, 40), action))

    # ---------------------------------------------------------------- roles
    def producer():
        tma(lambda: bars["kv_full"].arrive())
        for it in range(iters):
            st = it & 1
            yield ("wait", f"q_empty{st}", ((it >> 1) & 1) ^ 1)

            def q_done(it=it, st=st):
                buf.write(f"q{st}", "q", it)
                bars[f"q_full{st}"].arrive()
            tma(q_done)
            yield ("wait", "do_empty", (it & 1) ^ 1)

            def do_done(it=it):
                buf.write("do", "do", it)
                bars["do_full"].arrive()
            tma(do_done)

    def issue(reads, writes, name):
        pipe.append(("mma", reads, writes, name))

    def commit(bar):
        pipe.append(("commit", bar))

    def mma():
        yield ("wait", "kv_full", 0)
        yield ("wait", "q_full0", 0)
        issue([("q0", "q", 0, "S")], [("tm_s", "tm_s", 0)], "S0")
        commit("s_full")
        for it in range(iters):
            ph, st = it & 1, it & 1
            yield ("wait", "do_full", ph)
            if it > 0:
                yield ("wait", "dp_free", ph ^ 1)
            issue([("do", "do", it, "dP")], [("tm_dp", "tm_dp:dp", it)], f"dP{it}")
            commit("dp_full")
            yield ("wait", "p_full", ph)
            issue([("sP", "sP:p", it, "dV"), ("do", "do", it, "dV")], [], f"dV{it}")
            commit("do_empty")
            yield ("wait", "ds_full", ph)
            issue([("sdS", "sdS:ds", it, "dK"), (f"q{st}", "q", it, "dK")], [], f"dK{it}")
            commit(f"q_empty{st}")
            issue([("sdS", "sdS:ds", it, "dQ")], [("tm_dp", "tm_dp:dq", it)], f"dQ{it}")
            commit("dq_full")
            if it + 1 < iters:
                nst = (it + 1) & 1
                yield ("wait", f"q_full{nst}", ((it + 1) >> 1) & 1)
                yield ("wait", "s_free", ph)
                issue([(f"q{nst}", "q", it + 1, "S")], [("tm_s", "tm_s", it + 1)], f"S{it + 1}")
                commit("s_full")
        commit("acc_full")

    def softmax():
        for it in range(iters):
            ph = it & 1
            yield ("wait", "s_full", ph)
            buf.read("tm_s", "tm_s", it, "ldS")
            bars["s_free"].arrive()
            if it > 0:
                yield ("wait", "stage_free", (it - 1) & 1)
            yield ("work",)
            buf.write("sP", "sP:p", it)
            bars["p_full"].arrive()
            yield ("wait", "dp_full", ph)
            buf.read("tm_dp", "tm_dp:dp", it, "lddP")
            yield ("work",)
            buf.write("sdS", "sdS:ds", it)
            bars["ds_full"].arrive()
            yield ("wait", "dq_full", ph)
            buf.read("tm_dp", "tm_dp:dq", it, "lddQ")
            bars["dp_free"].arrive()
            yield ("work",)
            # the dQ staging area is the P and dS tiles together
            buf.write("sP", "stage", it)
            buf.write("sdS", "stage", it)
            bars["dqs_full"].arrive()
        yield ("wait", "acc_full", 0)

    def store():
        for it in range(iters):
            yield ("wait", "dqs_full", it & 1)
            buf.read("sP", "stage", it, "store")
            buf.read("sdS", "stage", it, "store")
            yield ("work",)
            bars["stage_free"].arrive()

    roles = {"producer": producer(), "mma": mma(), "softmax": softmax(), "store": store()}
    blocked = {}
    pipe_busy_until = 0
    for _ in range(200000):
        tick[0] += 1
        # TMA completions
        due = [x for x in inflight if x[0] <= tick[0]]
        for x in due:
            inflight.remove(x)
            x[1]()
        # tensor pipe: one entry at a time, in order
        if pipe and tick[0] >= pipe_busy_until:
            op = pipe.pop(0)
            if op[0] == "commit":
                bars[op[1]].arrive()
            else:
                for b, kind, it, reader in op[1]:
                    buf.read(b, kind, it, reader)
                for b, kind, it in op[2]:
                    buf.write(b, kind, it)
                pipe_busy_until = tick[0] + rng.randint(1, 12)
        # one step of a randomly chosen role that can move; on some ticks nobody moves, so that
        # a role can be late even when it is the only one able to run
        if rng.random() < 0.5:
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
        if not roles and not pipe and not inflight:
            return True
    raise AssertionError(f"no progress: blocked {blocked}, pipe {pipe[:3]}, roles left {list(roles)}")


@pytest.mark.parametrize("iters", [1, 2, 3, 4, 7, 12])
def test_protocol_neither_deadlocks_nor_races(iters):
    for seed in range(150):
        assert simulate(iters, seed)


def test_the_checker_sees_a_missing_wait():
    """The harness itself must notice a protocol error: dropping the wait that keeps dP of
    the next block off the columns that still hold dQ of this one (dp_free) has to surface
    as a stale read or an early overwrite in some schedule.  (Dropping s_free would not: the
    issue order already puts S of block i+1 behind ds_full of block i, which the softmax
    warps signal after they have loaded S of block i; the kernel keeps that wait as a guard.)"""
    import inspect
    import textwrap
    src = textwrap.dedent(inspect.getsource(simulate))
    broken = src.replace('yield ("wait", "dp_free", ph ^ 1)', 'pass')
    assert broken != src
    scope = {"random": random, "Barrier": Barrier, "Buffers": Buffers}
    exec(broken, scope)
    with pytest.raises(AssertionError):
        for seed in range(300):
            scope["simulate"](6, seed)
