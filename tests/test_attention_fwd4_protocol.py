"""Host restatement of the synchronisation of the fourth-generation attention
forward (csrc/kernels/attention_fwd4.cuh): TMA ring for K / V, one MMA issuer
serving two query tiles, and per tile two softmax threads per row (column halves)
that meet at a two-party named barrier before the probabilities overwrite the first
64 score columns.  Same harness idea as the backward's protocol test: phase-parity
barriers, an in-order tensor pipe, random completion delays and idle ticks; every
buffer carries a version, reads must see the expected one and writes must not come
before the readers of the previous contents.

Roles follow the statement order of the kernel; a change there must be repeated here.
"""
import random

import pytest

KV_STAGES = 2


class Barrier:
    def __init__(self, count=1):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self):
        self.arrived += 1
        if self.arrived == self.count:
            self.arrived, self.completed = 0, self.completed + 1

    def passed(self, parity):
        return (self.completed & 1) != parity


class Buffers:
    def __init__(self):
        self.version, self.pending = {}, {}

    def write(self, buf, version, readers):
        left = self.pending.get(buf)
        assert not left, f"{buf} overwritten with {version} while {left} still have to read {self.version[buf]}"
        self.version[buf] = version
        self.pending[buf] = set(readers)

    def read(self, buf, version, reader):
        assert self.version.get(buf) == version, f"{reader} expected {version} in {buf}, found {self.version.get(buf)}"
        self.pending[buf].discard(reader)


def simulate(n0, n1, seed, rescale_prob=0.3, skip_pair_sync=False):
    """n0 / n1: K/V blocks of the two query tiles (n1 may be 0: the tile does not exist)."""
    rng = random.Random(seed)
    nmax = max(n0, n1)
    n_t = (n0, n1)
    bars = {"q_full": Barrier()}
    for s in range(KV_STAGES):
        for n in ("k_full", "k_empty", "v_full", "v_empty"):
            bars[f"{n}{s}"] = Barrier()
    for t in range(2):
        bars[f"s_full{t}"] = Barrier()
        bars[f"p_full{t}"] = Barrier(2)          # both halves (256 threads in the kernel)
        bars[f"o_full{t}"] = Barrier()
    pair = {t: {"waiting": 0, "generation": 0} for t in range(2)}   # the 64-thread named barrier
    buf = Buffers()
    pipe, inflight, tick = [], [], [0]
    # whether a step grows the running maximum is a property of the data: both halves see the same
    grows = {(t, j): rng.random() < rescale_prob for t in range(2) for j in range(nmax)}

    def tma(action):
        inflight.append((tick[0] + rng.randint(1, 40), action))

    def producer():
        tma(lambda: bars["q_full"].arrive())
        for j in range(nmax):
            s, ph = j % KV_STAGES, (j // KV_STAGES) & 1
            yield ("wait", f"k_empty{s}", ph ^ 1)
            readers = {f"QK{t}" for t in range(2) if j < n_t[t]}

            def k_done(j=j, s=s, readers=readers):
                buf.write(f"K{s}", ("k", j), readers)
                bars[f"k_full{s}"].arrive()
            tma(k_done)
            yield ("wait", f"v_empty{s}", ph ^ 1)
            vreaders = {f"PV{t}" for t in range(2) if j < n_t[t]}

            def v_done(j=j, s=s, vreaders=vreaders):
                buf.write(f"V{s}", ("v", j), vreaders)
                bars[f"v_full{s}"].arrive()
            tma(v_done)

    def mma():
        def qk(t, j):
            s = j % KV_STAGES
            yield ("wait", f"k_full{s}", (j // KV_STAGES) & 1)
            pipe.append(("mma", [(f"K{s}", ("k", j), f"QK{t}")],
                         [(f"A0_{t}", ("s", j), {"h0"}), (f"A1_{t}", ("s", j), {"h0"}), (f"Shi_{t}", ("s", j), {"h1"})]))
            if t == 1 or j >= n1:
                pipe.append(("commit", f"k_empty{s}"))
            pipe.append(("commit", f"s_full{t}"))

        def pv(t, j):
            s = j % KV_STAGES
            yield ("wait", f"v_full{s}", (j // KV_STAGES) & 1)
            yield ("wait", f"p_full{t}", j & 1)
            pipe.append(("mma", [(f"V{s}", ("v", j), f"PV{t}"), (f"A0_{t}", ("p", j), "PV"), (f"A1_{t}", ("p", j), "PV")],
                         [(f"O_{t}", ("o", j), set())]))
            if t == 1 or j >= n1:
                pipe.append(("commit", f"v_empty{s}"))
            pipe.append(("commit", f"o_full{t}"))

        yield ("wait", "q_full", 0)
        yield from qk(0, 0)
        if n1 > 0:
            yield from qk(1, 0)
        for j in range(nmax):
            if j < n0:
                yield from pv(0, j)
            if j + 1 < n0:
                yield from qk(0, j + 1)
            if j < n1:
                yield from pv(1, j)
            if j + 1 < n1:
                yield from qk(1, j + 1)

    def pair_sync(t):
        if skip_pair_sync:
            return
        st = pair[t]
        gen = st["generation"]
        st["waiting"] += 1
        if st["waiting"] == 2:
            st["waiting"], st["generation"] = 0, gen + 1
        while st["generation"] == gen:
            yield ("spin",)

    def softmax(t, half):
        me = f"h{half}"
        for j in range(n_t[t]):
            yield ("wait", f"s_full{t}", j & 1)
            if half == 0:
                buf.read(f"A0_{t}", ("s", j), me)
                buf.read(f"A1_{t}", ("s", j), me)
            else:
                buf.read(f"Shi_{t}", ("s", j), me)
            yield ("work",)
            yield from pair_sync(t)                       # row maximum exchanged; all scores are in registers
            if grows[(t, j)] and j > 0:
                yield ("wait", f"o_full{t}", (j - 1) & 1)
                buf.read(f"O_{t}", ("o", j - 1), me)      # rescale reads and rewrites this thread's half of O
                yield ("work",)
            buf.write(f"A{half}_{t}", ("p", j), {"PV"})
            bars[f"p_full{t}"].arrive()
        if n_t[t] > 0:
            yield ("wait", f"o_full{t}", (n_t[t] - 1) & 1)
            yield from pair_sync(t)                       # row sums exchanged
            buf.read(f"O_{t}", ("o", n_t[t] - 1), me)

    roles = {"producer": producer(), "mma": mma()}
    for t in range(2):
        for half in range(2):
            roles[f"softmax{t}{half}"] = softmax(t, half)
    blocked, pipe_busy_until = {}, 0
    for _ in range(400000):
        tick[0] += 1
        for x in [x for x in inflight if x[0] <= tick[0]]:
            inflight.remove(x)
            x[1]()
        if pipe and tick[0] >= pipe_busy_until:
            op = pipe.pop(0)
            if op[0] == "commit":
                bars[op[1]].arrive()
            else:
                for b, version, reader in op[1]:
                    buf.read(b, version, reader)
                for b, version, readers in op[2]:
                    buf.write(b, version, readers)
                pipe_busy_until = tick[0] + rng.randint(1, 12)
        if not roles and not pipe and not inflight:
            return True
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
    raise AssertionError(f"no progress: blocked {blocked}, roles left {list(roles)}")


@pytest.mark.parametrize("n0,n1", [(1, 0), (1, 2), (3, 4), (5, 6), (7, 0), (9, 10)])
def test_protocol_neither_deadlocks_nor_races(n0, n1):
    for seed in range(100):
        assert simulate(n0, n1, seed)


def test_the_checker_sees_the_missing_pair_barrier():
    """Without the named barrier the second half may write its probabilities over score
    columns the first half has not loaded yet: the harness has to catch that."""
    with pytest.raises(AssertionError):
        for seed in range(300):
            simulate(5, 6, seed, skip_pair_sync=True)
