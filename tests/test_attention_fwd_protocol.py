"""Host restatement of the attention forward's synchronisation (csrc/kernels/attention_fwd2.cuh).

One CTA holds two query tiles; tile 0 needs n0 K/V blocks, tile 1 one more (or none: it may be
absent).  K_j and V_j stream through a two-stage ring.

  loader     per block j: waits k_empty[s] -> loads K_j -> k_full[s]; waits v_empty[s] -> V_j
  issuer     QK0(0), QK1(0), then per block j and tile t one hand-over: waits for V_j and K_j+1
             only where the tile is the first to read them, and for P_t(j); issues PV_t(j) and
             QK_t(j+1) back to back; the last reader of a stage commits its release
  softmax t  per block: waits s_full[t], reads S_t, writes P_t over it, arrives p_full[t]; at the
             end waits for the last PV

Replayed with phase-parity barriers, an in-order tensor pipe and random delays.  Checked: every
product reads the block it means to, no stage is refilled while a product still has to read it,
P_t(j) is consumed before S_t(j+1) lands on it, and the walk ends.  Two mutations must be
noticed: tile 1 not waiting for a block that tile 0 no longer reads, and a stage released by the
first reader instead of the last.
"""
import random

import pytest

STAGES = 2


class Barrier:
    def __init__(self, count=1):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self, n=1):
        self.arrived += n
        if self.arrived >= self.count:
            self.arrived, self.completed = 0, self.completed + 1

    def passed(self, parity):
        return (self.completed & 1) != parity


def simulate(n0, tile1, seed, mutate=None):
    rng = random.Random(seed)
    n1 = n0 + 1 if tile1 else 0
    nmax = max(n0, n1)
    n_of = (n0, n1)
    bars = {"q_full": Barrier()}
    for s in range(STAGES):
        for n in ("k_full", "k_empty", "v_full", "v_empty"):
            bars[f"{n}{s}"] = Barrier()
    for t in (0, 1):
        for n in ("s_full", "p_full", "o_full"):
            bars[f"{n}{t}"] = Barrier()
    holds = {f"{kv}{s}": None for kv in "KV" for s in range(STAGES)}
    pending = {k: 0 for k in holds}
    s_tile = {0: None, 1: None}            # ("S", j) after QK, ("P", j) once the softmax wrote P over it
    pv_done = {0: 0, 1: 0}
    pipe, inflight, tick = [], [], [0]

    def loader():
        bars["q_full"].arrive()
        for j in range(nmax):
            s, ph = j % STAGES, (j // STAGES) & 1
            for kv, full, empty in (("K", "k_full", "k_empty"), ("V", "v_full", "v_empty")):
                yield ("wait", f"{empty}{s}", ph ^ 1)

                def landed(kv=kv, s=s, j=j, full=full):
                    assert pending[f"{kv}{s}"] == 0, f"{kv} stage {s} refilled with block {j} while still to be read"
                    holds[f"{kv}{s}"] = j
                    bars[f"{full}{s}"].arrive()
                inflight.append((tick[0] + rng.randint(1, 40), landed))

    def issue_qk(t, j):
        s = j % STAGES
        pending[f"K{s}"] += 1
        pipe.append(("qk", t, j, s))
        last = (t == 1 or j >= n1) if mutate != "first_reader_releases" else (t == 0)
        if last:
            pipe.append(("commit", f"k_empty{s}"))
        pipe.append(("commit", f"s_full{t}"))

    def issue_pv(t, j):
        s = j % STAGES
        pending[f"V{s}"] += 1
        pipe.append(("pv", t, j, s))
        last = (t == 1 or j >= n1) if mutate != "first_reader_releases" else (t == 0)
        if last:
            pipe.append(("commit", f"v_empty{s}"))
        pipe.append(("commit", f"o_full{t}"))

    def issuer():
        yield ("wait", "q_full", 0)
        yield ("wait", "k_full0", 0)
        issue_qk(0, 0)
        if n1 > 0:
            issue_qk(1, 0)
        for j in range(nmax):
            for t in (0, 1):
                n_t = n_of[t]
                has_pv, has_qk = j < n_t, j + 1 < n_t
                first_v = True if t == 0 else j >= n0
                first_k = True if t == 0 else j + 1 >= n0
                if mutate == "tile1_never_waits" and t == 1:
                    first_v = first_k = False
                if has_pv:
                    if first_v:
                        yield ("wait", f"v_full{j % STAGES}", (j // STAGES) & 1)
                    yield ("wait", f"p_full{t}", j & 1)
                if has_qk and first_k:
                    yield ("wait", f"k_full{(j + 1) % STAGES}", ((j + 1) // STAGES) & 1)
                if has_pv:
                    issue_pv(t, j)
                if has_qk:
                    issue_qk(t, j + 1)

    def softmax(t):
        n_t = n_of[t]
        for j in range(n_t):
            yield ("wait", f"s_full{t}", j & 1)
            assert s_tile[t] == ("S", j), f"softmax of tile {t}, block {j} found {s_tile[t]}"
            if j > 0 and rng.random() < 0.2:                      # the rare rescale of O
                yield ("wait", f"o_full{t}", (j - 1) & 1)
            yield ("work",)
            s_tile[t] = ("P", j)
            bars[f"p_full{t}"].arrive()
        if n_t > 0:
            yield ("wait", f"o_full{t}", (n_t - 1) & 1)
            assert pv_done[t] == n_t

    roles = {"loader": loader(), "issuer": issuer(), "softmax0": softmax(0), "softmax1": softmax(1)}
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
            elif op[0] == "qk":
                _, t, j, s = op
                assert holds[f"K{s}"] == j, f"QK of tile {t}, block {j} found block {holds[f'K{s}']} in K stage {s}"
                pending[f"K{s}"] -= 1
                assert s_tile[t] is None or s_tile[t] == ("P", j - 1) and pv_done[t] == j, \
                    f"S of tile {t}, block {j} lands on {s_tile[t]} with {pv_done[t]} PV products done"
                s_tile[t] = ("S", j)
                busy_until = tick[0] + rng.randint(1, 8)
            else:
                _, t, j, s = op
                assert holds[f"V{s}"] == j, f"PV of tile {t}, block {j} found block {holds[f'V{s}']} in V stage {s}"
                pending[f"V{s}"] -= 1
                assert s_tile[t] == ("P", j), f"PV of tile {t}, block {j} found {s_tile[t]} where P should be"
                pv_done[t] += 1
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


@pytest.mark.parametrize("n0,tile1", [(1, False), (1, True), (2, True), (3, False), (5, True), (16, True)])
def test_protocol_neither_deadlocks_nor_races(n0, tile1):
    for seed in range(40):
        assert simulate(n0, tile1, seed)


@pytest.mark.parametrize("mutate", ["tile1_never_waits", "first_reader_releases"])
def test_the_checker_sees_the_mutations(mutate):
    with pytest.raises(AssertionError):
        for seed in range(300):
            simulate(6, True, seed, mutate=mutate)
