"""Host restatement of the CTA-pair GEMM's synchronisation (csrc/kernels/gemm2_kernel.cuh,
shared by the SwiGLU-epilogue variant in gemm2_swiglu.cuh): two CTAs, each with its own
TMA producer and four epilogue warps, one MMA issuer in the leader.

  full[s]        lives in the leader; armed with the bytes of BOTH CTAs' loads
  empty[s]       one per CTA; the leader's commit arrives on both
  tmem_full[a]   one per CTA; the leader's commit arrives on both
  tmem_empty[a]  lives in the leader; 8 arrivals (4 epilogue warps x 2 CTAs)

Replayed with phase-parity barriers, an in-order tensor pipe, random TMA / MMA delays and
idle ticks.  A stage must never be refilled before the product that reads it has run, an
accumulator never be overwritten before both CTAs' epilogues have drained it, and the run
must end for any number of tiles and k-blocks.
"""
import random

import pytest

STAGES = 6


class Barrier:
    def __init__(self, count=1):
        self.count, self.arrived, self.completed = count, 0, 0

    def arrive(self, n=1):
        self.arrived += n
        if self.arrived >= self.count:
            self.arrived, self.completed = 0, self.completed + 1

    def passed(self, parity):
        return (self.completed & 1) != parity


def simulate(tiles, kt, seed, drop_tmem_empty_wait=False):
    rng = random.Random(seed)
    bars = {}
    for s in range(STAGES):
        bars[f"full{s}"] = Barrier(2)                 # expect_tx of both CTAs' bytes: two completions
        for cta in (0, 1):
            bars[f"empty{s}_{cta}"] = Barrier()
    for a in (0, 1):
        bars[f"tmem_empty{a}"] = Barrier(8)
        for cta in (0, 1):
            bars[f"tmem_full{a}_{cta}"] = Barrier()
    stage_holds = {(cta, s): None for cta in (0, 1) for s in range(STAGES)}     # (tile, kb) or None once read
    stage_read = {(cta, s): True for cta in (0, 1) for s in range(STAGES)}
    acc_holds = {a: None for a in (0, 1)}
    acc_readers = {a: set() for a in (0, 1)}
    pipe, inflight, tick = [], [], [0]

    def producer(cta):
        stage, phase = 0, 0
        for t in range(tiles):
            for kb in range(kt):
                yield ("wait", f"empty{stage}_{cta}", phase ^ 1)

                def landed(cta=cta, stage=stage, t=t, kb=kb):
                    assert stage_read[(cta, stage)], f"stage {stage} of CTA {cta} refilled before it was read"
                    stage_holds[(cta, stage)] = (t, kb)
                    stage_read[(cta, stage)] = False
                    bars[f"full{stage}"].arrive()
                inflight.append((tick[0] + rng.randint(1, 30), landed))
                stage += 1
                if stage == STAGES:
                    stage, phase = 0, phase ^ 1

    def mma():
        stage, phase = 0, 0
        for it in range(tiles):
            acc, acc_phase = it & 1, (it >> 1) & 1
            if not drop_tmem_empty_wait:
                yield ("wait", f"tmem_empty{acc}", acc_phase ^ 1)
            for kb in range(kt):
                yield ("wait", f"full{stage}", phase)
                pipe.append(("mma", it, kb, stage, acc))
                pipe.append(("commit", [f"empty{stage}_0", f"empty{stage}_1"]))
                stage += 1
                if stage == STAGES:
                    stage, phase = 0, phase ^ 1
            pipe.append(("commit", [f"tmem_full{acc}_0", f"tmem_full{acc}_1"]))

    def epilogue(cta, warp):
        for it in range(tiles):
            acc, acc_phase = it & 1, (it >> 1) & 1
            yield ("wait", f"tmem_full{acc}_{cta}", acc_phase)
            assert acc_holds[acc] == it, f"epilogue of tile {it} found tile {acc_holds[acc]} in accumulator {acc}"
            yield ("work",)
            acc_readers[acc].discard((cta, warp))
            bars[f"tmem_empty{acc}"].arrive()

    roles = {"p0": producer(0), "p1": producer(1), "mma": mma()}
    for cta in (0, 1):
        for w in range(4):
            roles[f"e{cta}{w}"] = epilogue(cta, w)
    blocked, busy_until = {}, 0
    for _ in range(600000):
        tick[0] += 1
        for x in [x for x in inflight if x[0] <= tick[0]]:
            inflight.remove(x)
            x[1]()
        if pipe and tick[0] >= busy_until:
            op = pipe.pop(0)
            if op[0] == "commit":
                for b in op[1]:
                    bars[b].arrive()
            else:
                _, it, kb, stage, acc = op
                for cta in (0, 1):
                    assert stage_holds[(cta, stage)] == (it, kb), \
                        f"product ({it},{kb}) found {stage_holds[(cta, stage)]} in stage {stage} of CTA {cta}"
                    stage_read[(cta, stage)] = True
                if kb == 0:
                    assert not acc_readers[acc], f"accumulator {acc} overwritten while {acc_readers[acc]} still read it"
                    acc_holds[acc] = it
                if kb == kt - 1:
                    acc_readers[acc] = {(cta, w) for cta in (0, 1) for w in range(4)}
                busy_until = tick[0] + rng.randint(1, 6)
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


@pytest.mark.parametrize("tiles,kt", [(1, 1), (1, 9), (2, 5), (3, 13), (7, 4), (14, 2)])
def test_protocol_neither_deadlocks_nor_races(tiles, kt):
    for seed in range(40):
        assert simulate(tiles, kt, seed)


def test_the_checker_sees_a_missing_accumulator_wait():
    with pytest.raises(AssertionError):
        for seed in range(200):
            simulate(9, 2, seed, drop_tmem_empty_wait=True)
