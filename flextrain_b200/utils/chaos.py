"""Timing perturbation for race hunting: with ``FLEXTRAIN_CHAOS=<max milliseconds>`` the
background threads of the engine (host optimizer worker, NVMe completions) sleep a random
time at their hand-over points, which widens every window in which a consumer could run
ahead of a producer.  Results must not change; the CPU sweeps are run with it.  Unset
(the default) the hook is a constant-time no-op."""
import os
import random
import time

_MAX_MS = float(os.environ.get("FLEXTRAIN_CHAOS", "0") or 0)
_rng = random.Random(int(os.environ.get("FLEXTRAIN_CHAOS_SEED", "0") or 0))


def enabled() -> bool:
    return _MAX_MS > 0


def perturb(_where: str = ""):
    if _MAX_MS > 0:
        time.sleep(_rng.random() * _MAX_MS / 1e3)
