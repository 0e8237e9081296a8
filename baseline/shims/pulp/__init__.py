"""Stand-in for PuLP, used ONLY by the reference arm of bench.py.

The reference imports ``pulp`` (and ``LpProblem`` / ``LpVariable`` from it) at
module import time for its auto-config planner, although the package is not
among its requirements and is absent from this image.  The benchmark never runs
that planner, so importable names are all that is needed; constructing or using
any of them raises.
"""


class _Unavailable:
    def __init__(self, *args, **kwargs):
        raise ImportError("PuLP is not installed; the reference's auto_config cannot run here")


class LpProblem(_Unavailable):
    pass


class LpVariable(_Unavailable):
    pass


class _SolverDefault:
    msg = False


LpSolverDefault = _SolverDefault()


def value(*args, **kwargs):
    raise ImportError("PuLP is not installed; the reference's auto_config cannot run here")
