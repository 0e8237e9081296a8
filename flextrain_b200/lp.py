"""Small linear-programme front end for the offload planner.

``minimise c.x  s.t.  A_ub x <= b_ub,  A_eq x = b_eq,  lo <= x <= hi``

Uses SciPy's HiGHS when SciPy is importable and falls back to a dense two-phase
simplex (Bland's rule) written here, so the planner has no hard dependency -
the reference imports PuLP at module import time although it is not among its
requirements (flextrain/auto_config.py:3, flextrain/engine.py:7).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np


class LinearProgram:
    """Incrementally built LP over named variables."""

    def __init__(self):
        self.names: List[str] = []
        self.lo: List[float] = []
        self.hi: List[Optional[float]] = []
        self.cost: Dict[str, float] = {}
        self.ub: List[Tuple[Dict[str, float], float]] = []
        self.eq: List[Tuple[Dict[str, float], float]] = []

    def var(self, name: str, lo: float = 0.0, hi: Optional[float] = None) -> str:
        self.names.append(name)
        self.lo.append(lo)
        self.hi.append(hi)
        return name

    def minimise(self, terms: Dict[str, float]):
        self.cost = dict(terms)

    def add_le(self, terms: Dict[str, float], rhs: float):
        """sum(coef * var) <= rhs"""
        self.ub.append((dict(terms), float(rhs)))

    def add_ge(self, terms: Dict[str, float], rhs: float):
        self.ub.append(({k: -v for k, v in terms.items()}, -float(rhs)))

    def add_eq(self, terms: Dict[str, float], rhs: float):
        self.eq.append((dict(terms), float(rhs)))

    def _dense(self):
        idx = {n: i for i, n in enumerate(self.names)}
        n = len(self.names)

        def rows(cons):
            A = np.zeros((len(cons), n))
            b = np.zeros(len(cons))
            for r, (terms, rhs) in enumerate(cons):
                for k, v in terms.items():
                    A[r, idx[k]] += v
                b[r] = rhs
            return A, b

        c = np.zeros(n)
        for k, v in self.cost.items():
            c[idx[k]] += v
        A_ub, b_ub = rows(self.ub)
        A_eq, b_eq = rows(self.eq)
        return c, A_ub, b_ub, A_eq, b_eq

    def solve(self, prefer_scipy: bool = True) -> Optional[Dict[str, float]]:
        """Optimal assignment, or None when infeasible / unbounded."""
        c, A_ub, b_ub, A_eq, b_eq = self._dense()
        # Rows arrive in their natural units (bytes ~1e11 next to seconds ~1e-2): scale every row to
        # a largest coefficient of 1, or the solver's absolute tolerances swallow the small objective
        # terms that break ties between placements of equal step time.
        for A, b in ((A_ub, b_ub), (A_eq, b_eq)):
            for r in range(len(b)):
                scale = np.abs(A[r]).max()
                if scale > 0:
                    A[r] /= scale
                    b[r] /= scale
        x = None
        if prefer_scipy:
            try:
                from scipy.optimize import linprog
                res = linprog(c, A_ub=A_ub if len(b_ub) else None, b_ub=b_ub if len(b_ub) else None,
                              A_eq=A_eq if len(b_eq) else None, b_eq=b_eq if len(b_eq) else None,
                              bounds=list(zip(self.lo, self.hi)), method="highs")
                x = res.x if res.status == 0 else None
                if res.status in (2, 3):
                    return None
            except ImportError:
                x = None
        if x is None:
            x = _simplex(c, A_ub, b_ub, A_eq, b_eq, self.lo, self.hi)
            if x is None:
                return None
        return {n: float(v) for n, v in zip(self.names, x)}


def _simplex(c, A_ub, b_ub, A_eq, b_eq, lo, hi) -> Optional[np.ndarray]:
    """Dense two-phase simplex with Bland's rule.  Variables are shifted to
    ``y = x - lo >= 0``; finite upper bounds become extra rows."""
    n = len(c)
    lo = np.asarray(lo, dtype=float)
    rows_ub = [A_ub[i] for i in range(len(b_ub))]
    rhs_ub = [b_ub[i] - A_ub[i] @ lo for i in range(len(b_ub))]
    for j, h in enumerate(hi):
        if h is not None:
            e = np.zeros(n)
            e[j] = 1.0
            rows_ub.append(e)
            rhs_ub.append(h - lo[j])
    rows_eq = [A_eq[i] for i in range(len(b_eq))]
    rhs_eq = [b_eq[i] - A_eq[i] @ lo for i in range(len(b_eq))]
    m_ub, m_eq = len(rows_ub), len(rows_eq)
    m = m_ub + m_eq
    # columns: y (n) | slack (m_ub) | artificial (m)
    T = np.zeros((m, n + m_ub + m))
    b = np.zeros(m)
    for i in range(m_ub):
        T[i, :n] = rows_ub[i]
        T[i, n + i] = 1.0
        b[i] = rhs_ub[i]
    for i in range(m_eq):
        T[m_ub + i, :n] = rows_eq[i]
        b[m_ub + i] = rhs_eq[i]
    for i in range(m):
        if b[i] < 0:
            T[i] *= -1
            b[i] *= -1
        T[i, n + m_ub + i] = 1.0
    basis = [n + m_ub + i for i in range(m)]
    total = n + m_ub + m

    def run(cost, allowed):
        nonlocal T, b, basis
        for _ in range(20000):
            cb = cost[basis]
            reduced = cost - cb @ T
            enter = -1
            for j in range(allowed):
                if reduced[j] < -1e-9 and j not in basis:
                    enter = j
                    break
            if enter < 0:
                return True
            col = T[:, enter]
            ratios = [(b[i] / col[i], basis[i], i) for i in range(m) if col[i] > 1e-12]
            if not ratios:
                return False
            _, _, leave = min(ratios)
            piv = T[leave, enter]
            T[leave] /= piv
            b[leave] /= piv
            for i in range(m):
                if i != leave and abs(T[i, enter]) > 1e-15:
                    f = T[i, enter]
                    T[i] -= f * T[leave]
                    b[i] -= f * b[leave]
            basis[leave] = enter
        return False

    phase1 = np.zeros(total)
    phase1[n + m_ub:] = 1.0
    if not run(phase1, total):
        return None
    if sum(b[i] for i in range(m) if basis[i] >= n + m_ub) > 1e-7:
        return None
    cost = np.zeros(total)
    cost[:n] = c
    cost[n + m_ub:] = 1e9          # keep artificials out
    if not run(cost, n + m_ub):
        return None
    y = np.zeros(total)
    for i in range(m):
        y[basis[i]] = b[i]
    return y[:n] + lo
