"""Minimal PuLP-compatible modelling layer over ``scipy.optimize.milp`` (HiGHS).

Only for the benchmark harness: the reference imports ``pulp`` and drives the external CBC binary,
neither of which exists in this offline image.  This module implements the subset of the PuLP API
the reference touches – binary variables, affine expressions, ``lpSum``, named constraints,
``LpProblem`` with ``+=``, ``solve``, ``status``, ``value`` – so the *unmodified* reference code can
run; the solver underneath is HiGHS instead of CBC.
"""
from __future__ import annotations

from collections import OrderedDict

import numpy as np

LpBinary = "Binary"
LpInteger = "Integer"
LpContinuous = "Continuous"
LpMinimize = 1
LpMaximize = -1
LpStatusOptimal = 1
LpStatusInfeasible = -1
LpStatus = {1: "Optimal", -1: "Infeasible", 0: "Not Solved"}


class LpAffineExpression:
    __slots__ = ("terms", "const")

    def __init__(self, terms=None, const=0.0):
        self.terms = terms if terms is not None else {}
        self.const = const

    @staticmethod
    def _of(x):
        if isinstance(x, LpAffineExpression):
            return x
        if isinstance(x, LpVariable):
            return LpAffineExpression({x: 1.0})
        return LpAffineExpression({}, float(x))

    def copy(self):
        return LpAffineExpression(dict(self.terms), self.const)

    def __add__(self, o):
        r = self.copy()
        o = self._of(o)
        for v, c in o.terms.items():
            r.terms[v] = r.terms.get(v, 0.0) + c
        r.const += o.const
        return r

    __radd__ = __add__

    def __iadd__(self, o):
        o = self._of(o)
        for v, c in o.terms.items():
            self.terms[v] = self.terms.get(v, 0.0) + c
        self.const += o.const
        return self

    def __neg__(self):
        return LpAffineExpression({v: -c for v, c in self.terms.items()}, -self.const)

    def __sub__(self, o):
        return self + (-self._of(o))

    def __rsub__(self, o):
        return self._of(o) - self

    def __mul__(self, k):
        k = float(k)
        return LpAffineExpression({v: c * k for v, c in self.terms.items()}, self.const * k)

    __rmul__ = __mul__

    def __eq__(self, o):  # noqa: D105
        return LpConstraint(self - self._of(o), 0)

    def __le__(self, o):
        return LpConstraint(self - self._of(o), -1)

    def __ge__(self, o):
        return LpConstraint(self - self._of(o), 1)

    __hash__ = None

    def items(self):
        return self.terms.items()

    def value(self):
        return self.const + sum(c * (v.varValue or 0.0) for v, c in self.terms.items())


class LpVariable:
    _counter = 0

    def __init__(self, name, lowBound=None, upBound=None, cat=LpContinuous):
        self.name = name
        self.cat = cat
        self.lowBound = 0 if cat == LpBinary else lowBound
        self.upBound = 1 if cat == LpBinary else upBound
        self.varValue = None
        self._id = LpVariable._counter
        LpVariable._counter += 1

    def __hash__(self):
        return self._id

    def value(self):
        return self.varValue

    def _e(self):
        return LpAffineExpression({self: 1.0})

    def __add__(self, o):
        return self._e() + o

    __radd__ = __add__

    def __sub__(self, o):
        return self._e() - o

    def __rsub__(self, o):
        return LpAffineExpression._of(o) - self._e()

    def __mul__(self, k):
        return self._e() * k

    __rmul__ = __mul__

    def __neg__(self):
        return -self._e()

    def __eq__(self, o):
        if isinstance(o, LpVariable) and o is self:
            return True
        return self._e() == o

    def __le__(self, o):
        return self._e() <= o

    def __ge__(self, o):
        return self._e() >= o

    def __repr__(self):
        return self.name


class LpConstraint:
    """``expr (sense) 0`` with sense -1: <=, 0: ==, 1: >=."""

    def __init__(self, expr: LpAffineExpression, sense: int, name=None):
        self.expr = expr
        self.sense = sense
        self.name = name

    def items(self):
        return self.expr.terms.items()

    def value(self):
        return self.expr.value()

    def valid(self, eps=1e-6):
        v = self.value()
        if self.sense == 0:
            return abs(v) <= eps
        return v <= eps if self.sense < 0 else v >= -eps

    def __repr__(self):
        op = {0: "=", -1: "<=", 1: ">="}[self.sense]
        lhs = " + ".join(f"{c}*{v.name}" for v, c in list(self.expr.terms.items())[:8])
        return f"{lhs} {op} {-self.expr.const}"


def lpSum(items):
    r = LpAffineExpression()
    for it in items:
        if isinstance(it, LpVariable):
            r.terms[it] = r.terms.get(it, 0.0) + 1.0
        else:
            r += it
    return r


def value(x):
    if x is None:
        return None
    if isinstance(x, (LpAffineExpression, LpVariable, LpConstraint)):
        return x.value()
    return x


class PULP_CBC_CMD:
    def __init__(self, msg=False, timeLimit=None, **kw):
        self.msg = msg
        self.timeLimit = timeLimit


class LpProblem:
    def __init__(self, name="problem", sense=LpMinimize):
        self.name = name
        self.sense = sense
        self.objective = None
        self.constraints = OrderedDict()
        self.status = 0
        self._anon = 0

    def __iadd__(self, other):
        if isinstance(other, tuple):
            c, name = other
        else:
            c, name = other, None
        if isinstance(c, LpConstraint):
            if name is None:
                self._anon += 1
                name = f"_C{self._anon}"
            c.name = name
            self.constraints[name] = c
        elif isinstance(c, (LpAffineExpression, LpVariable)):
            self.objective = LpAffineExpression._of(c)
        elif c is True or c is False:
            pass
        else:
            raise TypeError(f"cannot add {type(c)} to a problem")
        return self

    def variables(self):
        seen = OrderedDict()
        if self.objective is not None:
            for v in self.objective.terms:
                seen[v] = None
        for c in self.constraints.values():
            for v in c.expr.terms:
                seen[v] = None
        return list(seen)

    def solve(self, solver=None):
        from scipy.optimize import Bounds, LinearConstraint, milp
        from scipy.sparse import coo_matrix

        vs = self.variables()
        idx = {v: i for i, v in enumerate(vs)}
        n = len(vs)
        cost = np.zeros(n)
        for v, c in (self.objective.terms.items() if self.objective is not None else ()):
            cost[idx[v]] = c * (1 if self.sense == LpMinimize else -1)
        rows, cols, vals, lo, hi = [], [], [], [], []
        for r, c in enumerate(self.constraints.values()):
            for v, k in c.expr.terms.items():
                rows.append(r)
                cols.append(idx[v])
                vals.append(k)
            rhs = -c.expr.const
            lo.append(rhs if c.sense >= 0 else -np.inf)
            hi.append(rhs if c.sense <= 0 else np.inf)
        m = len(self.constraints)
        A = coo_matrix((vals, (rows, cols)), shape=(m, n)).tocsr()
        lb = np.array([v.lowBound if v.lowBound is not None else -np.inf for v in vs], dtype=float)
        ub = np.array([v.upBound if v.upBound is not None else np.inf for v in vs], dtype=float)
        integrality = np.array([0 if v.cat == LpContinuous else 1 for v in vs])
        opts = {"disp": bool(getattr(solver, "msg", False))}
        if getattr(solver, "timeLimit", None):
            opts["time_limit"] = float(solver.timeLimit)
        res = milp(c=cost, constraints=LinearConstraint(A, np.array(lo), np.array(hi)) if m else None,
                   integrality=integrality, bounds=Bounds(lb, ub), options=opts)
        if res.x is None:
            self.status = LpStatusInfeasible
            for v in vs:
                v.varValue = 0.0
            return self.status
        for v, x in zip(vs, res.x):
            v.varValue = float(round(x)) if v.cat != LpContinuous else float(x)
        self.status = LpStatusOptimal
        return self.status
