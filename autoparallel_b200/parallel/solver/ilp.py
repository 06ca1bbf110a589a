"""Sharding search as a mixed-integer linear program.

Decision variables (binary):

* ``y[c, s]``      – node class ``c`` runs with its candidate strategy ``s``;
* ``z[e, s, j]``   – on edge class ``e`` (producer → consumer argument), the producer uses its
  strategy ``j`` while the consumer uses strategy ``s`` (so the tensor is redistributed from the
  producer's output placement ``j`` to the consumer's required input placement for ``s``).

Minimise  ``Σ mult_c · compute[c, s] · y[c, s]  +  Σ mult_e · (comm[e, s, j] + ε·changed) · z[e, s, j]``
subject to

1. one strategy per node:                 ``Σ_s y[c, s] = 1``
2. edge/consumer agreement:               ``Σ_j z[e, s, j] = y[consumer(e), s]``
3. edge/producer agreement (flow):        ``Σ_s z[e, s, j] = y[producer(e), j]``
4. impossible redistributions:            ``comm = ∞  ⇒  z = 0``
5. forward/backward twins (parameter & gradient, input & input-gradient, output & tangent)
   take the same placement;
6. mixed precision: the parameter all-gather happens on the low-precision side of the cast and
   the gradient reduction on the high-precision side;
7. user constraints: fixed placement of any node / input / output, and a band on the summed
   per-parameter shard ratio (the FSDP knob).

``class`` = set of nodes proven locally isomorphic by ``cluster.refine_colors``; ``mult`` is the
class size.  The model is handed to HiGHS through ``scipy.optimize.milp``.

The reference formulates the same search with one variable per (node, argument, output
strategy, input strategy) and solves it with PuLP/CBC (autoparallel/optimize_sharding.py:6-70,
481-588, 665-941); the node/edge split above is this framework's own and needs no external
solver binary.
"""
from __future__ import annotations

import dataclasses
import logging
import math
import operator
import time
from collections import defaultdict
from typing import Any, Optional, Sequence

import numpy as np
import torch
import torch.fx as fx

from ..cost import comm as comm_cost
from ..cost import compute as compute_cost
from ..frontend.graph_canon import all_input_nodes
from ..frontend.trace import JointGraph
from ..strategies import options as opt
from ..strategies.dtensor_adapter import (
    DTensorSpec,
    OpSpec,
    OpStrategy,
    Partial,
    Placement,
    Replicate,
    Shard,
    all_options,
    local_shape,
)
from .cluster import refine_colors

logger = logging.getLogger(__name__)

INF_COST = 1e12
TRANSITION_EPS = 1.0  # tie-breaker per redistributed edge, microseconds


class InfeasibleError(RuntimeError):
    pass


@dataclasses.dataclass
class Constraint:
    name: str
    kind: str  # "node" | "memory"
    node: Optional[fx.Node] = None
    allowed: Optional[list[int]] = None  # strategy indices allowed for ``node``
    low: float = 0.0
    high: float = 1.0
    description: str = ""


def _produces_tensor(val) -> bool:
    if isinstance(val, torch.Tensor):
        return True
    if isinstance(val, (tuple, list)):
        return any(isinstance(v, torch.Tensor) for v in val)
    return False


def _out_placements(spec: OpSpec):
    o = spec.output_specs
    if isinstance(o, DTensorSpec):
        return o.placements
    return tuple(x.placements if x is not None else None for x in o)


class ShardingOptimizer:
    def __init__(
        self,
        joint: JointGraph,
        mesh,
        *,
        force_grad_reduce_in_higher_precision: bool = False,
        repeated_subgraphs: bool = True,
        even_only: bool = True,
        cluster_rounds: int = 4,
        time_limit: Optional[float] = None,
    ):
        t0 = time.perf_counter()
        self.joint = joint
        self.gm = joint.gm
        self.graph = joint.gm.graph
        self.mesh = mesh
        self.even_only = even_only
        self.repeated_subgraphs = repeated_subgraphs
        self.cluster_rounds = cluster_rounds
        self.time_limit = time_limit
        self.force_grad_reduce_in_higher_precision = force_grad_reduce_in_higher_precision
        self.constraints: dict[str, Constraint] = {}
        self._constraint_seq = 0
        self.timings: dict[str, float] = {}
        self.solution: Optional[dict[fx.Node, OpSpec]] = None
        self.selected: Optional[dict[fx.Node, int]] = None
        self.objective_value: Optional[float] = None
        self.status: Optional[int] = None
        self.prefetch_discount: dict[tuple[fx.Node, int], float] = {}

        opt.stats.reset()
        self.strats = self._build_strategies()
        self.timings["strategies"] = time.perf_counter() - t0
        t1 = time.perf_counter()
        self.nodes = [n for n in self.graph.nodes if n in self.strats]
        self.node_index = {n: i for i, n in enumerate(self.nodes)}
        self.edges: list[tuple[fx.Node, int, fx.Node]] = []  # (consumer, arg slot, producer)
        for n in self.nodes:
            for slot, p in enumerate(self._inputs(n)):
                self.edges.append((n, slot, p))
        self._node_cost: dict[fx.Node, np.ndarray] = {}
        self._edge_cost: dict[tuple[fx.Node, int], np.ndarray] = {}
        self._build_costs()
        self.timings["costs"] = time.perf_counter() - t1
        self._pairs = self._forward_backward_pairs()
        self._no_redistribute_edges, self._no_reduce_edges = self._mixed_precision_edges()
        logger.info(
            "sharding problem: %d nodes, %d edges, %d node-strategy pairs (%.2fs strategies, %.2fs costs)",
            len(self.nodes),
            len(self.edges),
            sum(len(self.strats[n].strategies) for n in self.nodes),
            self.timings["strategies"],
            self.timings["costs"],
        )

    # ------------------------------------------------------------------ construction
    def _inputs(self, node: fx.Node) -> list[fx.Node]:
        return [i for i in all_input_nodes(node) if i in self.strats]

    def _build_strategies(self) -> dict[fx.Node, OpStrategy]:
        strats: dict[fx.Node, OpStrategy] = {}
        for node in self.graph.nodes:
            val = node.meta.get("val")
            if node.op == "placeholder":
                strats[node] = all_options(self.mesh, val if isinstance(val, torch.Tensor) else None, self.even_only)
            elif node.op == "get_attr":
                if isinstance(val, torch.Tensor):
                    strats[node] = all_options(self.mesh, val, self.even_only)
            elif node.op == "call_function":
                if not _produces_tensor(val):
                    continue  # shape arithmetic: invisible to the solver
                strats[node] = self._options_for(node, strats)
        return strats

    def _options_for(self, node, strats):
        from ..strategies.local_map_rules import is_local_map_node, local_map_options

        if is_local_map_node(node):
            return local_map_options(self.mesh, node, strats)
        from ..strategies.flex_rules import flex_attention_options, is_flex_attention_node

        if is_flex_attention_node(node):
            return flex_attention_options(self.mesh, node, strats)
        return opt.options_for_node(self.mesh, node, strats, self.even_only)

    def _build_costs(self) -> None:
        for n in self.nodes:
            st = self.strats[n].strategies
            if n.op == "call_function" and isinstance(n.target, (torch._ops.OpOverload, torch._ops.HigherOrderOperator)):
                self._node_cost[n] = np.array([compute_cost.strategy_compute_cost(n, s) for s in st], dtype=np.float64)
            else:
                self._node_cost[n] = np.zeros(len(st))
        # Repeated layers produce the same (consumer options, producer options, tensor) triples over and
        # over: the cost matrix of an edge is computed once per distinct triple and shared (read-only).
        memo: dict[tuple, np.ndarray] = {}

        def pl_of(spec):
            return None if spec is None else tuple(spec.placements)

        for n, slot, p in self.edges:
            cs, ps = self.strats[n].strategies, self.strats[p].strategies
            if n.op == "call_function" and n.target is operator.getitem:
                m = np.full((len(cs), len(ps)), INF_COST)
                np.fill_diagonal(m, 0.0)
                self._edge_cost[(n, slot)] = m
                continue
            srcs = []
            for psp in ps:
                src = psp.output_specs
                if isinstance(src, (tuple, list)):
                    # tuple producers are only consumed through getitem (handled above) or by HOPs
                    src = next((x for x in src if x is not None), None)
                srcs.append(src)
            dsts = [csp.input_specs[slot] for csp in cs]
            ref = next((x for x in srcs if x is not None), None)
            tm = None if ref is None or ref.tensor_meta is None else (tuple(ref.tensor_meta.shape), ref.tensor_meta.dtype)
            key = (tuple(pl_of(d) for d in dsts), tuple(pl_of(x) for x in srcs), tm)
            m = memo.get(key)
            if m is None:
                m = np.zeros((len(cs), len(ps)))
                for j, src in enumerate(srcs):
                    for o, dst in enumerate(dsts):
                        if src is None or dst is None:
                            continue
                        c = comm_cost.redistribute_cost(src, dst)
                        if c == math.inf:
                            m[o, j] = INF_COST
                        else:
                            m[o, j] = c + (TRANSITION_EPS if src.placements != dst.placements else 0.0)
                m.setflags(write=False)
                memo[key] = m
            self._edge_cost[(n, slot)] = m

    # ------------------------------------------------------------------ structural constraints
    def _forward_backward_pairs(self) -> list[tuple[fx.Node, fx.Node]]:
        j = self.joint
        pairs = []
        for fqn, p in j.param_nodes.items():
            g = j.param_grads.get(fqn)
            if isinstance(g, fx.Node) and g in self.strats:
                pairs.append((p, g))
        for i, n in enumerate(j.input_nodes):
            g = j.input_grads[i] if i < len(j.input_grads) else None
            if isinstance(n, fx.Node) and isinstance(g, fx.Node) and g in self.strats:
                pairs.append((n, g))
        for fqn, new in j.buffer_updates.items():  # a mutated buffer keeps its placement
            b = j.buffer_nodes.get(fqn)
            if isinstance(b, fx.Node) and isinstance(new, fx.Node) and b in self.strats and new in self.strats:
                pairs.append((b, new))
        for idx, o in enumerate(j.fwd_outputs[: j.num_user_outputs or len(j.fwd_outputs)]):
            t = j.tangent_of(idx)
            if isinstance(o, fx.Node) and t is not None and o in self.strats:
                pairs.append((o, t))
        return pairs

    def _mixed_precision_edges(self):
        """Edges on which nothing may be redistributed / nothing may be reduced.

        * parameter → narrowing ``dtype_cast``: gather *after* the cast (in the narrow dtype);
        * gradient chain up to a widening ``dtype_cast``: keep the partial sum pending until the
          cast, so the reduction runs in the wide dtype (only when the policy asks for it).
        Reference: autoparallel/optimize_sharding.py:1487-1604.
        """
        cast = torch.ops.apb200.dtype_cast.default
        no_redist: set[tuple[fx.Node, int]] = set()
        no_reduce: set[tuple[fx.Node, int]] = set()
        params = set(self.joint.param_nodes.values())
        for n in self.nodes:
            if n.op == "call_function" and n.target is cast:
                src = n.args[0]
                if src in params and n.args[1].itemsize < src.meta["val"].dtype.itemsize:
                    no_redist.add((n, 0))
        if self.force_grad_reduce_in_higher_precision:
            for fqn, g in self.joint.param_grads.items():
                if not isinstance(g, fx.Node):
                    continue
                # walk back from the gradient output through single-input ops to the widening cast
                cur = g
                chain = []
                while cur is not None and cur in self.strats and cur.op == "call_function":
                    ins = self._inputs(cur)
                    if len(ins) != 1:
                        break
                    chain.append(cur)
                    if cur.target is cast and cur.args[1].itemsize > ins[0].meta["val"].dtype.itemsize:
                        # everything from here back to the producing op must keep Partial pending
                        no_reduce.add((cur, 0))
                        back = ins[0]
                        while back in self.strats and back.op == "call_function":
                            bins = self._inputs(back)
                            if len(bins) != 1 or back.target is not torch.ops.aten.alias.default and not _is_layout_op(back):
                                break
                            no_reduce.add((back, 0))
                            back = bins[0]
                        break
                    cur = ins[0]
        return no_redist, no_reduce

    # ------------------------------------------------------------------ user constraints
    def _new_name(self, prefix: str) -> str:
        self._constraint_seq += 1
        return f"{prefix}_{self._constraint_seq}"

    def _strategies_matching(self, node: fx.Node, placement: Sequence[Placement]) -> list[int]:
        placement = tuple(placement)
        out = []
        for i, s in enumerate(self.strats[node].strategies):
            pl = _out_placements(s)
            if pl and isinstance(pl[0], tuple) or (pl and pl[0] is None):
                first = next((x for x in pl if x is not None), None)
                if first == placement:
                    out.append(i)
            elif pl == placement:
                out.append(i)
        return out

    def add_node_constraint(self, node: fx.Node, placement: Optional[Sequence[Placement]] = None, name_prefix="node") -> str:
        """Pin ``node``'s output placement.  Default: ``(Shard(0), Replicate(), ...)``."""
        if placement is None:
            placement = (Shard(0),) + (Replicate(),) * (self.mesh.ndim - 1)
        if len(placement) != self.mesh.ndim:
            raise ValueError(f"placement {placement} has {len(placement)} entries for a {self.mesh.ndim}-d mesh")
        if node not in self.strats:
            raise ValueError(f"{node} is not a tensor node of the traced graph")
        allowed = self._strategies_matching(node, placement)
        if not allowed:
            have = sorted({str(_out_placements(s)) for s in self.strats[node].strategies})
            raise ValueError(f"placement {tuple(placement)} is not available for {node.name}; options: {have}")
        name = self._new_name(f"{name_prefix}:{node.name}")
        self.constraints[name] = Constraint(name, "node", node=node, allowed=allowed, description=str(tuple(placement)))
        return name

    def add_sharded_input_constraint(self, placements: Sequence[Optional[Sequence[Placement]]]) -> list[str]:
        nodes = self.joint.input_nodes
        if len(placements) != len(nodes):
            raise ValueError(f"{len(placements)} input constraints given for {len(nodes)} flat inputs")
        names = []
        for i, (pl, n) in enumerate(zip(placements, nodes)):
            if pl is None:
                continue
            if n is None:
                raise ValueError(f"input {i} has no graph placeholder (non-tensor or aliased input); pass None for it")
            names.append(self.add_node_constraint(n, pl, name_prefix="input"))
        return names

    def add_sharded_output_constraint(self, placements: Sequence[Optional[Sequence[Placement]]]) -> list[str]:
        outs = self.joint.fwd_outputs[: self.joint.num_user_outputs or len(self.joint.fwd_outputs)]
        if len(placements) != len(outs):
            raise ValueError(f"{len(placements)} output constraints given for {len(outs)} flat outputs")
        names = []
        for pl, n in zip(placements, outs):
            if pl is None or not isinstance(n, fx.Node):
                continue
            names.append(self.add_node_constraint(n, pl, name_prefix="output"))
        return names

    def add_parameter_memory_constraint(self, low: float, high: float) -> str:
        name = self._new_name("memory")
        self.constraints[name] = Constraint(name, "memory", low=low, high=high, description=f"[{low}, {high}]")
        return name

    def add_parameter_bytes_constraint(self, budget_bytes: float, bytes_per_element: float = 16.0) -> str:
        """Per-rank bytes of parameter state (locally held elements x ``bytes_per_element``, summed over all
        parameters) must not exceed ``budget_bytes``.  Unlike the ratio form every parameter weighs in with its
        size, so a budget in GB can be stated directly."""
        name = self._new_name("memory_bytes")
        self.constraints[name] = Constraint(name, "memory_bytes", low=bytes_per_element, high=budget_bytes,
                                            description=f"<= {budget_bytes:.4g} B at {bytes_per_element:g} B/element")
        return name

    def remove_constraints(self, names: Sequence[str]) -> None:
        for n in names:
            self.constraints.pop(n, None)

    def apply_prefetch_discount(self, factor: float = 0.0) -> int:
        """Scale the comm cost of parameter all-gathers (edges out of the parameter-derived set
        whose source is sharded and target replicated) – models prefetch hiding them behind
        compute.  Not applied automatically (reference: optimize_sharding.py:824-875)."""
        from ..frontend.graph_canon import param_derived_set

        derived = param_derived_set(self.gm, self.joint.param_nodes.values())
        count = 0
        for n, slot, p in self.edges:
            if p in derived:
                self.prefetch_discount[(n, slot)] = factor
                count += 1
        return count

    # ------------------------------------------------------------------ solve
    def _initial_color(self, salts: dict[fx.Node, Any]):
        def color(n: fx.Node):
            val = n.meta.get("val")
            vfp = opt._fp_strategy(val)
            sfp = opt._fp_strategy(self.strats[n])
            if n.op == "call_function":
                consts = repr(torch.fx.node.map_arg((n.args, n.kwargs), lambda x: None))
                base = ("call", str(n.target), consts)
            else:
                kind = n.meta.get("apb200_kind", (n.op,))[0]
                base = (n.op, kind)
            return (base, vfp, sfp, salts.get(n))

        return color

    def _classes(self) -> dict[fx.Node, int]:
        if not self.repeated_subgraphs:
            return {n: i for i, n in enumerate(self.nodes)}
        salts: dict[fx.Node, Any] = {}
        for c in self.constraints.values():
            if c.kind == "node":
                salts[c.node] = (salts.get(c.node), tuple(c.allowed))
        for a, b in self._pairs:
            pass  # pairs are symmetric across repeats; no salt needed
        for key in list(self._no_redistribute_edges) + list(self._no_reduce_edges):
            salts[key[0]] = (salts.get(key[0]), "mp", key in self._no_reduce_edges)
        for (n, slot), f in self.prefetch_discount.items():
            salts[n] = (salts.get(n), "pf", slot, f)
        # forward / backward and first-gradient-use distinctions come from graph structure itself
        return refine_colors(self.nodes, self._inputs, self._initial_color(salts), self.cluster_rounds)

    def conflicting_constraints(self, max_solves: int = 24) -> dict:
        """Which user constraints clash, found by a deletion filter: starting from all constraints in force, each
        one is left out in turn; if the problem stays infeasible without it, it is not part of the conflict and is
        dropped for good.  What remains is an irreducible set: removing any single member makes the problem
        feasible.  (The reference prints the constraint rows its solver reports as violated,
        autoparallel/optimize_sharding.py:1115-1124; HiGHS returns no such list, so the set is computed.)"""
        saved = dict(self.constraints)
        saved_state = (self.solution, getattr(self, "selected", None), getattr(self, "objective_value", None))

        def feasible(names) -> bool:
            self.constraints = {k: saved[k] for k in names}
            try:
                self.get_solution(diagnose=False)
                return True
            except InfeasibleError:
                return False

        report = {"structural": False, "conflict": [], "exhaustive": True}
        try:
            if not feasible([]):
                report["structural"] = True
                report["text"] = ("infeasible even without user constraints: some node has no admissible strategy under the "
                                  "mesh (for example extents that no mesh dim divides while uneven_sharding is off)")
                return report
            keep = list(saved)
            solves = 0
            for name in list(keep):
                if solves >= max_solves:
                    report["exhaustive"] = False
                    break
                trial = [k for k in keep if k != name]
                solves += 1
                if not feasible(trial):
                    keep = trial  # still infeasible without it: not needed for the conflict
            report["conflict"] = [{"name": k, "kind": saved[k].kind, "node": getattr(saved[k].node, "name", None),
                                   "requires": saved[k].description} for k in keep]
            lines = [f"conflicting constraints ({len(keep)} of {len(saved)}; removing any one of them makes the problem feasible"
                     + ("" if report["exhaustive"] else "; search stopped early") + "):"]
            for c in report["conflict"]:
                where = f" on node {c['node']}" if c["node"] else ""
                lines.append(f"  - {c['name']} [{c['kind']}]{where}: requires {c['requires']}")
            report["text"] = "\n".join(lines)
            return report
        finally:
            self.constraints = saved
            self.solution, sel, obj = saved_state
            if sel is not None:
                self.selected = sel
            if obj is not None:
                self.objective_value = obj

    def get_solution(self, verbose: bool = False, diagnose: bool = True) -> dict[fx.Node, OpSpec]:
        from scipy.optimize import Bounds, LinearConstraint, milp
        from scipy.sparse import coo_matrix

        t0 = time.perf_counter()
        cls = self._classes()
        # representatives and multiplicities
        rep: dict[int, fx.Node] = {}
        mult: dict[int, int] = defaultdict(int)
        for n in self.nodes:
            rep.setdefault(cls[n], n)
            mult[cls[n]] += 1
        # y variable offsets
        y_off: dict[int, int] = {}
        nvar = 0
        for c, n in rep.items():
            y_off[c] = nvar
            nvar += len(self.strats[n].strategies)
        # edge classes
        e_rep: dict[tuple, tuple] = {}
        e_mult: dict[tuple, int] = defaultdict(int)
        for n, slot, p in self.edges:
            k = (cls[p], cls[n], slot)
            e_rep.setdefault(k, (n, slot, p))
            e_mult[k] += 1
        z_off: dict[tuple, int] = {}
        for k, (n, slot, p) in e_rep.items():
            z_off[k] = nvar
            nvar += len(self.strats[n].strategies) * len(self.strats[p].strategies)

        cost = np.zeros(nvar)
        ub = np.ones(nvar)
        for c, n in rep.items():
            k = len(self.strats[n].strategies)
            # sum the member costs (identical by construction, but cheap to be exact)
            cost[y_off[c] : y_off[c] + k] = self._node_cost[n] * mult[c]
        rows, cols, vals = [], [], []
        lo, hi = [], []
        r = 0

        def add_row(idx, coef, lb_, ub_):
            nonlocal r
            rows.extend([r] * len(idx))
            cols.extend(idx)
            vals.extend(coef)
            lo.append(lb_)
            hi.append(ub_)
            r += 1

        for c, n in rep.items():
            k = len(self.strats[n].strategies)
            add_row(list(range(y_off[c], y_off[c] + k)), [1.0] * k, 1.0, 1.0)
        for k_, (n, slot, p) in e_rep.items():
            nc, npd = len(self.strats[n].strategies), len(self.strats[p].strategies)
            m = self._edge_cost[(n, slot)].copy()
            disc = self.prefetch_discount.get((n, slot))
            if disc is not None:
                finite = m < INF_COST
                m[finite] *= disc
            forbid = m >= INF_COST
            if (n, slot) in self._no_redistribute_edges or (n, slot) in self._no_reduce_edges:
                cs, ps = self.strats[n].strategies, self.strats[p].strategies
                for o in range(nc):
                    dst = cs[o].input_specs[slot]
                    for j in range(npd):
                        src = ps[j].output_specs
                        if not isinstance(src, DTensorSpec) or dst is None:
                            continue
                        if (n, slot) in self._no_redistribute_edges:
                            if src.placements != dst.placements:
                                forbid[o, j] = True
                        else:
                            for a, b in zip(src.placements, dst.placements):
                                if isinstance(a, Partial) and not isinstance(b, Partial):
                                    forbid[o, j] = True
            base = z_off[k_]
            flat_cost = np.where(forbid, 0.0, m) * e_mult[k_]
            cost[base : base + nc * npd] = flat_cost.reshape(-1)
            ub[base : base + nc * npd] = np.where(forbid, 0.0, 1.0).reshape(-1)
            yc, yp = y_off[cls[n]], y_off[cls[p]]
            for o in range(nc):
                add_row([base + o * npd + j for j in range(npd)] + [yc + o], [1.0] * npd + [-1.0], 0.0, 0.0)
            for j in range(npd):
                add_row([base + o * npd + j for o in range(nc)] + [yp + j], [1.0] * nc + [-1.0], 0.0, 0.0)

        # forward/backward twins
        for a, b in self._pairs:
            sa, sb = self.strats[a].strategies, self.strats[b].strategies
            pa, pb = defaultdict(list), defaultdict(list)
            for i, s in enumerate(sa):
                pa[_out_placements(s)].append(i)
            for i, s in enumerate(sb):
                pb[_out_placements(s)].append(i)
            ya, yb = y_off[cls[a]], y_off[cls[b]]
            for pl in set(pa) | set(pb):
                ia, ib = pa.get(pl, []), pb.get(pl, [])
                if ia and ib:
                    add_row([ya + i for i in ia] + [yb + i for i in ib], [1.0] * len(ia) + [-1.0] * len(ib), 0.0, 0.0)
                else:
                    for i in ia:
                        ub[ya + i] = 0.0
                    for i in ib:
                        ub[yb + i] = 0.0

        # user constraints
        constrained_params = set()
        for cst in self.constraints.values():
            if cst.kind == "node":
                y0 = y_off[cls[cst.node]]
                k = len(self.strats[cst.node].strategies)
                allowed = set(cst.allowed)
                for i in range(k):
                    if i not in allowed:
                        ub[y0 + i] = 0.0
                if cst.node in self.joint.param_nodes.values():
                    constrained_params.add(cst.node)
        for cst in self.constraints.values():
            if cst.kind != "memory":
                continue
            idx, coef = [], []
            lo_sum = hi_sum = 0.0
            for fqn, p in self.joint.param_nodes.items():
                if p in constrained_params or p not in self.strats:
                    continue
                shape = list(p.meta["val"].shape)
                total = max(1, math.prod(shape))
                ratios = []
                for s in self.strats[p].strategies:
                    ls = local_shape(shape, self.mesh.shape, s.output_spec.placements)
                    ratios.append(math.prod(ls) / total if ls is not None else 1.0)
                best = min(ratios)
                lo_sum += max(best, cst.low)
                hi_sum += max(best, cst.high)
                y0 = y_off[cls[p]]
                for i, rt in enumerate(ratios):
                    idx.append(y0 + i)
                    coef.append(rt)
            if idx:
                # classes may repeat: merge duplicate columns
                merged = defaultdict(float)
                for i, cf in zip(idx, coef):
                    merged[i] += cf
                add_row(list(merged), list(merged.values()), lo_sum - 1e-6, hi_sum + 1e-6)

        for cst in self.constraints.values():
            if cst.kind != "memory_bytes":
                continue
            merged = defaultdict(float)
            fixed = 0.0  # parameters pinned by a node constraint still occupy memory: count their cheapest allowed option
            for fqn, p in self.joint.param_nodes.items():
                if p not in self.strats:
                    continue
                shape = list(p.meta["val"].shape)
                y0 = y_off[cls[p]]
                for i, s_ in enumerate(self.strats[p].strategies):
                    ls = local_shape(shape, self.mesh.shape, s_.output_spec.placements)
                    local_elems = math.prod(ls) if ls is not None else math.prod(shape)
                    # scaled to GB so the row's coefficients stay well conditioned next to the 0/1 rows
                    merged[y0 + i] += local_elems * cst.low / 1e9
            if merged:
                add_row(list(merged), list(merged.values()), -np.inf, cst.high / 1e9 - fixed)

        A = coo_matrix((vals, (rows, cols)), shape=(r, nvar)).tocsr()
        self.timings["build"] = time.perf_counter() - t0
        t1 = time.perf_counter()
        # Only the node choices are integer variables.  An edge variable z[o, j] is pinned by its row sums (= the
        # consumer's choice) and column sums (= the producer's choice): with one-hot node choices exactly one entry
        # is 1, so declaring the edge variables continuous is exact and leaves the branch-and-bound far fewer integers.
        integrality = np.zeros(nvar)
        n_node_vars = min(z_off.values()) if z_off else nvar
        integrality[:n_node_vars] = 1
        options = {"disp": bool(verbose), "presolve": True}
        if self.time_limit is not None:
            options["time_limit"] = float(self.time_limit)
        res = milp(
            c=cost,
            constraints=LinearConstraint(A, np.array(lo), np.array(hi)),
            integrality=integrality,
            bounds=Bounds(np.zeros(nvar), ub),
            options=options,
        )
        self.timings["solve"] = time.perf_counter() - t1
        self.status = res.status
        self.problem_size = {"variables": int(nvar), "constraints": int(r), "node_classes": len(rep), "edge_classes": len(e_rep)}
        logger.info(
            "ILP: %d vars, %d rows, %d node classes (of %d nodes); build %.2fs, solve %.2fs, status %s",
            nvar, r, len(rep), len(self.nodes), self.timings["build"], self.timings["solve"], res.status,
        )
        if res.x is None or res.status not in (0, 1):
            self.solution = None
            msg = ("the sharding optimizer found no feasible placement: "
                   f"{res.message}. User constraints in force: "
                   + "; ".join(f"{c.name}={c.description}" for c in self.constraints.values()))
            if diagnose and self.constraints:
                self.infeasibility_report = self.conflicting_constraints()
                msg += "\n" + self.infeasibility_report["text"]
            raise InfeasibleError(msg)
        x = res.x
        self.objective_value = float(res.fun)
        selected: dict[fx.Node, int] = {}
        for n in self.nodes:
            y0 = y_off[cls[n]]
            k = len(self.strats[n].strategies)
            selected[n] = int(np.argmax(x[y0 : y0 + k]))
        self.selected = selected
        self.solution = {n: self.strats[n].strategies[i] for n, i in selected.items()}
        self._validate()
        return self.solution

    def resolve(self, verbose: bool = False):
        return self.get_solution(verbose)

    def _validate(self) -> None:
        for n, slot, p in self.edges:
            c = self._edge_cost[(n, slot)][self.selected[n], self.selected[p]]
            if c >= INF_COST:
                raise RuntimeError(f"solver picked an impossible redistribution on {p.name} -> {n.name}[{slot}]")

    # ------------------------------------------------------------------ introspection
    def total_cost_breakdown(self) -> dict[str, float]:
        assert self.selected is not None
        comp = sum(float(self._node_cost[n][self.selected[n]]) for n in self.nodes)
        comm = 0.0
        for n, slot, p in self.edges:
            comm += float(self._edge_cost[(n, slot)][self.selected[n], self.selected[p]])
        return {"compute_us": comp, "comm_us": comm, "total_us": comp + comm}

    def edge_cost(self, node: fx.Node, slot: int) -> float:
        p = self._inputs(node)[slot]
        return float(self._edge_cost[(node, slot)][self.selected[node], self.selected[p]])

    def print_costs_for_node(self, node: fx.Node, file=None) -> str:
        lines = [f"costs for {node.name} ({node.target if node.op == 'call_function' else node.op})"]
        ins = self._inputs(node)
        for i, s in enumerate(self.strats[node].strategies):
            mark = "*" if self.selected is not None and self.selected.get(node) == i else " "
            lines.append(f" {mark}[{i}] out={_fmt_pl(_out_placements(s))} compute={self._node_cost[node][i]:.2f}us")
            for slot, p in enumerate(ins):
                row = self._edge_cost[(node, slot)][i]
                best = int(np.argmin(row))
                lines.append(
                    f"      arg{slot} needs {_fmt_pl(s.input_specs[slot].placements)}; cheapest from {p.name}"
                    f"[{best}]={_fmt_pl(_out_placements(self.strats[p].strategies[best]))} at {row[best]:.2f}us"
                )
        text = "\n".join(lines)
        print(text, file=file)
        return text

    def explain_placement(self, node: fx.Node) -> str:
        """Why ``node`` got its placement: chosen strategy vs. the alternatives, with the cost each
        alternative would incur locally (compute + redistribution from the chosen producers and to
        the chosen consumers)."""
        assert self.selected is not None, "solve first"
        ins = self._inputs(node)
        users = [(u, slot) for u in node.users if u in self.strats for slot, p in enumerate(self._inputs(u)) if p is node]
        lines = [f"placement of {node.name}:"]
        for i, s in enumerate(self.strats[node].strategies):
            local = float(self._node_cost[node][i])
            for slot, p in enumerate(ins):
                local += float(self._edge_cost[(node, slot)][i, self.selected[p]])
            for u, slot in users:
                local += float(self._edge_cost[(u, slot)][self.selected[u], i])
            mark = "=> " if self.selected[node] == i else "   "
            c = "inf" if local >= INF_COST else f"{local:.2f}us"
            lines.append(f"{mark}{_fmt_pl(_out_placements(s))}: local cost {c}")
        return "\n".join(lines)

    def diff_solutions(self, other: dict[fx.Node, OpSpec]) -> list[tuple[str, str, str]]:
        assert self.solution is not None
        out = []
        for n in self.nodes:
            a, b = self.solution.get(n), other.get(n)
            if a is None or b is None:
                continue
            pa, pb = _out_placements(a), _out_placements(b)
            if pa != pb:
                out.append((n.name, _fmt_pl(pa), _fmt_pl(pb)))
        return out

    def placement_of(self, node: fx.Node):
        return _out_placements(self.solution[node])

    def get_log(self, verbose: bool = False, colored: bool = False) -> str:
        from ...utils.log_format import format_sharding_log

        return format_sharding_log(self, verbose=verbose, colored=colored)

    def get_json(self) -> dict:
        from ...utils.export_json import export_sharding_json

        return export_sharding_json(self)

    def save(self, path: str) -> None:
        from ...utils.serialize import save_optimizer

        save_optimizer(self, path)

    @staticmethod
    def load(path: str) -> "LoadedOptimizer":  # noqa: F821
        from ...utils.serialize import load_optimizer

        return load_optimizer(path)

    def save_placements(self, path: str) -> None:
        from ...utils.serialize import save_placements

        save_placements(self, path)

    def load_placements(self, path: str) -> dict[fx.Node, OpSpec]:
        from ...utils.serialize import load_placements

        return load_placements(self, path)


def _is_layout_op(n: fx.Node) -> bool:
    aten = torch.ops.aten
    return n.target in (
        aten.view.default, aten._unsafe_view.default, aten.reshape.default, aten.permute.default, aten.t.default,
        aten.transpose.int, aten.alias.default,
    )


def _fmt_pl(pl) -> str:
    if pl is None:
        return "None"
    if len(pl) and (isinstance(pl[0], tuple) or pl[0] is None):
        return "(" + ", ".join(_fmt_pl(x) for x in pl) + ")"

    def one(p):
        if isinstance(p, Shard):
            return f"S({p.dim})"
        if isinstance(p, Replicate):
            return "R"
        if isinstance(p, Partial):
            return "P" if p.reduce_op == "sum" else f"P({p.reduce_op})"
        return str(p)

    return "".join(one(p) for p in pl) if len(pl) == 1 else "(" + ",".join(one(p) for p in pl) + ")"
