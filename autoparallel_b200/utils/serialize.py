"""Saving and reloading planner state.

* ``save_optimizer`` / ``load_optimizer`` – everything needed to inspect or re-solve a plan without
  the model, a process group or a GPU: node table (names, ops, shapes), candidate placements, cost
  arrays, edges, forward/backward twins, constraints, and the selected strategy per node.  The
  loaded object answers ``get_solution`` / ``resolve`` / ``placement_of`` / ``get_json``-style
  queries on that frozen problem.
* ``save_placements`` / ``load_placements`` – a small JSON file (node name → placement string),
  validated against the mesh shape and the node names of the optimizer it is loaded into.

Reference: autoparallel/serialization.py:104-475 (torch.save dict "version 1"; JSON placements).
"""
from __future__ import annotations

import json
import time
from typing import Optional

import numpy as np
import torch

FORMAT_VERSION = 1


def _pl_to_str(pl) -> str:
    from ..parallel.solver.ilp import _fmt_pl

    return _fmt_pl(pl)


def _parse_placement(s: str):
    """Inverse of the compact placement format for single-output nodes: ``S(0)``, ``R``, ``P`` or
    ``(S(0),R)`` for multi-dim meshes."""
    from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

    s = s.strip()
    items = []
    body = s[1:-1] if s.startswith("(") and s.endswith(")") and not s.startswith("(S(") or s.count(",") else s
    if s.startswith("(") and s.endswith(")"):
        body = s[1:-1]
    depth, cur = 0, ""
    for ch in body:
        if ch == "(":
            depth += 1
        if ch == ")":
            depth -= 1
        if ch == "," and depth == 0:
            items.append(cur)
            cur = ""
        else:
            cur += ch
    if cur:
        items.append(cur)
    out = []
    for it in items:
        it = it.strip()
        if it == "R":
            out.append(Replicate())
        elif it == "P":
            out.append(Partial())
        elif it.startswith("P(") and it.endswith(")"):
            out.append(Partial(it[2:-1]))
        elif it.startswith("S(") and it.endswith(")"):
            out.append(Shard(int(it[2:-1])))
        else:
            raise ValueError(f"cannot parse placement {it!r} in {s!r}")
    return tuple(out)


def save_optimizer(optimizer, path: str) -> None:
    from ..parallel.solver.ilp import _out_placements

    t0 = time.perf_counter()
    names = [n.name for n in optimizer.nodes]
    idx = {n: i for i, n in enumerate(optimizer.nodes)}
    node_rows = []
    for n in optimizer.nodes:
        v = n.meta.get("val")
        node_rows.append({
            "name": n.name,
            "op": n.op,
            "target": str(n.target),
            "shape": list(v.shape) if isinstance(v, torch.Tensor) else None,
            "dtype": str(v.dtype) if isinstance(v, torch.Tensor) else None,
            "placements": [_pl_to_str(_out_placements(s)) for s in optimizer.strats[n].strategies],
            "kind": list(n.meta.get("apb200_kind", ())) or None,
        })
    state = {
        "version": FORMAT_VERSION,
        "mesh_shape": list(optimizer.mesh.shape),
        "mesh_dim_names": list(optimizer.mesh.mesh_dim_names or []),
        "nodes": node_rows,
        "node_cost": [np.asarray(optimizer._node_cost[n]) for n in optimizer.nodes],
        "edges": [(idx[c], slot, idx[p]) for c, slot, p in optimizer.edges],
        "edge_cost": [np.asarray(optimizer._edge_cost[(c, slot)]) for c, slot, p in optimizer.edges],
        "pairs": [(idx[a], idx[b]) for a, b in optimizer._pairs],
        "param_ratios": _param_ratios(optimizer, idx),
        "classes": [optimizer._classes()[n] for n in optimizer.nodes] if optimizer.repeated_subgraphs else None,
        "constraints": [
            {"name": c.name, "kind": c.kind, "node": idx.get(c.node) if c.node is not None else None, "allowed": c.allowed,
             "low": c.low, "high": c.high, "description": c.description}
            for c in optimizer.constraints.values()
        ],
        "selected": [optimizer.selected[n] for n in optimizer.nodes] if optimizer.selected is not None else None,
        "objective": optimizer.objective_value,
        "graph_code": optimizer.gm.code,
        "saved_at": time.time(),
    }
    torch.save(state, path)
    optimizer.timings["save"] = time.perf_counter() - t0


def _param_ratios(optimizer, idx) -> list:
    """(node index, [local/global element ratio per candidate placement]) for every parameter."""
    import math

    from ..parallel.strategies.dtensor_adapter import local_shape

    out = []
    for p in optimizer.joint.param_nodes.values():
        if p not in idx:
            continue
        shape = list(p.meta["val"].shape)
        total = max(1, math.prod(shape))
        ratios = []
        for s in optimizer.strats[p].strategies:
            ls = local_shape(shape, optimizer.mesh.shape, s.output_spec.placements)
            ratios.append(math.prod(ls) / total if ls is not None else 1.0)
        out.append((idx[p], ratios))
    return out


class LoadedOptimizer:
    """A frozen sharding problem reloaded from disk (no model, mesh object or process group)."""

    def __init__(self, state: dict):
        if state.get("version") != FORMAT_VERSION:
            raise ValueError(f"unsupported optimizer file version {state.get('version')}")
        self.state = state
        self.names = [r["name"] for r in state["nodes"]]
        self.selected = list(state["selected"]) if state["selected"] is not None else None
        self.objective_value = state["objective"]
        self.mesh_shape = tuple(state["mesh_shape"])

    def placement_of(self, name: str) -> str:
        i = self.names.index(name)
        return self.state["nodes"][i]["placements"][self.selected[i]]

    def get_solution(self) -> dict[str, str]:
        return {r["name"]: r["placements"][s] for r, s in zip(self.state["nodes"], self.selected)}

    def total_cost(self, selected: Optional[list] = None) -> float:
        sel = selected or self.selected
        tot = sum(float(c[sel[i]]) for i, c in enumerate(self.state["node_cost"]))
        for (c, slot, p), m in zip(self.state["edges"], self.state["edge_cost"]):
            tot += float(m[sel[c], sel[p]])
        return tot

    def resolve(self, extra_fixed: Optional[dict[str, str]] = None) -> dict[str, str]:
        """Re-solve the frozen problem (optionally pinning nodes by name to a placement string)."""
        from scipy.optimize import Bounds, LinearConstraint, milp
        from scipy.sparse import coo_matrix

        st = self.state
        n_nodes = len(st["nodes"])
        y_off, nvar = [], 0
        for c in st["node_cost"]:
            y_off.append(nvar)
            nvar += len(c)
        z_off = []
        for m in st["edge_cost"]:
            z_off.append(nvar)
            nvar += m.size
        cost = np.zeros(nvar)
        ub = np.ones(nvar)
        rows, cols, vals, lo, hi = [], [], [], [], []
        r = 0
        for i, c in enumerate(st["node_cost"]):
            cost[y_off[i] : y_off[i] + len(c)] = c
            rows += [r] * len(c)
            cols += list(range(y_off[i], y_off[i] + len(c)))
            vals += [1.0] * len(c)
            lo.append(1.0)
            hi.append(1.0)
            r += 1
        for (c, slot, p), m, z0 in zip(st["edges"], st["edge_cost"], z_off):
            nc, npd = m.shape
            bad = m >= 1e11
            cost[z0 : z0 + m.size] = np.where(bad, 0.0, m).reshape(-1)
            ub[z0 : z0 + m.size] = np.where(bad, 0.0, 1.0).reshape(-1)
            for o in range(nc):
                rows += [r] * (npd + 1)
                cols += [z0 + o * npd + j for j in range(npd)] + [y_off[c] + o]
                vals += [1.0] * npd + [-1.0]
                lo.append(0.0)
                hi.append(0.0)
                r += 1
            for j in range(npd):
                rows += [r] * (nc + 1)
                cols += [z0 + o * npd + j for o in range(nc)] + [y_off[p] + j]
                vals += [1.0] * nc + [-1.0]
                lo.append(0.0)
                hi.append(0.0)
                r += 1
        # forward/backward twins share a placement
        for a, b in st.get("pairs", []):
            pa, pb = st["nodes"][a]["placements"], st["nodes"][b]["placements"]
            for pl in set(pa) | set(pb):
                ia = [k for k, x in enumerate(pa) if x == pl]
                ib = [k for k, x in enumerate(pb) if x == pl]
                if ia and ib:
                    rows += [r] * (len(ia) + len(ib))
                    cols += [y_off[a] + k for k in ia] + [y_off[b] + k for k in ib]
                    vals += [1.0] * len(ia) + [-1.0] * len(ib)
                    lo.append(0.0)
                    hi.append(0.0)
                    r += 1
                else:
                    for k in ia:
                        ub[y_off[a] + k] = 0.0
                    for k in ib:
                        ub[y_off[b] + k] = 0.0
        # parameters pinned by the user (saved constraints or ``extra_fixed``) do not count towards the memory band
        pinned = {c["node"] for c in st["constraints"] if c["kind"] == "node"} | {self.names.index(n) for n in (extra_fixed or {})}
        for cst in st["constraints"]:
            if cst["kind"] != "memory":
                continue
            lo_sum = hi_sum = 0.0
            first = True
            for i, ratios in st.get("param_ratios", []):
                if i in pinned:
                    continue
                best = min(ratios)
                lo_sum += max(best, cst["low"])
                hi_sum += max(best, cst["high"])
                rows += [r] * len(ratios)
                cols += [y_off[i] + k for k in range(len(ratios))]
                vals += list(ratios)
                first = False
            if not first:
                lo.append(lo_sum - 1e-6)
                hi.append(hi_sum + 1e-6)
                r += 1
        for cst in st["constraints"]:
            if cst["kind"] == "node" and cst["node"] is not None:
                allowed = set(cst["allowed"])
                i = cst["node"]
                for k in range(len(st["node_cost"][i])):
                    if k not in allowed:
                        ub[y_off[i] + k] = 0.0
        for name, pl in (extra_fixed or {}).items():
            i = self.names.index(name)
            opts = st["nodes"][i]["placements"]
            if pl not in opts:
                raise ValueError(f"{name} has no placement {pl}; options {opts}")
            for k, o in enumerate(opts):
                if o != pl:
                    ub[y_off[i] + k] = 0.0
        A = coo_matrix((vals, (rows, cols)), shape=(r, nvar)).tocsr()
        res = milp(c=cost, constraints=LinearConstraint(A, np.array(lo), np.array(hi)), integrality=np.ones(nvar),
                   bounds=Bounds(np.zeros(nvar), ub))
        if res.x is None:
            raise RuntimeError(f"reloaded problem is infeasible: {res.message}")
        self.selected = [int(np.argmax(res.x[y_off[i] : y_off[i] + len(st["node_cost"][i])])) for i in range(n_nodes)]
        self.objective_value = float(res.fun)
        return self.get_solution()


def load_optimizer(path: str) -> LoadedOptimizer:
    return LoadedOptimizer(torch.load(path, weights_only=False))


def save_placements(optimizer, path: str) -> None:
    from ..parallel.solver.ilp import _out_placements

    if optimizer.selected is None:
        raise RuntimeError("nothing to save: solve first")
    data = {
        "version": FORMAT_VERSION,
        "mesh_shape": list(optimizer.mesh.shape),
        "mesh_dim_names": list(optimizer.mesh.mesh_dim_names or []),
        "placements": {n.name: optimizer.selected[n] for n in optimizer.nodes},
        "readable": {n.name: _pl_to_str(_out_placements(optimizer.solution[n])) for n in optimizer.nodes},
    }
    with open(path, "w") as f:
        json.dump(data, f)


def load_placements(optimizer, path: str) -> dict:
    """Apply a saved solution to ``optimizer`` (same graph, same mesh) without solving."""
    from ..parallel.solver.ilp import _out_placements

    with open(path) as f:
        data = json.load(f)
    if data.get("version") != FORMAT_VERSION:
        raise ValueError(f"unsupported placements file version {data.get('version')}")
    if list(optimizer.mesh.shape) != data["mesh_shape"]:
        raise ValueError(f"placements were saved for mesh {data['mesh_shape']}, this optimizer uses {list(optimizer.mesh.shape)}")
    by_name = {n.name: n for n in optimizer.nodes}
    missing = set(by_name) - set(data["placements"])
    extra = set(data["placements"]) - set(by_name)
    if missing or extra:
        raise ValueError(f"placements file does not match the graph: missing {sorted(missing)[:5]}, unknown {sorted(extra)[:5]}")
    selected = {}
    for name, idx in data["placements"].items():
        node = by_name[name]
        strategies = optimizer.strats[node].strategies
        if idx >= len(strategies) or _pl_to_str(_out_placements(strategies[idx])) != data["readable"][name]:
            raise ValueError(f"placement of {name} in the file ({data['readable'][name]}) is not option {idx} of this graph")
        selected[node] = idx
    optimizer.selected = selected
    optimizer.solution = {n: optimizer.strats[n].strategies[i] for n, i in selected.items()}
    optimizer._validate()
    return optimizer.solution
