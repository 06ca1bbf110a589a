"""Save and reload a lowered per-rank graph for offline replay.

A capture is one JSON file: the forward and backward graphs of one rank after lowering and
partitioning (every node with its target by qualified name, arguments, and the shape / dtype of its
value), the mesh shape and, for every process-group name that occurs in a collective, the mesh dim it
stood for.  Group names are only meaningful inside the job that made them, so a replay never
resolves them: the simulator prices a collective through that recorded mapping.

``load_colls_table`` reads the measured collective tables of the reference's overlap simulator
(``autoparallel/tools/overlap_simulator/colls16_8.table`` and friends: one row per (mesh dim, group
size, collective), one column per message size in MB, values in ms) into this framework's table
format, so a capture can be replayed against either project's measurements.

Reference counterpart: autoparallel/tools/overlap_simulator/run.py:99-233 (graph replay with the
capture's group names), :236-373 (table loading).
"""
from __future__ import annotations

import json
import operator
import re
from typing import Optional

import torch
import torch.fx as fx

_DTYPES = {str(d): d for d in (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.int16,
                               torch.int8, torch.uint8, torch.bool, torch.complex64)}


def _enc_val(v):
    if isinstance(v, torch.Tensor):
        return {"shape": list(v.shape), "dtype": str(v.dtype)}
    if isinstance(v, (tuple, list)):
        return [_enc_val(x) for x in v]
    return None


def _dec_val(v):
    if isinstance(v, dict):
        return torch.empty(v["shape"], dtype=_DTYPES[v["dtype"]], device="meta")
    if isinstance(v, list):
        return tuple(_dec_val(x) for x in v)
    return None


def _enc_arg(a):
    if isinstance(a, fx.Node):
        return {"node": a.name}
    if isinstance(a, (tuple, list)):
        return {"seq": [_enc_arg(x) for x in a], "tuple": isinstance(a, tuple)}
    if isinstance(a, torch.dtype):
        return {"dtype": str(a)}
    if isinstance(a, slice):
        return {"slice": [a.start, a.stop, a.step]}
    if isinstance(a, (torch.device, torch.layout, torch.memory_format)):
        return {"repr": str(a)}
    if a is None or isinstance(a, (bool, int, float, str)):
        return a
    return {"repr": repr(a)}


def _dec_arg(a, env):
    if isinstance(a, dict):
        if "node" in a:
            return env[a["node"]]
        if "seq" in a:
            seq = [_dec_arg(x, env) for x in a["seq"]]
            return tuple(seq) if a["tuple"] else seq
        if "dtype" in a:
            return _DTYPES[a["dtype"]]
        if "slice" in a:
            return slice(*a["slice"])
        return a.get("repr")
    return a


def _target_name(t) -> str:
    if t is operator.getitem:
        return "operator.getitem"
    if isinstance(t, torch._ops.OpOverload):
        return f"torch.ops.{t.namespace}.{t._opname}.{t._overloadname}"
    return getattr(t, "__module__", "?") + "." + getattr(t, "__qualname__", repr(t))


def _resolve_target(name: str):
    if name == "operator.getitem":
        return operator.getitem
    if name.startswith("torch.ops."):
        _, _, ns, op, overload = name.split(".", 4)
        return getattr(getattr(getattr(torch.ops, ns), op), overload)
    mod, _, attr = name.rpartition(".")
    import importlib

    return getattr(importlib.import_module(mod), attr)


def graph_to_dict(gm: fx.GraphModule) -> list:
    out = []
    for n in gm.graph.nodes:
        out.append({"name": n.name, "op": n.op, "target": _target_name(n.target) if n.op == "call_function" else str(n.target),
                    "args": [_enc_arg(a) for a in n.args], "kwargs": {k: _enc_arg(v) for k, v in n.kwargs.items()},
                    "val": _enc_val(n.meta.get("val"))})
    return out


def graph_from_dict(nodes: list) -> fx.GraphModule:
    import autoparallel_b200  # noqa: F401  (registers the operator libraries the targets live in)

    g = fx.Graph()
    env: dict = {}
    for d in nodes:
        if d["op"] == "placeholder":
            n = g.placeholder(d["name"])
        elif d["op"] == "output":
            n = g.output(_dec_arg(d["args"][0], env))
        elif d["op"] == "call_function":
            n = g.call_function(_resolve_target(d["target"]), tuple(_dec_arg(a, env) for a in d["args"]),
                                {k: _dec_arg(v, env) for k, v in d["kwargs"].items()})
        elif d["op"] == "get_attr":
            n = g.placeholder(d["name"])  # constants of the capture become inputs of the replayed graph
        else:
            raise ValueError(f"cannot replay a {d['op']} node ({d['name']})")
        n.meta["val"] = _dec_val(d["val"])
        env[d["name"]] = n
    return fx.GraphModule(torch.nn.Module(), g)


def save_capture(path: str, forward: fx.GraphModule, backward: Optional[fx.GraphModule], mesh, extra: Optional[dict] = None) -> None:
    group_dim = {mesh.get_group(i).group_name: i for i in range(mesh.ndim)}
    doc = {"format": "autoparallel_b200.capture/1", "mesh_shape": list(mesh.shape), "mesh_dim_names": list(mesh.mesh_dim_names or ()),
           "group_dim": group_dim, "forward": graph_to_dict(forward), "backward": graph_to_dict(backward) if backward is not None else None,
           "extra": extra or {}}
    with open(path, "w") as f:
        json.dump(doc, f)


def load_capture(path: str) -> dict:
    with open(path) as f:
        doc = json.load(f)
    if doc.get("format") != "autoparallel_b200.capture/1":
        raise ValueError(f"{path} is not a graph capture of this framework")
    doc["forward_gm"] = graph_from_dict(doc["forward"])
    doc["backward_gm"] = graph_from_dict(doc["backward"]) if doc.get("backward") else None
    return doc


# ------------------------------------------------------------------------------------------ measured tables
_KIND = {"all_gather_into_tensor": "all_gather", "all_gather_into_tensor_out": None, "reduce_scatter_tensor": "reduce_scatter",
         "all_reduce": "all_reduce", "all_to_all_single": "all_to_all", "all_to_all": "all_to_all"}


def load_colls_table(path: str) -> dict:
    """``{(kind, group size): [(bytes, microseconds), ...]}`` from a text table with the columns ``Group``, ``Group
    Size``, ``Collective`` and one ``<N>MB (ms)`` column per message size (N = per-rank input size in MB).  The byte
    counts follow this framework's convention: the size of the full (gathered / pre-scatter) tensor."""
    with open(path) as f:
        lines = [l.rstrip("\n") for l in f if l.strip()]
    header = re.split(r"\s{2,}", lines[0].strip())
    sizes_mb = [float(re.match(r"([\d.]+)\s*MB", h).group(1)) for h in header[3:]]
    tables: dict = {}
    for line in lines[1:]:
        if set(line.strip()) <= {"-", " "}:
            continue
        cells = line.split()
        if len(cells) < 3 + len(sizes_mb):
            continue
        n, coll = int(cells[1]), cells[2]
        kind = _KIND.get(coll)
        if kind is None:
            continue
        pts = []
        for mb, ms in zip(sizes_mb, cells[3:3 + len(sizes_mb)]):
            per_rank = mb * 2**20
            # all-gather rows are labelled by the per-rank input; the full tensor is n times that.  The other
            # collectives are labelled by their (full) input already.
            full = per_rank * n if kind == "all_gather" else per_rank
            pts.append((full, float(ms) * 1e3))
        tables[(kind, n)] = sorted(pts)
    return tables
