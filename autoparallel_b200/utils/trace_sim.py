"""Simulated execution of a (lowered) graph from the cost models: timeline, metrics, traces.

``estimate_graph_metrics`` walks the graph in order with two clocks – a compute stream and one
communication stream per process group – advancing compute nodes by their estimated kernel time and
collective nodes by the comm model; a ``comm_wait`` (or a synchronous collective) joins the streams.
It returns total / compute / communication / exposed-communication time and the peak of live
tensor bytes.  ``create_execution_trace`` emits the same timeline as Chrome/Perfetto trace events.
Reference: autoparallel/graph_passes/estimate_graph_metrics.py:21-89 and
autoparallel/graph_passes/debug_helpers.py:27-91, 324-399.
"""
from __future__ import annotations

import dataclasses
import json
from typing import Callable, Optional

import torch
import torch.fx as fx

from ..parallel.cost import comm as comm_cost
from ..parallel.cost.device import get_device_limit
from ..runtime import comm_ops

LAUNCH_US = 1.0


@dataclasses.dataclass
class GraphMetrics:
    total_us: float
    compute_us: float
    comm_us: float
    exposed_comm_us: float
    peak_bytes: int
    num_collectives: int


def _nbytes(v) -> int:
    if isinstance(v, torch.Tensor):
        return v.numel() * v.element_size()
    if isinstance(v, (tuple, list)):
        return sum(_nbytes(x) for x in v)
    return 0


def make_runtime_estimator(mesh, plan_device: Optional[str] = None, group_dim: Optional[dict] = None,
                           topology=None) -> Callable[[fx.Node], float]:
    """node -> microseconds.  Collectives are priced by the active topology through their group
    name (resolved to a mesh dim), everything else by FLOPs / bytes on local shapes.
    ``group_dim`` / ``topology``: replaying a saved graph needs no live mesh - the capture records which mesh dim
    each group name stood for, and the topology (formula or measured table) is passed in."""
    from ..parallel.cost.device import DEVICE_LIMITS

    limit = DEVICE_LIMITS[plan_device] if plan_device else get_device_limit(mesh.device_type if mesh is not None else "cuda")
    topo = topology if topology is not None else comm_cost.get_topology(mesh)
    if group_dim is None:
        group_dim = {mesh.get_group(i).group_name: i for i in range(mesh.ndim)}
    C = comm_ops.ops

    def flops_of(node):
        t = node.target
        apb = torch.ops.apb200
        ins = [a.meta.get("val") for a in node.all_input_nodes]
        out = node.meta.get("val")
        if t in (apb.mm_nd.default, C.ag_mm.default, C.mm_rs.default) or t is apb.mm_wgrad.default or t is torch.ops.aten.mm.default:
            a, b = ins[0], ins[1]
            if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
                o = out[0] if isinstance(out, (tuple, list)) else out
                if t is apb.mm_wgrad.default or (t is C.mm_rs.default and node.args[2] == 2):
                    return 2.0 * a.numel() * b.shape[-1]
                n_ranks = node.args[-1] if t in (C.ag_mm.default, C.mm_rs.default) else 1
                k = a.shape[-1]
                return 2.0 * o.numel() * k * (n_ranks if t is C.mm_rs.default else 1)
        if t is apb.attention.default:
            q = ins[0]
            return 2.0 * q.shape[0] * q.shape[2] * q.shape[1] ** 2 * q.shape[3]
        if t is apb.attention_bwd.default:
            q = ins[1]
            return 5.0 * q.shape[0] * q.shape[2] * q.shape[1] ** 2 * q.shape[3]
        return 0.0

    def estimate(node: fx.Node) -> float:
        if node.op != "call_function":
            return 0.0
        t = node.target
        val = node.meta.get("val")
        if t in comm_ops.COLLECTIVE_OPS or t in comm_ops.START_OPS:
            g = node.args[-2]
            n = node.args[-1]
            dim = group_dim.get(g, 0)
            nb = _nbytes(val)
            if t in (C.all_gather.default, C.all_gather_start.default):
                return topo.all_gather(dim, n, nb)
            if t in (C.reduce_scatter.default, C.reduce_scatter_start.default):
                return topo.reduce_scatter(dim, n, nb * n)
            if t in (C.all_reduce.default, C.all_reduce_start.default, C.all_reduce_op.default):
                return topo.all_reduce(dim, n, nb)
            return topo.all_to_all(dim, n, nb)
        if t is C.comm_wait.default or not isinstance(t, torch._ops.OpOverload):
            return 0.0
        if t in (torch.ops.aten.view.default, torch.ops.aten.permute.default, torch.ops.aten.t.default, torch.ops.aten.alias.default,
                 torch.ops.aten.slice.Tensor, torch.ops.aten.expand.default, torch.ops.aten.unsqueeze.default, torch.ops.aten._unsafe_view.default,
                 torch.ops.aten.reshape.default):
            return 0.0
        nb = _nbytes(val) + sum(_nbytes(a.meta.get("val")) for a in node.all_input_nodes)
        dt = torch.bfloat16
        v0 = val[0] if isinstance(val, (tuple, list)) and val else val
        if isinstance(v0, torch.Tensor) and v0.dtype.is_floating_point:
            dt = v0.dtype
        fl = flops_of(node)
        if fl > 0:
            # a contraction runs at the rate of its operands (bf16 weight gradients accumulate into fp32 outputs)
            a0 = next((a.meta.get("val") for a in node.all_input_nodes if isinstance(a.meta.get("val"), torch.Tensor)
                       and a.meta["val"].dtype.is_floating_point), None)
            if a0 is not None:
                dt = a0.dtype
        t_us = max(fl / limit.flops_per_us(dt), nb / limit.bytes_per_us(), limit.launch_us)
        if t in comm_ops.FUSED_OPS:
            g, n = node.args[-2], node.args[-1]
            dim = group_dim.get(g, 0)
            moved = _nbytes(val[1]) if t is C.ag_mm.default else _nbytes(val) * n
            link = (topo.all_gather if t is C.ag_mm.default else topo.reduce_scatter)(dim, n, moved)
            t_us = max(t_us, link)  # fused: transfer hides under the tiles (roofline = the slower of the two)
        return t_us

    return estimate


def simulate(gm: fx.GraphModule, estimate: Callable[[fx.Node], float], events: Optional[list] = None) -> GraphMetrics:
    C = comm_ops.ops
    t_compute = 0.0
    stream_free: dict[str, float] = {}
    ready_at: dict[fx.Node, float] = {}
    compute_us = comm_us = exposed = 0.0
    n_coll = 0
    live: dict[fx.Node, int] = {}
    remaining = {n: len(n.users) for n in gm.graph.nodes}
    cur_bytes = peak = 0
    for node in gm.graph.nodes:
        if node.op == "placeholder":
            continue
        dur = estimate(node) if node.op == "call_function" else 0.0
        t = node.target if node.op == "call_function" else None
        if t in comm_ops.START_OPS:
            g = node.args[-2]
            start = max(t_compute, stream_free.get(g, 0.0))
            stream_free[g] = start + dur
            ready_at[node] = start + dur
            comm_us += dur
            n_coll += 1
            t_compute += LAUNCH_US
            if events is not None:
                events.append({"name": str(t).split(".")[-2], "ph": "X", "ts": start, "dur": dur, "pid": 0, "tid": f"group-{g}"})
        elif t is C.comm_wait.default:
            r = ready_at.get(node.args[0], t_compute)
            if r > t_compute:
                exposed += r - t_compute
                t_compute = r
        elif t in comm_ops.COLLECTIVE_OPS:
            g = node.args[-2]
            start = max(t_compute, stream_free.get(g, 0.0))
            stream_free[g] = start + dur
            exposed += start + dur - t_compute
            comm_us += dur
            n_coll += 1
            if events is not None:
                events.append({"name": str(t).split(".")[-2], "ph": "X", "ts": start, "dur": dur, "pid": 0, "tid": f"group-{g}"})
            t_compute = start + dur
        else:
            if dur > 0 and events is not None:
                events.append({"name": node.name, "ph": "X", "ts": t_compute, "dur": dur, "pid": 0, "tid": 0})
            compute_us += dur
            t_compute += dur + (LAUNCH_US if dur > 0 else 0.0)
        # liveness
        if node.op == "call_function":
            b = _nbytes(node.meta.get("val"))
            live[node] = b
            cur_bytes += b
            peak = max(peak, cur_bytes)
            for i in set(node.all_input_nodes):
                remaining[i] -= 1
                if remaining[i] == 0 and i in live:
                    cur_bytes -= live.pop(i)
    total = max([t_compute] + list(stream_free.values()))
    return GraphMetrics(total, compute_us, comm_us, exposed, peak, n_coll)


def estimate_graph_metrics(gm: fx.GraphModule, mesh, plan_device: Optional[str] = None, estimator=None) -> GraphMetrics:
    if estimator is not None:
        return simulate(gm, estimator)
    return _estimate_graph_metrics(gm, mesh, plan_device)


def _estimate_graph_metrics(gm: fx.GraphModule, mesh, plan_device: Optional[str] = None) -> GraphMetrics:
    return simulate(gm, make_runtime_estimator(mesh, plan_device))


def create_execution_trace(gm: fx.GraphModule, mesh, path: Optional[str] = None, plan_device: Optional[str] = None) -> dict:
    events: list = []
    metrics = simulate(gm, make_runtime_estimator(mesh, plan_device), events)
    trace = {"traceEvents": events, "displayTimeUnit": "ms", "metadata": dataclasses.asdict(metrics)}
    if path:
        with open(path, "w") as f:
            json.dump(trace, f)
    return trace
