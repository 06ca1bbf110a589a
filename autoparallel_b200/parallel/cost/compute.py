"""Compute-time estimate of one node under one sharding strategy (microseconds).

``time = max(FLOPs / tensor throughput, bytes moved / HBM bandwidth)`` on the *local* (sharded)
shapes, with a launch-latency floor; metadata-only ops cost nothing.  FLOPs come from closed
forms per op (GEMM-shaped ops, attention) rather than a FlopCounterMode run per candidate,
which keeps strategy pricing out of the planner's critical path.  Reference:
autoparallel/cost_models/compute_estimation.py:391-493.
"""
from __future__ import annotations

import math
import operator
from typing import Optional, Sequence

import torch

from ..strategies.dtensor_adapter import DTensorSpec, OpSpec, local_shape
from .device import DeviceLimit, get_device_limit

aten = torch.ops.aten
apb = torch.ops.apb200

_ZERO_COST = {
    aten.view.default,
    aten._unsafe_view.default,
    aten.reshape.default,
    aten.alias.default,
    aten.detach.default,
    aten.permute.default,
    aten.t.default,
    aten.transpose.int,
    aten.expand.default,
    aten.unsqueeze.default,
    aten.squeeze.dim,
    aten.squeeze.dims,
    aten.slice.Tensor,
    aten.select.int,
    aten.split_with_sizes.default,
    aten.split.Tensor,
    aten.unbind.int,
    operator.getitem,
}

_cache: dict = {}


def reset_cache() -> None:
    _cache.clear()


def _numel(shape: Sequence[int]) -> int:
    return math.prod(shape) if len(shape) else 1


def _local(spec: Optional[DTensorSpec]) -> Optional[list[int]]:
    if spec is None or spec.tensor_meta is None:
        return None
    return local_shape(spec.tensor_meta.shape, spec.mesh.shape, spec.placements)


def _flops(op, args, in_shapes: list[list[int]], out_shapes: list[list[int]]) -> float:
    if op is apb.mm_nd.default:
        a, b = in_shapes[0], in_shapes[1]
        n = b[0] if args[2] else b[1]
        return 2.0 * _numel(a) * n
    if op is apb.mm_wgrad.default:
        a, b = in_shapes[0], in_shapes[1]
        return 2.0 * _numel(a) * b[-1]
    if op is apb.grouped_mm.default:
        a, b = in_shapes[0], in_shapes[1]
        return 2.0 * _numel(a) * (b[1] if args[2] else b[2])
    if op is apb.grouped_mm_wgrad.default:
        a, b = in_shapes[0], in_shapes[1]
        return 2.0 * _numel(a) * b[2]
    if op is apb.gemm.default or op is aten.mm.default:
        a = in_shapes[0]
        return 2.0 * _numel(a) * out_shapes[0][-1] if op is aten.mm.default else 2.0 * _numel(a) * out_shapes[0][-1]
    if op is aten.bmm.default or op is aten.baddbmm.default:
        a = in_shapes[-2]
        return 2.0 * _numel(a) * out_shapes[0][-1]
    if op is aten.addmm.default:
        return 2.0 * _numel(in_shapes[1]) * out_shapes[0][-1]
    if op is apb.attention.default:
        b, s, h, d = in_shapes[0]
        sk = in_shapes[1][1]
        causal = 0.5 if args[3] else 1.0
        return 4.0 * b * h * s * sk * d * causal
    if op is apb.attention_bwd.default:
        b, s, h, d = in_shapes[1]
        sk = in_shapes[2][1]
        causal = 0.5 if args[6] else 1.0
        return 10.0 * b * h * s * sk * d * causal
    if isinstance(op, torch._ops.HigherOrderOperator):  # flex attention: the block mask's sparsity is not known here
        b, h, s, d = in_shapes[0]
        sk = in_shapes[1][2]
        return (10.0 if "backward" in op.name() else 4.0) * b * h * s * sk * d
    name = str(op)
    if "scaled_dot_product" in name or "_attention" in name:
        q = in_shapes[1] if "backward" in name else in_shapes[0]
        if len(q) == 4:
            b, h, s, d = q
            mult = 10.0 if "backward" in name else 4.0
            return mult * b * h * s * s * d * 0.5
    return 0.0


def strategy_compute_cost(node, spec: OpSpec, limit: Optional[DeviceLimit] = None) -> float:
    """Microseconds for ``node`` when run with ``spec``'s local shapes."""
    op = node.target
    flex = isinstance(op, torch._ops.HigherOrderOperator) and op.name() in ("flex_attention", "flex_attention_backward")
    if op in _ZERO_COST or not (isinstance(op, torch._ops.OpOverload) or flex):
        return 0.0
    outs = spec.output_specs if isinstance(spec.output_specs, (tuple, list)) else [spec.output_specs]
    # (``spec.mesh`` looks at the first output only, which is None when that output is not needed)
    mesh = next((x.mesh for x in list(outs) + list(spec.input_specs or []) if x is not None), None)
    if mesh is None:
        return 0.0
    limit = limit or get_device_limit(mesh.device_type)
    in_shapes, out_shapes = [], []
    nbytes = 0.0
    dtype = None
    for s in spec.input_specs or []:
        ls = _local(s)
        if ls is None:
            continue
        in_shapes.append(ls)
        nbytes += _numel(ls) * s.tensor_meta.dtype.itemsize
        if dtype is None and s.tensor_meta.dtype.is_floating_point:
            dtype = s.tensor_meta.dtype
    for s in outs:
        ls = _local(s)
        if ls is None:
            continue
        out_shapes.append(ls)
        nbytes += _numel(ls) * s.tensor_meta.dtype.itemsize
        if dtype is None and s.tensor_meta.dtype.is_floating_point:
            dtype = s.tensor_meta.dtype
    key = (op, repr(in_shapes), repr(out_shapes), dtype, limit.name, repr([a for a in node.args if isinstance(a, (bool, int, float))]))
    hit = _cache.get(key)
    if hit is not None:
        return hit
    try:
        flops = _flops(op, node.args, in_shapes, out_shapes)
    except Exception:
        flops = 0.0
    t_flops = flops / limit.flops_per_us(dtype or torch.float32)
    t_mem = nbytes / limit.bytes_per_us()
    cost = max(t_flops, t_mem, limit.launch_us)
    _cache[key] = cost
    return cost


# --------------------------------------------------------------------------------------------------
# Estimate against measurement: run a node on the device with its local (sharded) shapes and compare.
# Reference: autoparallel/cost_models/compute_estimation.py:496-556 (benchmark_strategy_runtime_cost,
# compare_estimated_with_benchmarked_throughput).
# --------------------------------------------------------------------------------------------------
def _materialize_args(node, spec: OpSpec, device, seed: int = 0):
    """Real tensors with the local shapes ``spec`` gives the node's tensor inputs; other arguments unchanged."""
    import torch.fx as fx

    gen = torch.Generator(device="cpu").manual_seed(seed)
    tensor_inputs = [a for a in node.all_input_nodes if isinstance(a.meta.get("val"), torch.Tensor)]
    by_node = {}
    for a, s in zip(tensor_inputs, spec.input_specs or []):
        v = a.meta["val"]
        shape = _local(s) if s is not None else list(v.shape)
        if v.dtype.is_floating_point:
            t = (torch.randn(shape, generator=gen) * 0.05).to(v.dtype)
        elif v.dtype == torch.bool:
            t = torch.zeros(shape, dtype=torch.bool)
        else:  # integer inputs are indices: stay inside the smallest extent anything could index
            t = torch.zeros(shape, dtype=v.dtype)
        by_node[a] = t.to(device)

    def conv(a):
        if isinstance(a, fx.Node):
            return by_node.get(a, a.meta.get("val"))
        if isinstance(a, (list, tuple)):
            return type(a)(conv(x) for x in a)
        return a

    return tuple(conv(a) for a in node.args), {k: conv(v) for k, v in node.kwargs.items()}


def benchmark_fn(fn, *args, warmup: int = 3, iters: int = 10, **kwargs) -> float:
    """Mean device time of ``fn(*args, **kwargs)`` in microseconds (CUDA events; wall clock on CPU)."""
    import time

    for _ in range(warmup):
        fn(*args, **kwargs)
    if torch.cuda.is_available() and any(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(iters):
            fn(*args, **kwargs)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters * 1e3
    t0 = time.perf_counter()
    for _ in range(iters):
        fn(*args, **kwargs)
    return (time.perf_counter() - t0) / iters * 1e6


def benchmark_strategy_runtime_cost(node, spec: OpSpec, device=None) -> float:
    """Counterpart of ``strategy_compute_cost`` that runs the node: microseconds measured on ``device`` (default:
    the current CUDA device, else CPU) with random inputs of the local shapes."""
    if node.target in _ZERO_COST or not isinstance(node.target, torch._ops.OpOverload):
        return 0.0
    device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    args, kwargs = _materialize_args(node, spec, device)
    with torch.no_grad():
        return benchmark_fn(node.target, *args, **kwargs)


def compare_estimated_with_benchmarked_throughput(graph, sharding_placement, tgt_ops="mm", device=None, limit=None) -> dict:
    """For every node of ``graph`` whose target is in ``tgt_ops`` ("mm": this framework's GEMM operators and the ATen
    matmuls; ``None``: every operator): ``node -> (measured us, estimated us, achieved TFLOP/s, device peak TFLOP/s,
    efficiency)`` under the placement the solver chose.  The estimate prices a node at ``max(FLOPs / peak, bytes /
    bandwidth)`` of the device table; this shows how far the table is from the kernels it prices."""
    if tgt_ops == "mm":
        tgt_ops = [apb.mm_nd.default, apb.mm_wgrad.default, apb.gemm.default, aten.mm.default, aten.bmm.default]
    data = {}
    for node in graph.nodes:
        if node.op != "call_function" or node not in sharding_placement:
            continue
        if tgt_ops is not None and node.target not in tgt_ops:
            continue
        spec = sharding_placement[node]
        in_shapes = [_local(s) for s in (spec.input_specs or []) if s is not None and _local(s) is not None]
        outs = spec.output_specs if isinstance(spec.output_specs, (tuple, list)) else [spec.output_specs]
        out_shapes = [_local(s) for s in outs if s is not None and _local(s) is not None]
        flops = _flops(node.target, node.args, in_shapes, out_shapes)
        real_us = benchmark_strategy_runtime_cost(node, spec, device)
        est_us = strategy_compute_cost(node, spec, limit)
        dtype = next((s.tensor_meta.dtype for s in (spec.input_specs or []) if s is not None and s.tensor_meta.dtype.is_floating_point),
                     torch.float32)
        lim = limit or get_device_limit("cuda" if torch.cuda.is_available() else "cpu")
        peak = lim.flops_per_us(dtype) / 1e6  # TFLOP/s
        achieved = flops / (real_us * 1e-6) * 1e-12 if real_us > 0 else 0.0
        data[node] = (real_us, est_us, achieved, peak, achieved / peak if peak else 0.0)
    return data
