"""``local_map`` regions in the planner.

A region written by the user with explicit per-mesh-dim placements (the MoE block: route →
dispatch all-to-all → grouped expert GEMM → combine) is captured as ONE graph node whose body
was traced on local shapes.  The planner does not look inside: the node has exactly one strategy –
inputs in the declared ``in_placements``, real outputs in ``out_placements``, the extra outputs the
autograd split adds (activations saved for the region's backward, already local) replicated; the
backward twin takes those saved tensors replicated, tangents in ``out_placements`` and returns
gradients in ``in_grad_placements`` (default: ``in_placements``).  Tensors with placement ``None``
(non-tensor or data-dependent shapes) are never redistributed.  At lowering the body is inlined.
Reference: autoparallel/shardings/placement_options.py:362-490, autoparallel/apply_sharding.py:186-238.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.fx as fx

from .dtensor_adapter import DTensorSpec, OpSpec, OpStrategy, Replicate, tensor_meta_of


def is_local_map_node(node: fx.Node) -> bool:
    return node.op == "call_function" and "local_map_kwargs" in node.meta and callable(node.target)


def local_map_body(node: fx.Node) -> fx.GraphModule:
    """The region's body (a GraphModule over local tensors) captured in the node's target."""
    fn = node.target
    for name, cell in zip(fn.__code__.co_freevars, fn.__closure__ or ()):
        v = cell.cell_contents
        if isinstance(v, fx.GraphModule):
            return v
    raise RuntimeError(f"cannot find the body of local_map node {node.name}")


def _is_backward(node: fx.Node) -> bool:
    return "fwd_nn_module_stack" in node.meta or node.meta.get("partitioner_tag") == "is_backward"


def _norm(pl, mesh) -> Optional[tuple]:
    if pl is None:
        return None
    return tuple(pl)


def local_map_options(mesh, node: fx.Node, strats) -> OpStrategy:
    kw = node.meta["local_map_kwargs"]
    in_pl = [_norm(p, mesh) for p in (kw.get("in_placements") or ())]
    out_pl = kw.get("out_placements")
    if out_pl is not None and len(out_pl) > 0 and not isinstance(out_pl[0], (tuple, list, type(None))):
        out_pl = (tuple(out_pl),)
    out_pl = [_norm(p, mesh) for p in (out_pl or ())]
    rep = (Replicate(),) * mesh.ndim
    vals = node.meta["val"]
    vals = list(vals) if isinstance(vals, (tuple, list)) else [vals]
    in_nodes = [a for a in node.args if isinstance(a, fx.Node) and isinstance(a.meta.get("val"), torch.Tensor)]

    def spec(pl, v):
        if not isinstance(v, torch.Tensor):
            return None
        return DTensorSpec(mesh, pl if pl is not None else rep, tensor_meta=tensor_meta_of(v))

    if not _is_backward(node):
        n_real = len(out_pl)
        outs = [spec(out_pl[i] if i < n_real else rep, v) for i, v in enumerate(vals)]
        tensor_in_pl = [p for p in in_pl]
        # in_placements lists one entry per positional argument, tensors and non-tensors alike
        ins = []
        ti = 0
        for a in node.args:
            if isinstance(a, fx.Node) and isinstance(a.meta.get("val"), torch.Tensor):
                pl = tensor_in_pl[ti] if ti < len(tensor_in_pl) else rep
                ins.append(spec(pl, a.meta["val"]))
            ti += 1
    else:
        # the backward twin's kwargs are already swapped by the HOP: ``in_placements`` describe the
        # tangents (the trailing tensor arguments; the saved activations come first),
        # ``out_placements`` the returned input gradients
        n_tan = len(in_pl)
        n_saved = len(in_nodes) - n_tan
        ins = []
        for i, a in enumerate(in_nodes):
            pl = rep if i < n_saved else in_pl[i - n_saved]
            ins.append(spec(pl, a.meta["val"]))
        outs = [spec(out_pl[i] if i < len(out_pl) else rep, v) for i, v in enumerate(vals)]
    out_specs = tuple(outs) if len(outs) != 1 or isinstance(node.meta["val"], (tuple, list)) else outs[0]
    return OpStrategy([OpSpec(out_specs, input_specs=ins)])
