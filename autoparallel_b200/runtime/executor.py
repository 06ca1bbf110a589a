"""Execution of the partitioned per-rank graphs.

``build_runtime`` wraps the forward and backward ``GraphModule``s in one
``torch.autograd.Function`` so the parallel module composes with ordinary autograd: gradients
w.r.t. local parameter shards flow back through ``DTensor.to_local`` into ``param.grad``.
Under ``torch.no_grad()`` the forward-only graph runs instead and nothing is saved.

Executors:

* ``graph``   – the FX-generated Python of each graph, one op launch per node, single stream;
* ``streams`` – same graphs after the overlap scheduler (``parallel/passes/overlap.py``) has
  split collectives into issue/wait pairs on a communication stream and hoisted parameter
  gathers ahead of their consumers.

Reference: autoparallel/api.py:615-651 (the AOT-compiled boxed callable driven by the FX
interpreter, api.py:92-94).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.fx as fx

from ..parallel.lower.apply import LoweredGraph
from ..parallel.lower.partition import PartitionedGraph


class Runtime:
    def __init__(self, lowered: LoweredGraph, parts: PartitionedGraph, fwd_only: fx.GraphModule, mesh, executor: Optional[str],
                 overlap_config=None):
        self.lowered = lowered
        self.parts = parts
        self.mesh = mesh
        self.executor = executor or "graph"
        self.fw = parts.fw
        self.bw = parts.bw
        self.fwd_only = fwd_only
        joint = lowered.joint
        # order of forward-graph inputs = order of joint primals; map (kind, key) -> position
        self._order = []
        pnames = list(joint.param_nodes)
        bnames = list(joint.buffer_nodes)
        p_idx = {n: i for i, n in enumerate(joint.param_nodes.values())}
        b_idx = {n: i for i, n in enumerate(joint.buffer_nodes.values())}
        i_idx = {}
        k = 0
        for n in joint.input_nodes:
            if n is not None:
                i_idx[n] = k
            k += 1
        self._tensor_input_pos = {}
        flat_tensor_counter = 0
        for n in joint.input_nodes:
            if n is not None:
                self._tensor_input_pos[n] = flat_tensor_counter
            flat_tensor_counter += 1
        for n in parts.fw_inputs:
            if n in p_idx:
                self._order.append(("param", p_idx[n]))
            elif n in b_idx:
                self._order.append(("buffer", b_idx[n]))
            else:
                self._order.append(("input", self._tensor_input_pos[n]))
        self._n_in = flat_tensor_counter
        # forward inputs that the module overwrites after the call (buffers the forward mutates: running statistics and
        # the like): a backward that reads them - a recomputed batch norm does - must see the value the forward saw
        self._mutated_inputs = {pos for pos, (kind, i) in enumerate(self._order)
                                if kind == "buffer" and bnames[i] in getattr(joint, "buffer_updates", {})}
        self._graph_device = torch.device("cpu")  # device constants inside the graphs (planning happens on CPU fake tensors)
        self._fn = _make_function(self)
        if self.executor == "streams":
            from ..parallel.passes.overlap import schedule_for_streams

            self.fw = schedule_for_streams(self.fw, mesh, overlap_config)
            self.bw = schedule_for_streams(self.bw, mesh, overlap_config)

    def _retarget(self, device: torch.device) -> None:
        """Planning runs on CPU fake tensors, so factory operators traced with an explicit ``device=`` (``torch.zeros(...,
        device=x.device)`` inside a user region, ``arange`` for index arithmetic) carry "cpu" as a constant.  Before the
        first run on another device the constant is replaced in every graph of this runtime, and operators that exist on
        the planning host only are swapped for device-neutral stand-ins."""
        if device == self._graph_device:
            return
        from .portable_ops import SWAPS

        for gm in (self.fw, self.bw, self.fwd_only):
            changed = False
            for n in gm.graph.nodes:
                if n.op == "get_attr":
                    # tensor constants the forward creates (``torch.tensor([...])``) were materialised on the planning host
                    t = getattr(gm, n.target, None) if "." not in n.target else None
                    if (isinstance(t, torch.Tensor) and type(t).__name__ != "FakeTensor" and t.device != device
                            and t.device.type != "meta"):
                        setattr(gm, n.target, t.to(device))
                    continue
                if n.op != "call_function":
                    continue
                if n.target in SWAPS and device.type != "cpu":
                    n.target = SWAPS[n.target]  # an operator only the planning host implements (runtime/portable_ops.py)
                    changed = True
                if isinstance(n.kwargs.get("device"), torch.device) and n.kwargs["device"] != device:
                    n.kwargs = {**n.kwargs, "device": device}
                    changed = True
                new_args = tuple(device if isinstance(a, torch.device) and a != device else a for a in n.args)
                if any(x is not y for x, y in zip(new_args, n.args)):
                    n.args = new_args
                    changed = True
            if changed:
                gm.recompile()
        self._graph_device = device

    def gather_inputs(self, params, buffers, inputs):
        src = {"param": params, "buffer": buffers, "input": inputs}
        return [src[k][i] for k, i in self._order]

    def __call__(self, params: Sequence[torch.Tensor], buffers, inputs, grad_enabled: bool):
        flat = self.gather_inputs(params, buffers, inputs)
        dev = next((t.device for t in flat if isinstance(t, torch.Tensor)), None)
        if dev is not None and dev != self._graph_device:
            self._retarget(dev)
        if not grad_enabled:
            with torch.no_grad():
                return tuple(self.fwd_only(*flat))
        return self._fn(*flat)


def _make_function(rt: Runtime):
    parts = rt.parts
    n_out = parts.num_fwd_outputs

    class ParallelGraphFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *flat):
            outs = rt.fw(*flat)
            fwd_outs, saved = outs[:n_out], outs[n_out:]
            prim = [flat[i].clone() if i in rt._mutated_inputs else flat[i] for kind, i in parts.bw_inputs if kind == "primal"]
            ctx.save_for_backward(*saved, *prim)
            ctx.n_saved = len(saved)
            for o in fwd_outs:
                if isinstance(o, torch.Tensor) and not o.dtype.is_floating_point:
                    ctx.mark_non_differentiable(o)
            return tuple(fwd_outs)

        @staticmethod
        def backward(ctx, *grads):
            st = ctx.saved_tensors
            saved, prim = st[: ctx.n_saved], st[ctx.n_saved :]
            args = list(saved) + list(prim)
            for kind, i in parts.bw_inputs:
                if kind == "tangent":
                    g = grads[i]
                    args.append(g.contiguous() if g is not None else None)
            outs = rt.bw(*args)
            res = []
            for gi in parts.grad_of_input:
                res.append(outs[gi] if gi is not None else None)
            return tuple(res)

    return ParallelGraphFunction.apply


def build_runtime(lowered, parts, fwd_only, mesh, executor=None, overlap_config=None) -> Runtime:
    return Runtime(lowered, parts, fwd_only, mesh, executor, overlap_config)
