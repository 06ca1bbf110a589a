"""Split the lowered joint graph into a forward and a backward graph.

* forward  = ancestors of the forward outputs;
* backward = everything that depends on a tangent, plus value-only side computations that only
  the backward consumes (they are materialised late instead of being saved);
* a forward node tagged ``recompute`` that the backward needs is *cloned* into the backward
  (together with its tagged producers) rather than saved – this is how FSDP re-gathers parameters
  in the backward pass and how activation checkpointing drops activations;
* everything else the backward reads from the forward becomes a saved tensor.

The reference delegates this to functorch's min-cut partitioner and replays its decisions
(autoparallel/compile.py:27-246, autoparallel/api.py:63-97); this partitioner is deterministic
and tag-driven, which is what the stream scheduler downstream wants.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.fx as fx

from ..frontend.trace import JointGraph

RECOMPUTE = "apb200_recompute"
MUST_SAVE = "apb200_must_save"


@dataclasses.dataclass
class PartitionedGraph:
    fw: fx.GraphModule
    bw: fx.GraphModule
    #: names of joint placeholders feeding the forward graph, in order
    fw_inputs: list[fx.Node]
    num_fwd_outputs: int
    num_saved: int
    #: for each backward input: ("saved", i) | ("primal", i into fw_inputs) | ("tangent", out idx)
    bw_inputs: list[tuple[str, int]]
    #: backward outputs: gradient w.r.t. fw_inputs[i] or None
    grad_of_input: list[Optional[int]]  # index into bw outputs for each fw input (None = no grad)
    saved_bytes: int = 0


def _is_tensor(n: fx.Node) -> bool:
    return isinstance(n.meta.get("val"), torch.Tensor)


def partition_joint(joint: JointGraph) -> PartitionedGraph:
    g = joint.gm.graph
    nodes = list(g.nodes)
    tangents = set(joint.tangent_nodes)
    primals = [n for n in nodes if n.op == "placeholder" and n not in tangents]

    # 1. tangent-dependent closure
    T: set[fx.Node] = set(tangents)
    for n in nodes:
        if n.op == "call_function" and any(i in T for i in n.all_input_nodes):
            T.add(n)
    # 2. forward-required closure
    F: set[fx.Node] = set()
    stack = [o for o in joint.fwd_outputs if isinstance(o, fx.Node)]
    while stack:
        n = stack.pop()
        if n in F:
            continue
        F.add(n)
        stack.extend(n.all_input_nodes)
    assert not (F & T), "a forward output depends on a tangent"
    # getitem of a forward multi-output node stays in the forward (tuples cannot be saved)
    import operator as _op

    for n in nodes:
        if n.op == "call_function" and n.target is _op.getitem and n.args[0] in F and n not in T:
            F.add(n)
    # 3. value-only side nodes go to the backward side
    out_node = next(n for n in nodes if n.op == "output")
    B: set[fx.Node] = {n for n in nodes if n.op == "call_function" and (n in T or n not in F)}
    # 4. recompute clones
    needed_from_fwd: list[fx.Node] = []
    clone: set[fx.Node] = set()

    def need(n: fx.Node):
        if n.op != "call_function" or n in B or n in clone:
            return
        if n.target is _op.getitem:
            src = n.args[0]
            # an element of a multi-output node is recomputed only together with its producer
            if not (src.op == "call_function" and src.meta.get(RECOMPUTE) and not src.meta.get(MUST_SAVE)):
                return
        if n.meta.get(RECOMPUTE) and not n.meta.get(MUST_SAVE):
            clone.add(n)
            for i in n.all_input_nodes:
                need(i)

    for n in nodes:
        if n in B:
            for i in n.all_input_nodes:
                need(i)
    bw_side = B | clone
    saved: list[fx.Node] = []
    used_primals: list[fx.Node] = []
    seen = set()
    for n in nodes:
        if n not in bw_side:
            continue
        for i in n.all_input_nodes:
            if i in bw_side or i in seen or i in tangents or i.op == "get_attr":
                continue  # attributes (constants, sub-graphs of higher-order operators) are re-read, not saved
            seen.add(i)
            if i.op == "placeholder":
                used_primals.append(i)
            else:
                saved.append(i)

    # ---- forward graph
    fw_g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    for p in primals:
        env[p] = fw_g.placeholder(p.name)
        env[p].meta = dict(p.meta)
    for n in nodes:
        if n.op == "call_function" and n in F or (n.op == "get_attr" and n in F):
            env[n] = fw_g.node_copy(n, lambda a: env[a])
    fw_outs = [env[o] if isinstance(o, fx.Node) else o for o in joint.fwd_outputs]
    fw_g.output(tuple(fw_outs + [env[s] for s in saved]))
    fw_gm = fx.GraphModule(joint.gm, fw_g)

    # ---- backward graph
    bw_g = fx.Graph()
    benv: dict[fx.Node, fx.Node] = {}
    bw_inputs: list[tuple[str, int]] = []
    for i, s in enumerate(saved):
        benv[s] = bw_g.placeholder(f"saved_{s.name}")
        benv[s].meta = dict(s.meta)
        bw_inputs.append(("saved", i))
    for p in used_primals:
        benv[p] = bw_g.placeholder(p.name)
        benv[p].meta = dict(p.meta)
        bw_inputs.append(("primal", primals.index(p)))
    for t in joint.tangent_nodes:
        benv[t] = bw_g.placeholder(t.name)
        benv[t].meta = dict(t.meta)
        bw_inputs.append(("tangent", t.meta.get("apb200_tangent_of", 0)))
    for n in nodes:
        if n in bw_side or (n.op == "get_attr" and any(u in bw_side for u in n.users)):
            benv[n] = bw_g.node_copy(n, lambda a: benv[a])
    grads: list[fx.Node] = []
    grad_of_input: list[Optional[int]] = []
    grad_nodes = {}
    for fqn, p in joint.param_nodes.items():
        grad_nodes[p] = joint.param_grads.get(fqn)
    for i, p in enumerate(joint.input_nodes):
        if p is not None:
            grad_nodes[p] = joint.input_grads[i] if i < len(joint.input_grads) else None
    for p in primals:
        gn = grad_nodes.get(p)
        if isinstance(gn, fx.Node):
            grad_of_input.append(len(grads))
            # a gradient that is itself a forward value / primal (rare) is passed through
            if gn not in benv:
                raise RuntimeError(f"gradient node {gn.name} of {p.name} is not part of the backward graph (stale graph index?)")
            grads.append(benv[gn])
        else:
            grad_of_input.append(None)
    bw_g.output(tuple(grads))
    bw_gm = fx.GraphModule(joint.gm, bw_g)

    saved_bytes = 0
    for s in saved:
        v = s.meta.get("val")
        if isinstance(v, torch.Tensor):
            saved_bytes += v.numel() * v.element_size()
    for gm_ in (fw_gm, bw_gm):
        gm_.graph.eliminate_dead_code()
        gm_.graph.lint()
        gm_.recompile()
    return PartitionedGraph(
        fw=fw_gm,
        bw=bw_gm,
        fw_inputs=primals,
        num_fwd_outputs=len(fw_outs),
        num_saved=len(saved),
        bw_inputs=bw_inputs,
        grad_of_input=grad_of_input,
        saved_bytes=saved_bytes,
    )


def extract_forward(joint: JointGraph) -> fx.GraphModule:
    """Forward-only graph for inference: primals in, forward outputs out, nothing saved
    (reference: autoparallel/graph_passes/extract_forward.py:13-75)."""
    g = joint.gm.graph
    tangents = set(joint.tangent_nodes)
    F: set[fx.Node] = set()
    stack = [o for o in joint.fwd_outputs if isinstance(o, fx.Node)]
    while stack:
        n = stack.pop()
        if n in F:
            continue
        F.add(n)
        stack.extend(n.all_input_nodes)
    fw_g = fx.Graph()
    env: dict[fx.Node, fx.Node] = {}
    for n in g.nodes:
        if n.op == "placeholder" and n not in tangents:
            env[n] = fw_g.placeholder(n.name)
            env[n].meta = dict(n.meta)
        elif n in F and n.op in ("call_function", "get_attr"):
            env[n] = fw_g.node_copy(n, lambda a: env[a])
    fw_g.output(tuple(env[o] if isinstance(o, fx.Node) else o for o in joint.fwd_outputs))
    gm = fx.GraphModule(joint.gm, fw_g)
    gm.graph.lint()
    gm.recompile()
    return gm
