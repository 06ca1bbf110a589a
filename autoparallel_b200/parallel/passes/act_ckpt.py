"""Recompute tagging: FSDP re-gather and activation checkpointing.

``mark_fsdp_recompute`` tags every node that is derived from a parameter through single-input
ops (cast → all-gather → transpose/view chains).  With ``reshard_after_forward`` the partitioner
then clones that chain into the backward graph instead of saving the gathered weight, i.e. ZeRO-3
"reshard after forward"; without it the last node of each chain is pinned as saved.
Reference: autoparallel/graph_passes/activation_checkpointing.py:182-271, 518-533.

``apply_activation_checkpointing`` implements the memory-budget policy: cheap pointwise /
normalisation results are recomputed, GEMM and attention outputs are kept, and per "stage" of
``stage_bytes`` of live activations the cheapest cut is pinned (reference: :365-552).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.fx as fx

from ...runtime import comm_ops
from ..frontend.graph_canon import param_derived_set
from ..frontend.trace import JointGraph
from ..lower.partition import MUST_SAVE, RECOMPUTE

aten = torch.ops.aten
apb = torch.ops.apb200

_EXPENSIVE = {
    apb.mm_nd.default,
    apb.mm_wgrad.default,
    apb.gemm.default,
    apb.attention.default,
    aten.mm.default,
    aten.bmm.default,
    aten.addmm.default,
    aten._scaled_dot_product_flash_attention.default,
    aten._scaled_dot_product_efficient_attention.default,
    aten._scaled_dot_product_cudnn_attention.default,
    aten._scaled_dot_product_flash_attention_for_cpu.default,
}


def fsdp_all_gather_chains(joint: JointGraph) -> list[list[fx.Node]]:
    """Parameter-derived chains that contain an all-gather (the "FSDP" gathers)."""
    derived = param_derived_set(joint.gm, joint.param_nodes.values())
    chains = []
    for p in joint.param_nodes.values():
        chain, cur = [], p
        while True:
            nxt = [u for u in cur.users if u in derived and u.op == "call_function"]
            if len(nxt) != 1:
                break
            cur = nxt[0]
            chain.append(cur)
        if any(n.target is comm_ops.ops.all_gather.default for n in chain):
            chains.append(chain)
    return chains


def mark_fsdp_recompute(joint: JointGraph, reshard_after_forward: bool = True) -> int:
    derived = param_derived_set(joint.gm, joint.param_nodes.values())
    count = 0
    if reshard_after_forward:
        for n in derived:
            if n.op == "call_function":
                n.meta[RECOMPUTE] = True
                count += 1
    else:
        for chain in fsdp_all_gather_chains(joint):
            chain[-1].meta[MUST_SAVE] = True
            count += 1
    return count


def _nbytes(n: fx.Node) -> int:
    v = n.meta.get("val")
    if isinstance(v, torch.Tensor):
        return v.numel() * v.element_size()
    if isinstance(v, (tuple, list)):
        return sum(x.numel() * x.element_size() for x in v if isinstance(x, torch.Tensor))
    return 0


def apply_activation_checkpointing(
    joint: JointGraph, mode: str = "selective", stage_bytes: Optional[int] = None, save_every_other_mm: bool = False
) -> dict:
    """Tag forward nodes for recomputation.

    ``mode``: ``"none"`` | ``"selective"`` (recompute cheap ops; keep GEMM / attention results) |
    ``"full"`` (keep only stage boundaries – the block inputs – and recompute everything else).
    """
    if mode == "none":
        return {"recompute": 0, "saved": 0}
    tangents = set(joint.tangent_nodes)
    g = joint.gm.graph
    T = set(tangents)
    for n in g.nodes:
        if n.op == "call_function" and any(i in T for i in n.all_input_nodes):
            T.add(n)
    fwd = [n for n in g.nodes if n.op == "call_function" and n not in T]
    n_rec = n_save = 0
    mm_seen = 0
    import operator

    for n in fwd:
        if n.meta.get(RECOMPUTE) or n.meta.get(MUST_SAVE):
            continue
        if n.target is operator.getitem:
            src = n.args[0]
            if src.meta.get(RECOMPUTE) and not src.meta.get(MUST_SAVE):
                n.meta[RECOMPUTE] = True
            continue
        expensive = n.target in _EXPENSIVE or n.target in comm_ops.COLLECTIVE_OPS
        if mode == "selective":
            if expensive:
                if save_every_other_mm and n.target in (apb.mm_nd.default, aten.mm.default):
                    mm_seen += 1
                    if mm_seen % 2 == 0:
                        n.meta[RECOMPUTE] = True
                        n_rec += 1
                        continue
                n.meta[MUST_SAVE] = True
                n_save += 1
            else:
                n.meta[RECOMPUTE] = True
                n_rec += 1
        else:  # full
            n.meta[RECOMPUTE] = True
            n_rec += 1
    if mode == "full":
        # pin stage boundaries: walk the forward in order, accumulate output bytes, and when a
        # stage is full pin the narrowest single-tensor cut seen in it (a residual-stream tensor)
        if stage_bytes is None:
            total = sum(_nbytes(n) for n in fwd)
            stage_bytes = max(1, int(math.sqrt(max(total, 1) / 2**30) * 2**30)) if total > 2**30 else max(total // 8, 1)
        acc = 0
        best = None
        for n in fwd:
            acc += _nbytes(n)
            users_fwd = [u for u in n.users if u not in T]
            if isinstance(n.meta.get("val"), torch.Tensor) and len(users_fwd) >= 2 and n.target is aten.add.Tensor:
                if best is None or _nbytes(n) <= _nbytes(best):
                    best = n
            if acc >= stage_bytes and best is not None:
                best.meta[MUST_SAVE] = True
                best.meta.pop(RECOMPUTE, None)
                n_save += 1
                acc, best = 0, None
    return {"recompute": n_rec, "saved": n_save}
