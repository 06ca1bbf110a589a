"""Recompute tagging: FSDP re-gather and activation checkpointing.

``mark_fsdp_recompute`` tags every node that is derived from a parameter through single-input
ops (cast → all-gather → transpose/view chains).  With ``reshard_after_forward`` the partitioner
then clones that chain into the backward graph instead of saving the gathered weight, i.e. ZeRO-3
"reshard after forward"; without it the last node of each chain is pinned as saved.
Reference: autoparallel/graph_passes/activation_checkpointing.py:182-271, 518-533.

``apply_user_checkpoint_tags`` honours what the user wrote with ``torch.utils.checkpoint``: nodes
traced inside a checkpointed region carry ``meta["recompute"]`` (a ``CheckpointPolicy`` from the
region's selective-checkpoint policy, or "prefer recompute" for a plain region) and
``meta["ac_graph_id"]``; save policies become ``must_save`` tags and recompute policies
``recompute`` tags of the partitioner.  User tags are applied first and the framework's own policy
never overrides them; parameter-gather chains stay "recompute" whatever the user region says
(reference: :34, 224-235, 356, 410).

``apply_activation_checkpointing`` implements the memory-budget policy: cheap pointwise /
normalisation results are recomputed, GEMM and attention outputs are kept ("selective"), or
everything is recomputed from stage boundaries ("full"): the forward is cut into stages of
``stage_bytes`` of produced activations and in every stage the set of tensors alive at the point of
least live memory is saved (reference: :365-494).
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
                n.meta["apb200_param_chain"] = True
                count += 1
    else:
        for chain in fsdp_all_gather_chains(joint):
            chain[-1].meta[MUST_SAVE] = True
            count += 1
    return count


def _forward_nodes(joint: JointGraph):
    """(forward call_function nodes in order, set of tangent-dependent nodes)."""
    T = set(joint.tangent_nodes)
    for n in joint.gm.graph.nodes:
        if n.op == "call_function" and any(i in T for i in n.all_input_nodes):
            T.add(n)
    # forward = what the forward outputs need; value-only nodes that only the backward reads (the cosine
    # of a saved input, say) run on the backward side and must not count as forward activations
    F, stack = set(), [o for o in joint.fwd_outputs if isinstance(o, fx.Node)]
    while stack:
        n = stack.pop()
        if n in F:
            continue
        F.add(n)
        stack.extend(n.all_input_nodes)
    import operator as _op

    for n in joint.gm.graph.nodes:
        if n.op == "call_function" and n.target is _op.getitem and n.args[0] in F and n not in T:
            F.add(n)
    return [n for n in joint.gm.graph.nodes if n.op == "call_function" and n in F and n not in T], T


def apply_user_checkpoint_tags(joint: JointGraph) -> dict:
    """Translate ``CheckpointPolicy`` tags left by ``torch.utils.checkpoint`` regions into partitioner tags."""
    from torch.utils.checkpoint import CheckpointPolicy

    save = {CheckpointPolicy.MUST_SAVE, CheckpointPolicy.PREFER_SAVE}
    recompute = {CheckpointPolicy.MUST_RECOMPUTE, CheckpointPolicy.PREFER_RECOMPUTE}
    fwd, _ = _forward_nodes(joint)
    stats = {"user_saved": 0, "user_recompute": 0, "regions": set()}
    for n in fwd:
        pol = n.meta.get("recompute")
        if pol is None or n.meta.get("ac_graph_id") is None:
            continue
        stats["regions"].add(n.meta["ac_graph_id"])
        if n.meta.get(RECOMPUTE) and not n.meta.get(MUST_SAVE):
            continue  # parameter-gather chain: re-gathered in the backward whatever the region's policy says
        if pol in save:
            n.meta[MUST_SAVE] = True
            n.meta.pop(RECOMPUTE, None)
            stats["user_saved"] += 1
        elif pol in recompute:
            n.meta[RECOMPUTE] = True
            stats["user_recompute"] += 1
        n.meta["apb200_user_ac"] = True
    stats["regions"] = len(stats["regions"])
    return stats


def min_live_memory_cuts(fwd: list, stage_bytes: int) -> list:
    """Nodes to save so that no recomputation chain is longer than one stage.

    The forward nodes are walked in order while tracking which results are alive (produced and still
    needed by a later forward node; results that are always recomputed, such as gathered parameters, are
    looked through).  A new stage starts whenever ``stage_bytes`` of results have been produced; in each
    stage the position with the least live memory is the cut, and everything alive there is saved."""
    in_fwd = set(fwd)
    always_recomputed = {n for n in fwd if n.meta.get(RECOMPUTE) and not n.meta.get(MUST_SAVE) and not n.meta.get("apb200_user_ac")
                         and n.meta.get("apb200_param_chain")}
    preds: dict = {}
    for n in fwd:
        ps = []
        for i in n.all_input_nodes:
            if i in always_recomputed:
                ps.extend(preds.get(i, ()))
            elif i in in_fwd:
                ps.append(i)
        preds[n] = ps
    last_user: dict = {}
    for n in fwd:
        last_user[n] = n
        for p_ in preds[n]:
            last_user[p_] = n
    dies_at: dict = {}
    for prod, cons in last_user.items():
        dies_at.setdefault(cons, []).append(prod)
    alive: dict = {}
    live_bytes = 0
    stages, cur, produced = [], [], 0
    for n in fwd:
        if n not in always_recomputed:
            alive[n] = None
            live_bytes += _nbytes(n)
            for d in dies_at.get(n, ()):
                if d in alive and d is not n:
                    del alive[d]
                    live_bytes -= _nbytes(d)
            produced += _nbytes(n)
        cur.append((live_bytes, n, list(alive)))
        if produced >= stage_bytes:
            stages.append(cur)
            cur, produced = [], 0
    if cur:
        stages.append(cur)
    cuts = []
    for st in stages[:-1] if len(stages) > 1 else []:  # nothing follows the last stage: its results are consumed by the backward at once
        _, _, live = min(st, key=lambda e: e[0])
        cuts.extend(live)
    return list(dict.fromkeys(cuts))


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
    fwd, T = _forward_nodes(joint)
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
        if stage_bytes is None:  # "auto": the square root of the recomputable memory, in GiB
            total = sum(_nbytes(n) for n in fwd)
            stage_bytes = max(1, int(math.sqrt(max(total, 1) / 2**30) * 2**30)) if total > 2**30 else max(total // 8, 1)
        for cut in min_live_memory_cuts(fwd, stage_bytes):
            if cut.meta.get("apb200_user_ac") or cut.target is operator.getitem:
                continue  # user annotations take precedence; tuple elements follow their producer
            if cut.meta.get(RECOMPUTE):
                cut.meta.pop(RECOMPUTE, None)
                n_rec -= 1
            if not cut.meta.get(MUST_SAVE):
                cut.meta[MUST_SAVE] = True
                n_save += 1
    return {"recompute": n_rec, "saved": n_save}
