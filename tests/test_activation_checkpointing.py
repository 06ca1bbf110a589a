"""Activation checkpointing: user regions (``torch.utils.checkpoint`` with and without a selective policy), the
framework's own policies, and the stage cut of the "full" mode.

Modelled on the reference's tests/test_activation_checkpointing.py:137-300 (user tags reach the joint graph
and decide what is saved) and :365-494 of its AC pass (stage cuts by least live memory)."""
import functools
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from conftest import free_port
from torch.distributed.tensor.placement_types import Shard
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from autoparallel_b200 import AutoParallel
from autoparallel_b200.parallel.lower.partition import MUST_SAVE, RECOMPUTE

apb = torch.ops.apb200
aten = torch.ops.aten


def _save_matmuls(ctx, op, *args, **kwargs):
    if op in (aten.mm.default, aten.addmm.default, aten.linear.default):
        return CheckpointPolicy.MUST_SAVE
    return CheckpointPolicy.PREFER_RECOMPUTE


class Block(nn.Module):
    def __init__(self, d, f, context_fn=None, wrap=True):
        super().__init__()
        self.w1 = nn.Linear(d, f, bias=False)
        self.w2 = nn.Linear(f, d, bias=False)
        self.context_fn, self.wrap = context_fn, wrap

    def _inner(self, x):
        return self.w2(torch.relu(self.w1(x)).sin())

    def forward(self, x):
        if not self.wrap:
            return x + self._inner(x)
        if self.context_fn is not None:
            return x + checkpoint(self._inner, x, use_reentrant=False, context_fn=self.context_fn)
        return x + checkpoint(self._inner, x, use_reentrant=False)


class Stack(nn.Module):
    def __init__(self, n=2, d=64, f=128, context_fn=None, wrap=True):
        super().__init__()
        self.blocks = nn.ModuleList([Block(d, f, context_fn, wrap) for _ in range(n)])

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x


def _plan(mesh, model, ac="none", **kw):
    ap = AutoParallel(model, lambda: torch.rand(64, 16, 64), mesh, activation_checkpointing=ac, **kw)
    ap.__enter__()
    ap.add_input_constraints([(Shard(0),)])
    ap.optimize_placement()
    return ap


def _targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


def test_selective_policy_of_the_user_decides_what_is_saved(mesh_1d):
    ctx = functools.partial(create_selective_checkpoint_contexts, _save_matmuls)
    with torch.device("meta"):
        model = Stack(context_fn=ctx)
    ap = _plan(mesh_1d, model)
    try:
        low = ap.lower()
        assert ap.user_ac_stats["regions"] == 2 and ap.user_ac_stats["user_saved"] == 4
        fwd_mm = [n for n in low.gm.graph.nodes if n.target is apb.mm_nd.default and n.meta.get("recompute") is not None]
        assert len(fwd_mm) == 4 and all(n.meta.get(MUST_SAVE) for n in fwd_mm)
        cheap = [n for n in low.gm.graph.nodes if n.target in (aten.relu.default, aten.sin.default)]
        assert len(cheap) == 4 and all(n.meta.get(RECOMPUTE) and not n.meta.get(MUST_SAVE) for n in cheap)
        ap.apply_placement()
        bw = _targets(ap.partitioned.bw)
        # relu is recomputed in the backward from the saved matmul result; no matmul of the forward is run again
        assert bw.count(aten.relu.default) == 2
        assert bw.count(apb.mm_nd.default) == 3  # input gradients only (the model input needs none)
    finally:
        ap.__exit__(None, None, None)


def test_plain_checkpoint_region_is_recomputed_and_unwrapped_model_is_not(mesh_1d):
    with torch.device("meta"):
        wrapped, plain = Stack(), Stack(wrap=False)
    a = _plan(mesh_1d, wrapped)
    try:
        a.apply_placement()
        saved_wrapped, bw_wrapped = a.partitioned.saved_bytes, _targets(a.partitioned.bw)
    finally:
        a.__exit__(None, None, None)
    b = _plan(mesh_1d, plain)
    try:
        b.apply_placement()
        saved_plain, bw_plain = b.partitioned.saved_bytes, _targets(b.partitioned.bw)
    finally:
        b.__exit__(None, None, None)
    assert saved_wrapped < saved_plain
    assert bw_wrapped.count(apb.mm_nd.default) > bw_plain.count(apb.mm_nd.default)  # first matmul of each region runs again


def test_own_policy_never_overrides_a_user_tag(mesh_1d):
    ctx = functools.partial(create_selective_checkpoint_contexts, _save_matmuls)
    with torch.device("meta"):
        model = Stack(context_fn=ctx)
    ap = _plan(mesh_1d, model, ac="full")
    try:
        low = ap.lower()
        for n in low.gm.graph.nodes:
            if n.target is apb.mm_nd.default and n.meta.get("recompute") is not None:
                assert n.meta.get(MUST_SAVE) and not n.meta.get(RECOMPUTE)
    finally:
        ap.__exit__(None, None, None)


def test_stage_cut_saves_the_narrowest_live_set(mesh_1d):
    from autoparallel_b200.parallel.passes.act_ckpt import _forward_nodes, _nbytes, min_live_memory_cuts

    with torch.device("meta"):
        model = Stack(n=6, wrap=False)
    ap = _plan(mesh_1d, model, ac="full")
    try:
        ap.ac_stage_bytes = 1  # placeholder, replaced below
        low = ap.lower()
        fwd, _ = _forward_nodes(low.joint)
        total = sum(_nbytes(n) for n in fwd)
        cuts = min_live_memory_cuts(fwd, total // 3)
        # three stages -> two cuts, each a single residual-stream tensor (the narrowest point between blocks)
        assert 1 <= len(cuts) <= 4
        widest = max(_nbytes(n) for n in fwd)
        assert all(_nbytes(c) < widest for c in cuts)
        # the cut tensors are saved, everything else of the forward is recomputed
        ap.ac_stage_bytes = total // 3
        low = ap.lower()
        saved = [n for n in low.gm.graph.nodes if n.meta.get(MUST_SAVE)]
        assert saved and all(_nbytes(n) < widest for n in saved)
        smaller = ap.ac_stats["saved"]
        ap.ac_stage_bytes = total // 6
        ap.lower()
        assert ap.ac_stats["saved"] >= smaller  # shorter stages, more boundaries
    finally:
        ap.__exit__(None, None, None)


def _numerics_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    ctx = functools.partial(create_selective_checkpoint_contexts, _save_matmuls)
    results = {}
    for label, kwargs, ac in (("user_sac", dict(context_fn=ctx), "none"), ("user_plain", dict(), "none"), ("own_full", dict(wrap=False), "full")):
        torch.manual_seed(0)
        ref = Stack(n=3, **{**kwargs, "wrap": False, "context_fn": None})
        with torch.device("meta"):
            model = Stack(n=3, **kwargs)
        with AutoParallel(model, lambda: torch.rand(8, 16, 64), mesh, activation_checkpointing=ac) as ap:
            ap.add_parameter_memory_constraint()
            ap.add_input_constraints([(Shard(0),)])
            ap.optimize_placement()
            if ac == "full":
                ap.ac_stage_bytes = 64 * 1024
            pm = ap.apply_placement()
        pm.to_empty(device="cpu")
        from torch.distributed.tensor import distribute_tensor

        with torch.no_grad():
            for (n, p), (_, rp) in zip(pm.named_parameters(), ref.named_parameters()):
                p.copy_(distribute_tensor(rp.detach(), mesh, p.placements))
        torch.manual_seed(1)
        x = torch.rand(8, 16, 64)
        out = pm(x.chunk(ws, 0)[rank])
        out.square().sum().backward()
        ro = ref(x)
        ro.square().sum().backward()
        worst = max(((p.grad.full_tensor() - rp.grad).abs().max() / (rp.grad.abs().max() + 1e-12)).item()
                    for (_, p), (_, rp) in zip(pm.named_parameters(), ref.named_parameters()))
        results[label] = worst
    if rank == 0:
        q.put(results)
    dist.destroy_process_group()


def test_checkpointed_models_give_the_same_gradients_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_numerics_worker, args=(2, free_port(), q), nprocs=2, join=True)
    res = q.get()
    assert set(res) == {"user_sac", "user_plain", "own_full"}
    assert all(v < 1e-5 for v in res.values()), res


def test_compile_backend_turns_checkpointing_on_for_a_module_built_without(mesh_1d):
    import autoparallel_b200
    from autoparallel_b200 import autoparallel_backend

    assert autoparallel_b200.with_sharding_constraint is not None
    with torch.device("meta"):
        model = Stack(n=4, wrap=False)
    ap = _plan(mesh_1d, model)
    try:
        pm = ap.apply_placement()
        before = ap.partitioned.saved_bytes
        backend = autoparallel_backend(enable_ac=True, ac_stage_size_in_GiB=1e-4)
        lin = nn.Linear(8, 8)
        torch.compile(lin, backend=backend, fullgraph=True)(torch.randn(2, 8))  # first call runs the backend
        assert pm.__dict__["_apb200_ac_mode"] == "full"
        assert ap.partitioned.saved_bytes < before
        assert backend.reconfigured and backend.reconfigured[0]["mode"] == "full"
        # a module built with an explicit policy is left alone
        with pytest.raises(ValueError):
            autoparallel_backend(ac_stage_size_in_GiB=-1)
    finally:
        ap.__exit__(None, None, None)
