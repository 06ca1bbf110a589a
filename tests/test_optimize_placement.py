"""Solver outcomes on fake ranks: what plan emerges from which constraints.

Mirrors the expectations of the reference's tests/test_optimize_placement.py:95-300 (FSDP when the
parameter-memory constraint is on, DDP when it allows full replication, Megatron-style tensor
parallelism on a 2-D mesh with a fast inner dim) on this framework's own graph vocabulary.
"""
import pytest
import torch
import torch.nn as nn
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200 import AutoParallel
from autoparallel_b200.parallel.cost import comm, device
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
from autoparallel_b200.parallel.solver.ilp import _out_placements

apb = torch.ops.apb200


class FFN(nn.Module):
    def __init__(self, d=1024, h=4096):
        super().__init__()
        self.up = nn.Linear(d, h, bias=False)
        self.down = nn.Linear(h, d, bias=False)

    def forward(self, x):
        return self.down(torch.relu(self.up(x)))


def _plan(mesh, high, batch=512, seq=128, d=1024, mp=None, topo=None, input_placement=None):
    with torch.device("meta"):
        m = FFN(d, 4 * d)

    def input_fn():
        return torch.randn(batch, seq, d)

    ap = AutoParallel(m, input_fn, mesh, mp_policy=mp, cost_model=topo or "auto", plan_device="B200")
    with ap:
        if high is not None:
            ap.add_parameter_memory_constraint(low=0.0, high=high)
        ap.add_input_constraints([input_placement or ((Shard(0),) + (Replicate(),) * (mesh.ndim - 1))])
        sol = ap.optimize_placement()
        nodes = {n.name: n for n in ap.gm.graph.nodes}
        return ap, sol, nodes


def _by_target(ap, sol, target):
    return [(n, sol[n]) for n in ap.gm.graph.nodes if n.op == "call_function" and n.target is target]


def test_default_memory_constraint_gives_fsdp(mesh_1d):
    ap, sol, _ = _plan(mesh_1d, high=None if False else 1 / 8)
    for p in ap.joint.param_nodes.values():
        assert _out_placements(sol[p]) == (Shard(0),) or _out_placements(sol[p]) == (Shard(1),)
    # forward linears run data-parallel on gathered weights
    fwd_mm = [s for n, s in _by_target(ap, sol, apb.mm_nd.default)][:2]
    for s in fwd_mm:
        assert s.input_specs[0].placements == (Shard(0),)
        assert s.input_specs[1].placements == (Replicate(),)
        assert s.output_specs.placements == (Shard(0),)
    # weight gradients are pending sums that get reduce-scattered onto the parameter's shards
    for n, s in _by_target(ap, sol, apb.mm_wgrad.default):
        assert s.output_specs.placements == (Partial(),)
    for fqn, g in ap.joint.param_grads.items():
        assert _out_placements(sol[g]) == _out_placements(sol[ap.joint.param_nodes[fqn]])


def test_without_memory_pressure_parameters_replicate(mesh_1d):
    ap, sol, _ = _plan(mesh_1d, high=1.0)
    for p in ap.joint.param_nodes.values():
        assert _out_placements(sol[p]) == (Replicate(),)
    for n, s in _by_target(ap, sol, apb.mm_wgrad.default):
        assert s.output_specs.placements == (Partial(),)  # DDP: all-reduce of the gradient follows
    for g in ap.joint.param_grads.values():
        assert _out_placements(sol[g]) == (Replicate(),)


def test_2d_mesh_finds_tensor_parallel_ffn(mesh_2d):
    # small batch per dp rank, large hidden: sharding the FFN weights on the fast inner dim wins
    ap, sol, _ = _plan(mesh_2d, high=1 / 8, batch=2, seq=256, d=2048)
    up, down = list(ap.joint.param_nodes.values())
    pu, pd = _out_placements(sol[up]), _out_placements(sol[down])
    fwd = [s for n, s in _by_target(ap, sol, apb.mm_nd.default)][:2]
    # column-parallel up projection feeds a row-parallel down projection without communication
    assert fwd[0].output_specs.placements[1] == Shard(2)
    assert fwd[1].input_specs[0].placements[1] == Shard(2)
    assert fwd[1].output_specs.placements[1] == Partial()
    assert pu[1] == Shard(0) and pd[1] == Shard(1)


def test_node_constraint_and_resolve(mesh_1d):
    ap, sol, _ = _plan(mesh_1d, high=1.0)
    opt = ap.sharding_optimizer
    p = next(iter(ap.joint.param_nodes.values()))
    with ap.__class__.__enter__.__get__(ap) if False else _reentered(ap):
        pass
    name = opt.add_node_constraint(p, (Shard(0),))
    sol2 = opt.resolve()
    assert _out_placements(sol2[p]) == (Shard(0),)
    diff = opt.diff_solutions(sol)
    assert any(d[0] == p.name for d in diff)
    opt.remove_constraints([name])
    sol3 = opt.resolve()
    assert _out_placements(sol3[p]) == (Replicate(),)


class _reentered:
    def __init__(self, ap):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def test_unavailable_placement_is_rejected(mesh_1d):
    ap, sol, _ = _plan(mesh_1d, high=1.0)
    p = next(iter(ap.joint.param_nodes.values()))
    with pytest.raises(ValueError, match="not available"):
        ap.sharding_optimizer.add_node_constraint(p, (Partial(),))
    with pytest.raises(ValueError):
        ap.sharding_optimizer.add_node_constraint(p, (Shard(0), Shard(1)))  # wrong mesh rank


def test_contradictory_constraints_are_reported(mesh_1d):
    with torch.device("meta"):
        m = FFN(64, 256)
    with AutoParallel(m, lambda: torch.randn(16, 8, 64), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        # the output gradient twin must match the output: pin it differently to make it infeasible
        t = ap.joint.tangent_nodes[0]
        bad = ap.sharding_optimizer.add_node_constraint(t, (Replicate(),))
        with pytest.raises(RuntimeError, match="feasible") as err:
            ap.optimize_placement()
        # the report names the clashing pair (output pinned Shard(0), its gradient pinned Replicate) and
        # leaves the input constraint, which is compatible with either, out of it
        rep = ap.sharding_optimizer.infeasibility_report
        names = {c["name"] for c in rep["conflict"]}
        assert bad in names and len(names) == 2 and any(n.startswith("output:") for n in names)
        assert not any(n.startswith("input:") for n in names)
        assert "conflicting constraints (2 of 3" in str(err.value)
        # removing one member of the reported set is enough
        ap.sharding_optimizer.remove_constraints([bad])
        assert ap.optimize_placement() is not None


def test_mixed_precision_orders_casts_and_collectives(mesh_1d):
    ap, sol, _ = _plan(mesh_1d, high=1 / 8, mp=MPPolicy(torch.bfloat16, torch.float32))
    cast = apb.dtype_cast.default
    params = set(ap.joint.param_nodes.values())
    for n in ap.gm.graph.nodes:
        if n.op == "call_function" and n.target is cast and n.args[0] in params:
            # gather happens after the narrowing cast: the cast itself sees the sharded fp32 parameter
            assert sol[n].input_specs[0].placements == _out_placements(sol[n.args[0]])
            assert sol[n].output_specs.placements == _out_placements(sol[n.args[0]])
    # gradient: pending sum survives the widening cast, the reduction runs in fp32 afterwards
    for fqn, g in ap.joint.param_grads.items():
        chain = g
        while chain.op == "call_function" and chain.target is not cast:
            chain = chain.args[0]
        assert chain.target is cast and chain.args[1] == torch.float32
        assert sol[chain].output_specs.placements == (Partial(),)


def test_clustering_shares_variables_between_layers(mesh_1d):
    from autoparallel_b200 import ForwardInputs
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug

    sizes = {}
    for layers in (2, 6):
        with torch.device("meta"):
            m = Transformer(llama3_debug(n_layers=layers))

        def input_fn():
            return ForwardInputs((torch.randint(0, 1024, (8, 64)),), {"labels": torch.randint(0, 1024, (8, 64))})

        with AutoParallel(m, input_fn, mesh_1d) as ap:
            ap.add_parameter_memory_constraint()
            ap.add_input_constraints([(Shard(0),)] * 2)
            ap.optimize_placement()
            sizes[layers] = ap.sharding_optimizer.problem_size["variables"]
    assert sizes[6] < 1.3 * sizes[2]  # four more layers add almost nothing to the ILP


def test_parameter_budget_in_bytes_decides_between_replication_and_sharding(mesh_1d):
    """The bytes form of the parameter-memory constraint: a generous budget leaves the cheaper replicated
    (data-parallel) plan in place, a budget below the replicated state forces sharded parameters."""
    d = 1024
    n_elems = 2 * d * 4 * d
    replicated_bytes = n_elems * 16.0

    def plan(budget):
        with torch.device("meta"):
            m = FFN(d, 4 * d)
        with AutoParallel(m, lambda: torch.randn(512, 128, d), mesh_1d, plan_device="B200") as ap:
            ap.add_parameter_memory_constraint(budget_bytes=budget, bytes_per_element=16.0)
            ap.add_input_constraints([(Shard(0),)])
            sol = ap.optimize_placement()
            held = 0
            for p in ap.joint.param_nodes.values():
                pl = _out_placements(sol[p])
                held += p.meta["val"].numel() // (8 if any(isinstance(x, Shard) for x in pl) else 1)
            return held * 16.0

    assert plan(2 * replicated_bytes) == replicated_bytes       # budget not binding: replicate
    tight = plan(replicated_bytes / 4)
    assert tight <= replicated_bytes / 4                          # both weights sharded eightfold
    with pytest.raises(RuntimeError, match="feasible"):
        plan(replicated_bytes / 64)                                # below the fully sharded state: no plan
    with torch.device("meta"):
        m = FFN(d, 4 * d)
    with AutoParallel(m, lambda: torch.randn(512, 128, d), mesh_1d, plan_device="B200") as ap:
        with pytest.raises(ValueError, match="either"):
            ap.add_parameter_memory_constraint(high=0.5, budget_bytes=1e9)
