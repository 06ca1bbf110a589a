"""Forward-only extraction (the inference path), simulated graph metrics and reduction strategies.
(Reference behaviours restated on this framework's API: tests/test_inference_path.py, tests/test_estimate_graph_metrics.py,
tests/test_reduction_strategies.py.)"""
import copy

import pytest
import torch
import torch.fx as fx
import torch.nn as nn
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200 import AutoParallel
from autoparallel_b200.parallel.lower.partition import extract_forward, partition_joint
from autoparallel_b200.runtime import comm_ops
from autoparallel_b200.utils.trace_sim import GraphMetrics, create_execution_trace, estimate_graph_metrics, simulate

C = comm_ops.ops


class Linear2(nn.Module):
    def __init__(self, d=64):
        super().__init__()
        self.a = nn.Linear(d, d, bias=False)
        self.b = nn.Linear(d, d, bias=False)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


class TwoOutputs(nn.Module):
    def __init__(self, d=64):
        super().__init__()
        self.a = nn.Linear(d, d, bias=False)
        self.b = nn.Linear(d, d, bias=False)

    def forward(self, x):
        h = self.a(x)
        return h, self.b(torch.relu(h))


def _plan(model_cls, mesh, n_out=1, **kw):
    with torch.device("meta"):
        m = model_cls()
    ap = AutoParallel(m, lambda: torch.randn(32, 64), mesh, **kw)
    ap.__enter__()
    ap.add_parameter_memory_constraint()
    ap.add_input_constraints([(Shard(0),)])
    ap.add_output_constraints([(Shard(0),)] * n_out)
    ap.optimize_placement()
    return ap


# ---------------------------------------------------------------------------------------------- forward extraction
def test_forward_graph_has_no_tangents_fewer_nodes_and_leaves_the_joint_alone(mesh_1d):
    ap = _plan(Linear2, mesh_1d)
    try:
        low = ap.lower()
        joint = low.joint
        assert len(joint.tangent_nodes) > 0
        before = [(n.op, str(n.target)) for n in joint.gm.graph.nodes]
        fwd = extract_forward(joint)
        names = {n.name for n in fwd.graph.nodes if n.op == "placeholder"}
        assert not any(t.name in names for t in joint.tangent_nodes)
        out = next(n for n in fwd.graph.nodes if n.op == "output")
        assert len(out.args[0]) == joint.num_fwd_outputs == 1
        assert len(list(fwd.graph.nodes)) < len(before)
        # no backward operator survives and the joint graph was not edited
        assert not any(n.op == "call_function" and n.target is torch.ops.apb200.mm_wgrad.default for n in fwd.graph.nodes)
        assert [(n.op, str(n.target)) for n in joint.gm.graph.nodes] == before
    finally:
        ap.__exit__(None, None, None)


def test_forward_graph_of_a_two_output_model(mesh_1d):
    ap = _plan(TwoOutputs, mesh_1d, n_out=2)
    try:
        low = ap.lower()
        fwd = extract_forward(low.joint)
        out = next(n for n in fwd.graph.nodes if n.op == "output")
        assert len(out.args[0]) == 2
    finally:
        ap.__exit__(None, None, None)


def test_inference_equals_training_forward_and_carries_no_graph(mesh_1d):
    ap = _plan(TwoOutputs, mesh_1d, n_out=2)
    try:
        pm = ap.apply_placement()
    finally:
        ap.__exit__(None, None, None)
    pm.to_empty(device="cpu")
    with torch.no_grad():
        for p in pm.parameters():
            p.to_local().normal_(std=0.1)
    x = torch.randn(32 // mesh_1d.size(0), 64)
    h_t, y_t = pm(x)
    assert y_t.requires_grad
    with torch.no_grad():
        h_i, y_i = pm(x)
    assert not y_i.requires_grad and y_i.grad_fn is None
    assert torch.equal(h_i, h_t.detach()) and torch.equal(y_i, y_t.detach())


# ---------------------------------------------------------------------------------------------- simulated metrics
def _compute_graph(n):
    g = fx.Graph()
    x = g.placeholder("x")
    x.meta["val"] = torch.empty(1024, 1024)
    cur = x
    for _ in range(n):
        cur = g.call_function(torch.ops.aten.relu.default, (cur,))
        cur.meta["val"] = torch.empty(1024, 1024)
    g.output((cur,))
    return fx.GraphModule(nn.Module(), g)


def test_compute_only_graph_has_no_communication_and_time_accumulates(mesh_1d):
    one = estimate_graph_metrics(_compute_graph(1), mesh_1d, "B200")
    five = estimate_graph_metrics(_compute_graph(5), mesh_1d, "B200")
    assert isinstance(one, GraphMetrics)
    assert one.comm_us == 0 and one.exposed_comm_us == 0 and one.num_collectives == 0
    assert one.compute_us > 0 and five.compute_us == pytest.approx(5 * one.compute_us)
    assert five.total_us > one.total_us
    # the same graph gives the same numbers
    again = estimate_graph_metrics(_compute_graph(5), mesh_1d, "B200")
    assert again == five
    # one relu output + its input alive at a time
    assert five.peak_bytes >= 2 * 1024 * 1024 * 4


def test_metrics_of_a_planned_model_training_vs_inference_and_layers(mesh_1d):
    ap = _plan(Linear2, mesh_1d)
    try:
        low = ap.lower()
        parts = partition_joint(low.joint)
        fw = estimate_graph_metrics(parts.fw, mesh_1d, "B200")
        bw = estimate_graph_metrics(parts.bw, mesh_1d, "B200")
        inf = estimate_graph_metrics(extract_forward(low.joint), mesh_1d, "B200")
        # FSDP: parameters are gathered in forward and gradients reduced in backward - communication is guaranteed
        assert fw.num_collectives >= 1 and fw.comm_us > 0
        assert bw.num_collectives >= 1 and bw.comm_us > 0
        assert fw.total_us + bw.total_us > inf.total_us
        assert inf.compute_us <= fw.compute_us + 1e-9
        trace = create_execution_trace(parts.fw, mesh_1d, None, "B200")
        tids = {e["tid"] for e in trace["traceEvents"]}
        assert 0 in tids and any(str(t).startswith("group-") for t in tids)  # a compute lane and one lane per process group
        assert trace["metadata"]["num_collectives"] == fw.num_collectives
    finally:
        ap.__exit__(None, None, None)


def test_sharded_and_replicated_parameter_plans_differ_in_their_collectives(mesh_1d):
    """The default budget shards parameters (gathers in forward, gradient reduce-scatters); a budget that forces every
    rank to hold every parameter makes it data parallel: no parameter gather, gradients all-reduced."""
    with torch.device("meta"):
        m1, m2 = Linear2(), Linear2()

    def plan(m, **kw):
        # a batch large enough that recomputing it on every rank is no alternative to reducing the gradients
        with AutoParallel(m, lambda: torch.randn(65536, 64), mesh_1d) as ap:
            ap.add_parameter_memory_constraint(**kw)
            ap.add_input_constraints([(Shard(0),)])
            ap.add_output_constraints([(Shard(0),)])
            ap.optimize_placement()
            low = ap.lower()
            params = [ap.sharding_optimizer.placement_of(n) for n in ap.joint.param_nodes.values()] \
                if hasattr(ap.sharding_optimizer, "placement_of") else None
            return dict(low.num_collectives), params

    fsdp, _ = plan(m1)
    ddp, _ = plan(m2, low=1.0, high=1.0)
    assert fsdp["all_gather"] >= 2 and fsdp["reduce_scatter"] >= 2 and fsdp["all_reduce"] == 0
    assert ddp["all_reduce"] >= 2 and ddp["reduce_scatter"] == 0 and ddp["all_gather"] == 0


# ---------------------------------------------------------------------------------------------- reductions
class Reductions(nn.Module):
    def forward(self, x):
        return x.sum(dim=1), x.mean(dim=0), x.sum()


def test_reduction_strategies_partial_over_reduced_dims_and_shard_elsewhere(mesh_2d):
    with torch.device("meta"):
        m = Reductions()
    with AutoParallel(m, lambda: torch.randn(1024, 2048, 64), mesh_2d) as ap:
        opt = ap.sharding_optimizer
        sums = [n for n in ap.joint.gm.graph.nodes if n.op == "call_function" and n.target in
                (torch.ops.aten.sum.dim_IntList, torch.ops.aten.mean.dim, torch.ops.aten.sum.default)]
        assert len(sums) >= 3
        s_dim1 = next(n for n in sums if n.target is torch.ops.aten.sum.dim_IntList and list(n.args[1]) == [1])
        seen = {(s.input_specs[0].placements, s.output_specs.placements) for s in opt.strats[s_dim1].strategies}
        # sharding the reduced dim gives partial sums; a dim that survives keeps its shard (renumbered after the reduction)
        assert any(i[0] == Shard(1) and isinstance(o[0], Partial) for i, o in seen)
        assert any(i[0] == Shard(0) and o[0] == Shard(0) for i, o in seen)
        assert any(i[0] == Shard(2) and o[0] == Shard(1) for i, o in seen)
        # mixed: one mesh dim on the reduced dim, the other on a surviving one
        assert any(i == (Shard(1), Shard(0)) and isinstance(o[0], Partial) and o[1] == Shard(0) for i, o in seen)
        full = next(n for n in sums if n.target is torch.ops.aten.sum.default
                    or (n.target is torch.ops.aten.sum.dim_IntList and len(n.args[1]) == 3))
        seen_full = {(s.input_specs[0].placements, s.output_specs.placements) for s in opt.strats[full].strategies}
        assert any(isinstance(o[0], Partial) and isinstance(o[1], Partial) for i, o in seen_full)
        ap.add_input_constraints([(Shard(0), Shard(1))])
        ap.add_output_constraints([(Shard(0), Replicate()), (Replicate(), Replicate()), (Replicate(), Replicate())])
        ap.optimize_placement()
        low = ap.lower()
        # partial sums are completed by reductions, never by gathering the operand first
        assert low.num_collectives["all_reduce"] + low.num_collectives["reduce_scatter"] >= 2


class MeanLoss(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(64, 64)

    def forward(self, x):
        y = self.lin(x)
        return y.mean() + y.mean(dim=0).square().mean()


def test_mean_over_a_sharded_dim_is_a_partial_sum_not_a_gather(mesh_1d):
    """``loss = out.mean()`` on batch-sharded activations: the mean is planned as a sum with partial results and a
    scalar-sized all-reduce; no activation is gathered."""
    with torch.device("meta"):
        m = MeanLoss()
    with AutoParallel(m, lambda: torch.randn(65536, 64), mesh_1d) as ap:
        assert not any(n.op == "call_function" and n.target in (torch.ops.aten.mean.default, torch.ops.aten.mean.dim)
                       for n in ap.joint.gm.graph.nodes)
        ap.add_parameter_memory_constraint(low=1.0, high=1.0)
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        low = ap.lower()
        gathered = [n for n in low.gm.graph.nodes if n.op == "call_function" and n.target is C.all_gather.default]
        # nothing of the size of the activations moves
        assert all(n.meta["val"].numel() <= 64 * 64 for n in gathered)
        assert low.num_collectives["all_reduce"] >= 2


def test_mean_rewrite_keeps_values_and_gradients():
    from autoparallel_b200.parallel.frontend.graph_canon import rewrite_means_as_scaled_sums
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(x):
        return x.mean(), x.mean(dim=1, keepdim=True), x.mean(dim=(0, 2))

    x = torch.randn(4, 6, 5, dtype=torch.float64)
    gm = make_fx(f)(x)
    for n in gm.graph.nodes:  # the pass reads shapes from the nodes' metadata
        if "val" not in n.meta and "tensor_meta" in n.meta:
            n.meta["val"] = torch.empty(n.meta["tensor_meta"].shape, dtype=n.meta["tensor_meta"].dtype)
    assert rewrite_means_as_scaled_sums(gm) == 3
    a, b, c = gm(x)
    ra, rb, rc = f(x)
    assert torch.allclose(a, ra) and torch.allclose(b, rb) and torch.allclose(c, rc) and b.shape == rb.shape
