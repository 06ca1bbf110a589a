"""Unit tests of planner pieces: graph canonicalisation, cost models, partitioner, serialization,
JSON export / log / visualizer, simulated metrics."""
import json
import os

import pytest
import torch
import torch.nn as nn
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.parallel.cost import comm, nccl_model
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy

apb = torch.ops.apb200
aten = torch.ops.aten


class Tied(nn.Module):
    def __init__(self, v=128, d=32):
        super().__init__()
        self.emb = nn.Embedding(v, d)
        self.mid = nn.Linear(d, d)
        self.out = nn.Linear(d, v, bias=False)
        self.out.weight = self.emb.weight

    def forward(self, t):
        return self.out(torch.relu(self.mid(self.emb(t))))


def _plan(mesh, model_fn, input_fn, **kw):
    with torch.device("meta"):
        m = model_fn()
    ap = AutoParallel(m, input_fn, mesh, **kw)
    ap.__enter__()
    return ap


def test_linear_patterns_become_nd_ops_and_aliases_are_inserted(mesh_1d):
    ap = _plan(mesh_1d, Tied, lambda: torch.randint(0, 128, (16, 8)))
    try:
        targets = [n.target for n in ap.gm.graph.nodes if n.op == "call_function"]
        assert aten.mm.default not in targets and aten.addmm.default not in targets
        assert targets.count(apb.mm_nd.default) >= 4 and targets.count(apb.mm_wgrad.default) >= 2
        # tied weight = one placeholder whose gradient sums both uses
        assert len(ap.joint.param_nodes) == 3  # emb(=out).weight, mid.weight, mid.bias
        # every multi-consumer tensor and every output goes through a redistribution point
        for n in ap.gm.graph.nodes:
            if n.op == "call_function" and n.target is not aten.alias.default and isinstance(n.meta.get("val"), torch.Tensor):
                assert len(n.users) <= 1 or all(u.target is aten.alias.default for u in n.users)
    finally:
        ap.__exit__(None, None, None)


def test_user_collectives_in_the_model_are_rejected(mesh_1d):
    from autoparallel_b200.parallel.frontend.graph_canon import assert_has_no_collectives
    import torch.fx as fx

    g = fx.Graph()
    x = g.placeholder("x")
    y = g.call_function(torch.ops.apb200_comm.all_reduce.default, (x, "0", 8))
    g.output(y)
    with pytest.raises(RuntimeError, match="local_map"):
        assert_has_no_collectives(fx.GraphModule(nn.Module(), g))


def test_redistribute_cost_semantics(mesh_2d):
    from autoparallel_b200.parallel.strategies.dtensor_adapter import DTensorSpec, tensor_meta_of

    comm.set_topology(comm.Topology([comm.NVLINK5, comm.NVLINK5]))
    try:
        tm = tensor_meta_of(torch.empty(4096, 4096, dtype=torch.bfloat16))
        spec = lambda *pl: DTensorSpec(mesh_2d, pl, tensor_meta=tm)  # noqa: E731
        c = comm.redistribute_cost
        assert c(spec(Shard(0), Replicate()), spec(Shard(0), Replicate())) == 0.0
        assert c(spec(Replicate(), Replicate()), spec(Partial(), Replicate())) == float("inf")
        ag, ar, rs = c(spec(Replicate(), Shard(0)), spec(Replicate(), Replicate())), c(spec(Replicate(), Partial()), spec(Replicate(), Replicate())), c(spec(Replicate(), Partial()), spec(Replicate(), Shard(0)))
        assert 0 < rs <= ag * 1.1 and ar > ag  # all-reduce moves twice the data
        assert c(spec(Replicate(), Replicate()), spec(Replicate(), Shard(0))) < 0.2 * ag  # a local slice is nearly free
        small = DTensorSpec(mesh_2d, (Replicate(), Shard(0)), tensor_meta=tensor_meta_of(torch.empty(64, 64, dtype=torch.bfloat16)))
        rep = DTensorSpec(mesh_2d, (Replicate(), Replicate()), tensor_meta=small.tensor_meta)
        assert c(small, rep) < ag  # monotone in size, latency floor for small messages
        assert c(small, rep) >= comm.NVLINK5.alpha(4)
    finally:
        comm.set_topology(None)


def test_nccl_model_shapes():
    t = nccl_model.b200_topo()
    h = nccl_model.h100_topo()
    for coll in (nccl_model.Coll.ALL_GATHER, nccl_model.Coll.ALL_REDUCE, nccl_model.Coll.REDUCE_SCATTER, nccl_model.Coll.ALL_TO_ALL):
        times = [nccl_model.collective_time_us(coll, s, 8, t) for s in (1 << 16, 1 << 20, 1 << 26, 1 << 30)]
        assert all(a < b for a, b in zip(times, times[1:]))  # monotone in bytes
        assert nccl_model.collective_time_us(coll, 1 << 30, 8, t) < nccl_model.collective_time_us(coll, 1 << 30, 8, h)
    # detection goes by ranks per host, not by device name: an 8-GPU B200 host is one NVSwitch node
    d = nccl_model.detect_topology(8, device_name="NVIDIA B200")
    assert d.gpus_per_node == 8 and d.n_nodes == 1 and d.arch is nccl_model.Arch.BLACKWELL
    two = nccl_model.detect_topology(16, ranks_per_host=8, device_name="NVIDIA H100")
    assert two.n_nodes == 2
    assert nccl_model.collective_time_us(nccl_model.Coll.ALL_REDUCE, 1 << 28, 16, two) > nccl_model.collective_time_us(nccl_model.Coll.ALL_REDUCE, 1 << 28, 8, two)
    assert not nccl_model.eligible(nccl_model.Algo.TREE, nccl_model.Coll.ALL_GATHER, t, 8)
    assert nccl_model.eligible(nccl_model.Algo.NVLS, nccl_model.Coll.ALL_REDUCE, t, 8)
    assert not nccl_model.eligible(nccl_model.Algo.NVLS, nccl_model.Coll.ALL_REDUCE, nccl_model.a100_topo(), 8)


def test_partitioner_saves_or_recomputes_by_tag(mesh_1d):
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug
    from autoparallel_b200.parallel.lower.partition import partition_joint

    cfg = llama3_debug()

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (8, 64)),), {"labels": torch.randint(0, cfg.vocab_size, (8, 64))})

    saved = {}
    for mode in ("none", "selective", "full"):
        ap = _plan(mesh_1d, lambda: Transformer(cfg), input_fn, activation_checkpointing=mode, mp_policy=MPPolicy(torch.bfloat16, torch.float32))
        try:
            ap.add_parameter_memory_constraint()
            ap.add_input_constraints([(Shard(0),)] * 2)
            ap.optimize_placement()
            low = ap.lower()
            parts = partition_joint(low.joint)
            saved[mode] = parts.saved_bytes
            # gathered parameters are never saved: the gather chain is recomputed in backward
            for n in parts.fw.graph.nodes:
                if n.op == "output":
                    outs = n.args[0][parts.num_fwd_outputs:]
                    for o in outs:
                        cur = o
                        while cur.op == "call_function" and len(cur.all_input_nodes) == 1:
                            cur = cur.all_input_nodes[0]
                        from_param = cur.op == "placeholder" and cur.meta.get("apb200_kind", ("",))[0] == "param"
                        assert not (from_param and o is not cur), f"{o.name} (derived from a parameter) is saved"
        finally:
            ap.__exit__(None, None, None)
    assert saved["full"] < saved["selective"] < saved["none"]


def test_save_load_json_log_html_and_metrics(mesh_1d, tmp_path):
    from autoparallel_b200.parallel.solver.ilp import ShardingOptimizer
    from autoparallel_b200.utils.trace_sim import create_execution_trace, estimate_graph_metrics
    from autoparallel_b200.utils.visualizer import generate_visualization_html

    ap = _plan(mesh_1d, Tied, lambda: torch.randint(0, 128, (16, 8)))
    try:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        opt = ap.sharding_optimizer
        log = opt.get_log(verbose=True)
        assert "total: compute" in log and "mm_nd" in log
        assert "local cost" in opt.explain_placement(next(iter(ap.joint.param_nodes.values())))
        plan = opt.get_json()
        json.dumps(plan)
        assert plan["mesh"]["shape"] == [8] and {n["phase"] for n in plan["nodes"]} == {"forward", "backward"}
        html = generate_visualization_html(plan)
        assert "<table" in html and "id=treemap" in html
        # the three views the reference's report has: module treemap, parameter tree, simulated-step timeline
        from autoparallel_b200.utils.visualizer import module_tree, parameter_tree, write_report

        mt = module_tree(plan["nodes"])
        assert mt["name"] == "model" and mt["children"] and abs(mt["compute"] - plan["summary"]["compute_us"]) < 1e-3 * max(1, mt["compute"])
        pt = parameter_tree(plan["nodes"], plan["mesh"]["shape"])
        assert pt["count"] == len(ap.joint.param_nodes) and 0 < pt["local_bytes"] <= pt["bytes"]
        low = ap.lower()
        report = write_report(str(tmp_path / "plan.html"), opt, low.gm, ap.mesh)
        doc = open(report).read()
        for marker in ("id=modules", "id=parameters", "id=timeline", "drawTreemap", "traceEvents", "download Chrome-trace JSON"):
            assert marker in doc, marker
        embedded = json.loads(doc.split("const DATA=", 1)[1].split(";\nfunction show", 1)[0])
        assert embedded["trace"]["traceEvents"] and embedded["modules"]["n"] == len(plan["nodes"])
        p1, p2 = str(tmp_path / "opt.pt"), str(tmp_path / "pl.json")
        opt.save(p1)
        opt.save_placements(p2)
        loaded = ShardingOptimizer.load(p1)
        assert abs(loaded.total_cost() - opt.objective_value) < 1e-6 * max(1.0, abs(opt.objective_value))
        saved_obj = loaded.objective_value
        loaded.resolve()  # same constraints, layers no longer tied together: never worse than the saved optimum
        assert loaded.objective_value <= saved_obj * (1 + 1e-6) + 1e-6
        some_param = next(iter(ap.joint.param_nodes.values())).name
        pinned = loaded.resolve({some_param: "R"})
        assert pinned[some_param] == "R"
        sol = opt.load_placements(p2)
        assert len(sol) == len(opt.nodes)
        bad = json.load(open(p2))
        bad["mesh_shape"] = [4]
        json.dump(bad, open(p2, "w"))
        with pytest.raises(ValueError, match="mesh"):
            opt.load_placements(p2)
        low = ap.lower()
        m = estimate_graph_metrics(low.gm, mesh_1d)
        assert m.total_us > 0 and m.num_collectives > 0 and m.exposed_comm_us <= m.comm_us + 1e-6 and m.peak_bytes > 0
        tr = create_execution_trace(low.gm, mesh_1d, str(tmp_path / "trace.json"))
        assert os.path.exists(tmp_path / "trace.json") and len(tr["traceEvents"]) > 0
    finally:
        ap.__exit__(None, None, None)


def test_overlap_schedule_prefetches_and_defers(mesh_1d):
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug
    from autoparallel_b200.parallel.lower.partition import partition_joint
    from autoparallel_b200.parallel.passes.overlap import exposed_collectives, schedule_for_streams
    from autoparallel_b200.runtime import comm_ops

    cfg = llama3_debug(n_layers=3)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (8, 64)),), {"labels": torch.randint(0, cfg.vocab_size, (8, 64))})

    ap = _plan(mesh_1d, lambda: Transformer(cfg), input_fn, fuse_collectives=False)
    try:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)] * 2)
        ap.optimize_placement()
        parts = partition_joint(ap.lower().joint)
        fw = schedule_for_streams(parts.fw, mesh_1d)
        nodes = list(fw.graph.nodes)
        starts = [i for i, n in enumerate(nodes) if n.target is comm_ops.ops.all_gather_start.default]
        waits = {n.args[0]: i for i, n in enumerate(nodes) if n.target is comm_ops.ops.comm_wait.default}
        gaps = [waits[nodes[i]] - i for i in starts if nodes[i] in waits]
        assert max(gaps) > 5  # gathers are issued well ahead of their first use
        assert exposed_collectives(fw) < len(starts)
        bw = schedule_for_streams(parts.bw, mesh_1d)
        bn = list(bw.graph.nodes)
        rs = [i for i, n in enumerate(bn) if n.target is comm_ops.ops.reduce_scatter_start.default]
        rs_waits = {n.args[0]: i for i, n in enumerate(bn) if n.target is comm_ops.ops.comm_wait.default}
        assert any(rs_waits[bn[i]] - i > 3 for i in rs)  # gradient reductions overlap later compute
        # and they are spread through the backward, not bunched at its end: the longest stretch of compute without a
        # reduction being issued is a fraction of the graph (about one layer)
        from autoparallel_b200.parallel.passes.overlap import max_compute_run_between_reductions

        n_compute = sum(1 for n in bn if n.op == "call_function")
        assert 0 < max_compute_run_between_reductions(bw) < n_compute // 2
        assert max_compute_run_between_reductions(fw) > 0
        # every split-phase collective is consumed through its wait, never directly, and none is left un-waited
        for gm_ in (fw, bw):
            for n in gm_.graph.nodes:
                if n.op == "call_function" and n.target in comm_ops.START_OPS:
                    assert n.users and all(u.target is comm_ops.ops.comm_wait.default for u in n.users), n.name
    finally:
        ap.__exit__(None, None, None)


def test_reductions_whose_results_are_added_up_are_not_deferred_as_a_unit(mesh_1d):
    """A parameter used three times (a tied embedding) gets three reduced gradients that are added on their way out.  The
    scheduler may defer a reduction together with its tail only when that tail is a unary chain; here every node must still
    be scheduled exactly once."""
    import torch.nn as nn

    from autoparallel_b200.parallel.lower.partition import partition_joint
    from autoparallel_b200.parallel.passes.overlap import schedule_for_streams

    class Tied3(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(64, 32)
            self.mid = nn.Linear(32, 32)

        def forward(self, a, b):
            h = self.mid(self.emb(a) + self.emb(b))
            return h @ self.emb.weight.t()

    with torch.device("meta"):
        m = Tied3()
    with AutoParallel(m, lambda: (torch.randint(0, 64, (16, 8)), torch.randint(0, 64, (16, 8))), mesh_1d) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)] * 2)
        ap.optimize_placement()
        parts = partition_joint(ap.lower().joint)
        for gm_ in (parts.fw, parts.bw):
            n_before = sum(1 for n in gm_.graph.nodes if n.op == "call_function")
            sched = schedule_for_streams(gm_, mesh_1d)
            n_after = sum(1 for n in sched.graph.nodes if n.op == "call_function")
            assert n_after >= n_before  # (split collectives add their waits; nothing is lost or doubled beyond that)
            sched.graph.lint()
