"""Auxiliary subsystems on CPU: debug interpreter and numerics log, measured collective tables, bucketing and
cast-fusion passes, activation-checkpoint tagging, compile backend, permutation helper, overlap simulator."""
import json
import os

import pytest
import torch
import torch.fx as fx
import torch.nn as nn
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy

apb = torch.ops.apb200


def _llama(mesh, n_layers=2, **kw):
    from autoparallel_b200.models.llama3 import Transformer, llama3_debug

    cfg = llama3_debug(n_layers=n_layers)
    with torch.device("meta"):
        m = Transformer(cfg)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (8, 64)),), {"labels": torch.randint(0, cfg.vocab_size, (8, 64))})

    ap = AutoParallel(m, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), **kw)
    ap.__enter__()
    ap.add_parameter_memory_constraint()
    ap.add_input_constraints([(Shard(0),)] * 2)
    ap.optimize_placement()
    return ap


def test_debug_interpreter_hashes_and_flags_non_finite(tmp_path):
    from autoparallel_b200.utils.debug import DebugInterpreter, NumericsLogger, tensor_hash

    class M(nn.Module):
        def forward(self, x):
            return torch.log(x) * 2.0

    gm = fx.symbolic_trace(M())
    x = torch.rand(4, 4) + 0.5
    a = DebugInterpreter(gm)
    a.run(x)
    b = DebugInterpreter(gm)
    b.run(x.clone())
    assert [r["hash"] for r in a.records] == [r["hash"] for r in b.records] and len(a.records) == 2
    assert tensor_hash(x) != tensor_hash(x + 1)
    with pytest.raises(FloatingPointError, match="log"):
        DebugInterpreter(gm).run(-x)
    la, lb = NumericsLogger(str(tmp_path), "a"), NumericsLogger(str(tmp_path), "b")
    la.log_records(a.records, "fwd")
    c = DebugInterpreter(gm)
    c.run(x * 1.5)
    lb.log_records(c.records, "fwd")
    assert NumericsLogger.diff(la.dir, lb.dir, "fwd") == [r["node"] for r in a.records]
    lin = nn.Linear(3, 3)
    la.log_weights(lin)
    lb.log_weights(lin)
    assert NumericsLogger.diff(la.dir, lb.dir, "weights") == []
    la.log_scalar("loss", 0, 1.25)
    assert json.loads(open(la.dir + "/scalars.jsonl").read())["value"] == 1.25


def test_measured_collective_table_replaces_the_link_model(tmp_path):
    from autoparallel_b200.parallel.cost import comm

    topo = comm.Topology([comm.NVLINK5])
    model = topo.all_gather(0, 8, 1 << 24)
    path = tmp_path / "table.json"
    path.write_text(json.dumps({"collectives": {"all_gather": {"8": [[1 << 20, 50.0], [1 << 24, 400.0], [1 << 28, 6400.0]]}}}))
    topo.load_table(str(path))
    assert topo.all_gather(0, 8, 1 << 24) == pytest.approx(400.0) and model != pytest.approx(400.0)
    assert 50.0 < topo.all_gather(0, 8, 1 << 22) < 400.0  # interpolated between measured sizes
    assert topo.all_gather(0, 8, 1 << 29) == pytest.approx(12800.0)  # extrapolated at the last measured bandwidth
    assert topo.all_gather(0, 8, 1 << 10) == pytest.approx(50.0)  # latency floor = smallest measured message
    assert topo.reduce_scatter(0, 8, 1 << 24) > 0  # kinds without a table keep the model


def test_bucketing_groups_small_parameter_collectives(mesh_1d):
    from autoparallel_b200.runtime import comm_ops

    ap = _llama(mesh_1d, fuse_collectives=False)
    try:
        plain = ap.lower()
        n_ag = sum(1 for n in plain.gm.graph.nodes if n.target is comm_ops.ops.all_gather.default)
    finally:
        ap.__exit__(None, None, None)
    ap = _llama(mesh_1d, fuse_collectives=False, bucket_collectives=True)
    try:
        low = ap.lower()
        assert ap.bucket_stats["all_gather_buckets"] >= 1 and ap.bucket_stats["members"] >= 2
        n_ag_b = sum(1 for n in low.gm.graph.nodes if n.target is comm_ops.ops.all_gather.default)
        assert n_ag_b < n_ag  # the norm weights of a layer travel in one collective
        low.gm.graph.lint()
    finally:
        ap.__exit__(None, None, None)


def test_cast_fusion_and_recompute_tags(mesh_1d):
    from autoparallel_b200.parallel.passes.act_ckpt import fsdp_all_gather_chains

    ap = _llama(mesh_1d, activation_checkpointing="selective", fuse_collectives=False)
    try:
        low = ap.lower()
        # GEMMs produce the consumer's dtype directly: no dtype_cast hangs off a GEMM output
        for n in low.gm.graph.nodes:
            if n.op == "call_function" and n.target in (apb.mm_nd.default, apb.mm_wgrad.default):
                assert not any(u.target is apb.dtype_cast.default for u in n.users)
        from autoparallel_b200.parallel.passes.act_ckpt import RECOMPUTE

        chains = fsdp_all_gather_chains(low.joint)
        assert len(chains) >= 7 * 2  # the seven projections of each layer are gathered where they are used
        # gathered parameters are recomputed in backward, never saved
        assert all(n.meta.get(RECOMPUTE) for c in chains for n in c)
    finally:
        ap.__exit__(None, None, None)


def test_compile_backend_returns_runnable_graph():
    from autoparallel_b200.compile import autoparallel_backend

    backend = autoparallel_backend(enable_ac=True, ac_stage_size_in_GiB=1.5)
    assert backend.enable_ac and backend.ac_stage_size_in_GiB == 1.5
    lin = nn.Linear(8, 8)
    compiled = torch.compile(lin, backend=backend, fullgraph=True)
    x = torch.randn(4, 8)
    assert torch.allclose(compiled(x), lin(x), atol=1e-6)


def test_permutation_helper():
    from autoparallel_b200.user_ops import permutation

    g = torch.Generator().manual_seed(0)
    p = permutation(17, generator=g)
    assert sorted(p.tolist()) == list(range(17)) and p.dtype == torch.int64
    pb = permutation(9, generator=g, independent=True, batch=5)
    assert pb.shape == (5, 9) and all(sorted(r.tolist()) == list(range(9)) for r in pb)
    assert len({tuple(r.tolist()) for r in pb}) > 1


def test_overlap_simulator_cli(fake_world, tmp_path, capsys):
    from autoparallel_b200.tools import overlap_simulator

    trace = tmp_path / "trace.json"
    overlap_simulator.main(["--model", "llama3_debug", "--mesh", "8", "--layers", "2", "--seq-len", "64", "--trace", str(trace)])
    out = capsys.readouterr().out
    report = json.loads(out)
    assert report["plan"]["collectives"]["all_gather"] > 0 and "exposed_collectives_after" in json.dumps(report)
    assert (tmp_path / "trace_fw.json").exists() or any(p.name.startswith("trace_") for p in tmp_path.iterdir())


def test_shipped_measured_table_changes_the_prices(mesh_1d):
    from autoparallel_b200.parallel.cost import comm

    path = comm.Topology.measured_table_path("B200", "nccl")
    assert path is not None and comm.Topology.measured_table_path("B200", "symm") is not None
    model = comm.Topology([comm.NVLINK5])
    measured = comm.Topology([comm.NVLINK5])
    measured.load_table(path)
    for n in (2, 4, 8):
        a, b = model.all_gather(0, n, 1 << 26), measured.all_gather(0, n, 1 << 26)
        assert b > 0 and 0.2 < a / b < 5  # same order of magnitude as the link model, but not the same number
        assert measured.reduce_scatter(0, n, 1 << 28) > measured.reduce_scatter(0, n, 1 << 24)
    ap = _llama(mesh_1d, plan_device="B200", cost_model="measured")
    try:
        assert ap.sharding_optimizer.objective_value > 0
    finally:
        ap.__exit__(None, None, None)


def test_estimate_against_measurement_helpers(mesh_1d):
    """benchmark_strategy_runtime_cost / compare_estimated_with_benchmarked_throughput run the nodes with their local shapes."""
    from autoparallel_b200.parallel.cost.compute import benchmark_strategy_runtime_cost, compare_estimated_with_benchmarked_throughput

    ap = _llama(mesh_1d)
    try:
        sol = ap.optimize_placement()
        data = compare_estimated_with_benchmarked_throughput(ap.gm.graph, sol, device=torch.device("cpu"))
        assert len(data) >= 7
        for node, (real_us, est_us, tflops, peak, eff) in data.items():
            assert node.target in (apb.mm_nd.default, apb.mm_wgrad.default)
            assert real_us > 0 and est_us > 0 and tflops > 0 and peak > 0 and eff == tflops / peak
        norm = next(n for n in ap.gm.graph.nodes if n.target is apb.rms_norm.default)
        assert benchmark_strategy_runtime_cost(norm, sol[norm], torch.device("cpu")) > 0
        view = next(n for n in ap.gm.graph.nodes if n.op == "call_function" and "view" in str(n.target))
        assert benchmark_strategy_runtime_cost(view, sol[view], torch.device("cpu")) == 0.0
    finally:
        ap.__exit__(None, None, None)


def test_structured_trace_artifacts(mesh_1d, tmp_path, monkeypatch):
    """With a structured trace being written, planning dumps the four artifacts under the reference's names."""
    import torch._logging._internal as tl

    seen = {}

    def fake(name, metadata_fn=None, payload_fn=None, **kw):
        md = metadata_fn() if metadata_fn else {}
        seen[md.get("name")] = (md.get("encoding"), payload_fn())

    import autoparallel_b200.api as api_mod

    monkeypatch.setattr("torch._logging.trace_structured", fake)
    ap = _llama(mesh_1d)
    try:
        ap.lower()
    finally:
        ap.__exit__(None, None, None)
    assert set(seen) >= {"autoparallel_joint_graph", "autoparallel_sharding_optimizer_log", "autoparallel_solution",
                         "autoparallel_parallel_graph"}
    assert seen["autoparallel_solution"][0] == "json" and json.loads(seen["autoparallel_solution"][1])
    assert "apb200.mm_nd" in seen["autoparallel_joint_graph"][1] and "apb200_comm" in seen["autoparallel_parallel_graph"][1]


def test_overlap_simulator_replays_a_capture_with_a_measured_table(fake_world, tmp_path, capsys):
    """A saved per-rank graph is simulated again without model or process group, priced by a measured table in the
    reference's text format."""
    from autoparallel_b200.tools import overlap_simulator
    from autoparallel_b200.tools.graph_capture import load_capture, load_colls_table

    cap = tmp_path / "step.capture.json"
    overlap_simulator.main(["--model", "llama3_debug", "--mesh", "8", "--layers", "2", "--seq-len", "64", "--save-capture", str(cap)])
    live = json.loads(capsys.readouterr().out)
    doc = load_capture(str(cap))
    assert doc["mesh_shape"] == [8] and len(doc["group_dim"]) == 1
    n_coll = sum(1 for d in doc["forward"] if "apb200_comm" in d["target"])
    assert n_coll == sum(live["plan"]["collectives"].values()) or n_coll > 0
    table = tmp_path / "colls.table"
    table.write_text(
        "  Group    Group Size  Collective                    1MB (ms)    64MB (ms)    1024MB (ms)\n"
        "-------  ------------  --------------------------  ----------  -----------  -------------\n"
        "      0             8  all_gather_into_tensor          0.0495       1.3371        20.9105\n"
        "      0             8  reduce_scatter_tensor           0.0173       0.1953         2.6420\n"
        "      0             8  all_reduce                      0.0280       0.3822         5.2756\n")
    t = load_colls_table(str(table))
    assert t[("all_gather", 8)][0] == (8 * 2**20, 49.5) and t[("reduce_scatter", 8)][1] == (64 * 2**20, 195.3)
    rep = overlap_simulator.main(["--replay", str(cap), "--table", str(table)])
    capsys.readouterr()
    assert rep["forward"]["after"]["num_collectives"] == live["forward"]["after"]["num_collectives"]
    assert rep["step_ms_after"] > 0
    # a slower table makes the replayed step slower: the table really prices the collectives
    slow = tmp_path / "slow.table"
    slow.write_text(table.read_text().replace("0.0495", "9.0495").replace("0.0173", "9.0173").replace("0.0280", "9.0280"))
    rep2 = overlap_simulator.main(["--replay", str(cap), "--table", str(slow)])
    capsys.readouterr()
    assert rep2["forward"]["before"]["comm_us"] > rep["forward"]["before"]["comm_us"]


def test_simulated_llama3_8b_step_is_close_to_the_measured_one():
    """The cost model prices the kernels it plans for: the simulated Llama-3 8B step (forward + backward graphs after
    the overlap scheduler + a bandwidth-bound AdamW pass) against the step measured on a B200
    (profiles/bench_llama3_8b_reference_vs_own_n1.txt: 418.8 ms in kernels, 445.6 ms per step with eager launches).
    Idle time between launches is not modelled, so the simulation sits below the measurement."""
    import subprocess
    import sys

    # its own process: the tool creates a one-rank fake process group, the suite's fixtures own another
    out = subprocess.run([sys.executable, "-m", "autoparallel_b200.tools.overlap_simulator", "--model", "llama3_8b", "--mesh", "1",
                          "--ac", "selective"], capture_output=True, text=True, timeout=900,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stderr[-2000:]
    rep = json.loads(out.stdout[out.stdout.index("{"):])
    assert abs(rep["kernel_ms"] - 418.8) / 418.8 < 0.10, rep["kernel_ms"]
    assert abs(rep["step_ms_after"] - 445.6) / 445.6 < 0.15, rep["step_ms_after"]
    assert rep["step_ms_after"] <= 445.6
    # AdamW over 8.03e9 fp32 parameters with a bf16 copy: measured 39.9 ms
    assert abs(rep["optimizer_us"] / 1e3 - 39.9) / 39.9 < 0.15


# ---------------------------------------------------------------------------------------------------------------
# cost-driven bucket plan (reference behaviours: tests/test_auto_bucketing_patches.py - merge within caps, split on
# bytes, split on span, skip what depends on a member - restated for the priced planner)
# ---------------------------------------------------------------------------------------------------------------
def _gather_chain_graph(sizes, compute_between=1, group="g0", n_ranks=4, lead=0):
    """placeholders p_i -> all_gather(p_i) -> relu-consumer chain; ``compute_between`` compute nodes before each use,
    ``lead`` compute nodes in front of everything."""
    import torch.fx as fx

    from autoparallel_b200.runtime import comm_ops

    C = comm_ops.ops
    g = fx.Graph()
    x = g.placeholder("x")
    x.meta["val"] = torch.empty(1024, 1024)
    ps = []
    for i, sz in enumerate(sizes):
        p = g.placeholder(f"p{i}")
        p.meta["val"] = torch.empty(sz // n_ranks, dtype=torch.float32)
        ps.append(p)
    cur = x
    for _ in range(lead):
        cur = g.call_function(torch.ops.aten.relu.default, (cur,))
        cur.meta["val"] = torch.empty(1024, 1024)
    gathers = []
    for i, p in enumerate(ps):
        ag = g.call_function(C.all_gather.default, (p, 0, group, n_ranks))
        ag.meta["val"] = torch.empty(sizes[i], dtype=torch.float32)
        gathers.append(ag)
        for _ in range(compute_between):
            cur = g.call_function(torch.ops.aten.relu.default, (cur,))
            cur.meta["val"] = torch.empty(1024, 1024)
        s = g.call_function(torch.ops.aten.sum.default, (ag,))
        s.meta["val"] = torch.empty(())
        cur = g.call_function(torch.ops.aten.add.Tensor, (cur, s))
        cur.meta["val"] = torch.empty(1024, 1024)
    g.output((cur,))
    return fx.GraphModule(torch.nn.Module(), g), gathers


def _priced(alpha_us=10.0, gbps=100.0, compute_us=5.0, **kw):
    from autoparallel_b200.parallel.passes.bucketing import BucketCost

    return BucketCost(lambda kind, nb, n, group: alpha_us + nb / (gbps * 1e3), lambda node: compute_us, **kw)


def _count(gm, target):
    return sum(1 for n in gm.graph.nodes if n.op == "call_function" and n.target is target)


def test_priced_bucket_plan_merges_latency_bound_gathers_and_leaves_bandwidth_bound_ones():
    from autoparallel_b200.parallel.passes.bucketing import bucket_collectives
    from autoparallel_b200.runtime import comm_ops

    C = comm_ops.ops
    # eight 4 KiB gathers: each costs ~alpha; merging two saves one alpha
    gm, _ = _gather_chain_graph([1024] * 8)
    stats = bucket_collectives(gm, cost=_priced(max_fraction=1.0))
    assert stats["all_gather_buckets"] == 1 and stats["members"] == 8 and _count(gm, C.all_gather.default) == 1
    assert stats["saved_us"] == pytest.approx(7 * 10.0, rel=1e-3)
    gm.graph.lint()
    # the same gathers when latency is free: nothing to gain, nothing merged
    gm, _ = _gather_chain_graph([1024] * 8)
    stats = bucket_collectives(gm, cost=_priced(alpha_us=0.0, max_fraction=1.0))
    assert stats["members"] == 0 and stats["rejected_saving"] >= 1 and _count(gm, C.all_gather.default) == 8


def test_priced_bucket_plan_respects_window_memory_and_fraction():
    from autoparallel_b200.parallel.passes.bucketing import bucket_collectives
    from autoparallel_b200.runtime import comm_ops

    C = comm_ops.ops
    # 4 MiB gathers at 100 GB/s take ~52 us each; the window in front of the first consumer is 12 nodes x 5 us = 60 us,
    # so a second member (94 us merged) would expose communication: every gather stays alone
    gm, _ = _gather_chain_graph([1 << 20] * 6, lead=12)
    stats = bucket_collectives(gm, cost=_priced(max_fraction=1.0))
    assert stats["members"] == 0 and stats["rejected_window"] >= 1
    # a long compute window admits them ...
    gm, _ = _gather_chain_graph([1 << 20] * 6, lead=12)
    stats = bucket_collectives(gm, cost=_priced(compute_us=100.0, max_fraction=1.0))
    assert stats["members"] == 6 and _count(gm, C.all_gather.default) == 1
    # ... unless the memory the bucket keeps alive does not fit the headroom (4 MiB members, 6 MiB headroom)
    gm, _ = _gather_chain_graph([1 << 20] * 6, lead=12)
    stats = bucket_collectives(gm, cost=_priced(compute_us=100.0, max_fraction=1.0, headroom_bytes=6 << 20))
    assert stats["members"] == 0 and stats["rejected_memory"] >= 1
    # ... and no bucket takes more than the given fraction of all candidate bytes (0.5 of six members = three each)
    gm, _ = _gather_chain_graph([1 << 20] * 6, lead=12)
    stats = bucket_collectives(gm, cost=_priced(compute_us=100.0, max_fraction=0.5))
    assert stats["all_gather_buckets"] == 2 and stats["members"] == 6 and stats["rejected_fraction"] >= 1


def test_priced_bucket_plan_on_llama_keeps_numerics_and_reduces_collectives(mesh_1d):
    """End to end: ``bucket_collectives="auto"`` prices the collectives with the mesh's topology; the lowered graph has
    fewer collectives and a simulated step that is not slower."""
    from autoparallel_b200.runtime import comm_ops
    from autoparallel_b200.utils.trace_sim import estimate_graph_metrics

    C = comm_ops.ops
    ap = _llama(mesh_1d, fuse_collectives=False)
    try:
        plain = ap.lower()
        n_plain = _count(plain.gm, C.all_gather.default) + _count(plain.gm, C.reduce_scatter.default)
        t_plain = estimate_graph_metrics(plain.gm, mesh_1d, "B200").total_us
    finally:
        ap.__exit__(None, None, None)
    ap = _llama(mesh_1d, fuse_collectives=False, bucket_collectives="auto")
    try:
        low = ap.lower()
        low.gm.graph.lint()
        n_auto = _count(low.gm, C.all_gather.default) + _count(low.gm, C.reduce_scatter.default)
        t_auto = estimate_graph_metrics(low.gm, mesh_1d, "B200").total_us
        assert ap.bucket_stats["members"] >= 2 and ap.bucket_stats["saved_us"] > 0
        assert n_auto < n_plain
        assert t_auto <= t_plain * 1.001
    finally:
        ap.__exit__(None, None, None)


def test_arena_shadows_are_only_for_evenly_sharded_parameters(mesh_1d, mesh_2d):
    """The peer arena hands out offsets by allocation order; a peer's shard is read at the reader's own offset, so only
    parameters whose shards have the same shape on every rank may live there."""
    from torch.distributed.tensor import DTensor
    from torch.distributed.tensor.placement_types import Replicate

    from autoparallel_b200.optim import AdamW

    def dt(shape, mesh, placements):
        local = list(shape)
        for i, p in enumerate(placements):
            if p.is_shard():
                local[p.dim] = -(-local[p.dim] // mesh.size(i))
        return DTensor.from_local(torch.zeros(local), mesh, placements, run_check=False, shape=torch.Size(shape),
                                  stride=torch.zeros(shape).stride())

    assert AdamW._even_shards(torch.zeros(3, 5))                                   # a plain tensor
    assert AdamW._even_shards(dt((16, 4), mesh_1d, (Shard(0),)))
    assert not AdamW._even_shards(dt((20, 4), mesh_1d, (Shard(0),)))               # 20 rows over 8 ranks
    assert AdamW._even_shards(dt((16, 4), mesh_2d, (Shard(0), Shard(0))))          # nested: 16 / 2 / 4
    assert not AdamW._even_shards(dt((12, 4), mesh_2d, (Shard(0), Shard(0))))      # 12 / 2 = 6, not divisible by 4
    assert AdamW._even_shards(dt((12, 4), mesh_2d, (Shard(0), Replicate())))
