"""Behaviours that the reference pins with small dedicated tests, checked here against this package on fake
ranks: parameters that do not divide, a parameter smaller than the mesh, the parameter / gradient pairing when
a gradient lacks an option, user methods on the parallel module, dict inputs and input validation, in-graph
constructors and fresh mutations, log rendering, alias-preserving fake conversion, node constraints against
the memory budget with removal and re-solve.
(Reference: tests/test_optimize_placement.py:519-700, tests/test_paired_output_constraint.py,
tests/test_api.py, tests/test_input_validation.py, tests/test_propagation_rules.py, tests/test_log_formatting.py,
tests/test_tracing.py.)"""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs


def test_parameter_that_does_not_divide_keeps_the_memory_constraint_feasible(mesh_2d):
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l1 = nn.Linear(64, 21, bias=True)
            s.l2 = nn.Linear(21, 64, bias=True)
        def forward(s, x):
            return s.l2(F.relu(s.l1(x)))
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 64), mesh_2d) as ap:
        ap.add_input_constraints([(Shard(0), Replicate())])
        ap.add_output_constraints([(Shard(0), Replicate())])
        ap.add_parameter_memory_constraint(low=None, high=None)
        sol = ap.optimize_placement()
        assert all(p in sol for p in ap.joint.param_nodes.values())


def test_parameter_smaller_than_the_mesh(mesh_1d):
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l1 = nn.Linear(64, 4, bias=True)
            s.scale = nn.Parameter(torch.ones(1))
        def forward(s, x):
            return s.l1(x) * s.scale
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 64), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.add_parameter_memory_constraint(low=None, high=None)
        ap.optimize_placement()
        pm = ap.apply_placement()


def test_parameter_cannot_take_a_placement_its_gradient_lacks(mesh_2d):
    with torch.device("meta"):
        m = nn.Linear(64, 128, bias=False)
    ap = AutoParallel(m, lambda: torch.rand(32, 64), mesh_2d)
    ap.__enter__()
    try:
        opt = ap.sharding_optimizer
        p = next(iter(ap.joint.param_nodes.values()))
        g = next(iter(ap.joint.param_grads.values()))
        removed = (Shard(0), Shard(0))
        opt.strats[g].strategies = [s for s in opt.strats[g].strategies if tuple(s.output_spec.placements) != removed]
        opt._node_cost.clear()
        opt._edge_cost.clear()
        opt._build_costs()
        ap.add_input_constraints([(Shard(0), Replicate())])
        ap.add_output_constraints([(Shard(0), Replicate())])
        ap.add_parameter_memory_constraint(low=None, high=None)
        sol = ap.optimize_placement()
        chosen = tuple(sol[p].output_spec.placements)
        assert chosen != removed, chosen
        assert chosen in {tuple(s.output_spec.placements) for s in opt.strats[g].strategies}
    finally:
        ap.__exit__(None, None, None)


def test_user_methods_properties_and_buffer_updates_on_the_parallel_module(mesh_1d):
    class Base(nn.Module):
        def helper(s):
            return "base"
    class M(Base):
        tag = "x"
        def __init__(s):
            super().__init__()
            s.l = nn.Linear(16, 16)
            s.register_buffer("ema", torch.zeros(16))
            s.decay = 0.9
        def forward(s, x):
            return s.l(x) + s.ema
        @torch.no_grad()
        def update_ema(s):
            s.ema.mul_(s.decay).add_(1.0)
        @classmethod
        def make(cls):
            return cls.tag
        @property
        def width(s):
            return s.l.in_features
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(8, 16), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    assert isinstance(pm, M) and isinstance(pm, Base) and pm.helper() == "base" and pm.make() == "x" and pm.width == 16 and pm.decay == 0.9
    with torch.no_grad():
        pm.ema.zero_()
    pm.update_ema()
    assert torch.allclose(pm.ema.to_local(), torch.ones_like(pm.ema.to_local()))


def test_dict_inputs_outputs_and_shape_validation(mesh_1d):
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l = nn.Linear(16, 16)
        def forward(s, batch):
            return {"y": s.l(batch["x"]) + batch["bias"], "aux": batch["x"].mean()}
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: ForwardInputs(({"x": torch.rand(16, 16), "bias": torch.rand(16)},), {}), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),), (Replicate(),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    out = pm({"x": torch.rand(2, 16), "bias": torch.rand(16)})
    assert set(out) == {"y", "aux"} and out["y"].shape[1] == 16
    try:
        pm({"x": torch.rand(3, 16), "bias": torch.rand(16)})
        raise AssertionError("wrong shape accepted")
    except ValueError:
        pass


def test_in_graph_constructors_index_put_and_fresh_mutation(mesh_1d):
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l = nn.Linear(16, 16)
        def forward(s, x):
            idx = torch.arange(x.shape[0], device=x.device)
            buf = torch.zeros(x.shape[0], 16, device=x.device)
            buf = buf.index_put((idx,), s.l(x))
            buf[0] = 1.0
            return buf * (idx.unsqueeze(1) + 1)
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 16), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    pm(torch.rand(2, 16)).sum().backward()


def test_log_plain_verbose_and_colored(mesh_1d):
    with torch.device("meta"):
        m = nn.Linear(16, 16)
    with AutoParallel(m, lambda: torch.rand(16, 16), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        opt = ap.sharding_optimizer
        a = opt.get_log(verbose=False)
        b = opt.get_log(verbose=True)
        c = opt.get_log(colored=True)
        assert "placement" in a.lower() or "Shard" in a or "S(0)" in a, a[:200]
        assert len(b) >= len(a) and "\x1b[" in c


def test_fake_conversion_keeps_aliases():
    from autoparallel_b200.parallel.frontend.trace import move_to_fake
    from torch._subclasses import FakeTensorMode
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.a = nn.Linear(4, 4)
            s.b = nn.Linear(4, 4)
            s.b.weight = s.a.weight
            s.register_buffer("u", torch.zeros(4))
            s.register_buffer("v", s.u)
            s.c = s.a
    with torch.device("meta"):
        m = M()
    f = move_to_fake(m, FakeTensorMode(), "cpu")
    assert f.a.weight is f.b.weight and f.u is f.v and f.c is f.a and f.a.bias is not f.b.bias


def test_node_constraint_against_memory_budget_then_removal_and_resolve(mesh_1d):
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l1 = nn.Linear(64, 64)
            s.l2 = nn.Linear(64, 64)
        def forward(s, x):
            return s.l2(F.relu(s.l1(x)))
    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 64), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        name = ap.add_parameter_memory_constraint(low=None, high=None)
        opt = ap.sharding_optimizer
        w1 = ap.joint.param_nodes["l1.weight"]
        c = opt.add_node_constraint(w1, (Replicate(),))
        sol = ap.optimize_placement()
        assert tuple(sol[w1].output_spec.placements) == (Replicate(),)
        assert any(isinstance(p, Shard) for p in sol[ap.joint.param_nodes["l2.weight"]].output_spec.placements)
        opt.remove_constraints([c])
        sol = opt.resolve() if hasattr(opt, "resolve") else opt.get_solution()
        assert any(isinstance(p, Shard) for p in sol[w1].output_spec.placements)
        opt.remove_constraints([name])
        sol = opt.resolve() if hasattr(opt, "resolve") else opt.get_solution()
        assert tuple(sol[w1].output_spec.placements) == (Replicate(),)



def test_norm_as_first_op_on_an_input_without_gradient(mesh_1d):
    # native_layer_norm_backward then has no input gradient: its first output spec is None
    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.n = nn.LayerNorm(32)
            s.l = nn.Linear(32, 32)

        def forward(s, x):
            return s.l(s.n(x))

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 32), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    pm(torch.rand(2, 32)).sum().backward()
    assert all(p.grad is not None for p in pm.parameters())


def test_strided_factories_get_local_sizes_and_strides(mesh_1d):
    from autoparallel_b200.parallel.lower.apply import _strides_like

    assert _strides_like([64, 1, 8], [2, 8, 8]) == [64, 1, 8]  # dim order of the original strides is kept
    assert _strides_like([1, 4], [4, 2]) == [1, 4]
    assert _strides_like([12, 4, 1], [2, 3, 0]) == [3, 1, 1]   # empty extents count as 1 when accumulating

    class M(nn.Module):
        def __init__(s):
            super().__init__()
            s.l = nn.Linear(16, 16)

        def forward(s, x):
            y = s.l(x)
            buf = y.new_empty_strided((x.shape[0], 16), (16, 1))
            buf.copy_(y)
            return buf * 2.0

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.rand(16, 16), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    out = pm(torch.rand(2, 16))
    assert out.shape == (2, 16)
    out.sum().backward()


def test_gradients_flow_through_an_output_that_is_a_view_of_another_output(mesh_1d):
    """``return y.t(), y``: the differentiated graph has no tangent for an output that aliases another one (a run-time wrapper
    is expected to rebuild it as a view); here such an output gets a copy of its own, so a loss on it reaches the parameters."""
    import torch.nn as nn

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(8, 8)

        def forward(self, x):
            y = self.l(x)
            return y.t(), y, x.t()          # a view of another output, the output itself, a view of an input

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.randn(16, 8), mesh_1d) as ap:
        assert len(ap.joint.tangent_nodes) >= 2
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(1),), (Shard(0),), None])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    with torch.no_grad():
        for p in pm.parameters():
            p.to_local().normal_()
    x = torch.randn(16 // mesh_1d.size(0), 8)
    a, b, c = pm(x)
    assert torch.equal(a, b.t())
    a.sum().backward()
    g_view = pm.l.weight.grad.to_local().clone()
    pm.l.weight.grad = None
    a, b, c = pm(x)
    b.sum().backward()
    assert g_view.abs().sum() > 0 and torch.allclose(g_view, pm.l.weight.grad.to_local())


def test_operators_of_the_planning_host_are_swapped_when_the_graphs_move_to_another_device(mesh_1d):
    """Attention that the pattern pass does not take over is traced (on CPU fake tensors) to operators only the CPU has; when
    the runtime retargets its graphs they become device-neutral functions, and device constants follow."""
    import torch.nn as nn
    import torch.nn.functional as F

    from autoparallel_b200.runtime import portable_ops

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = nn.Linear(64, 192)

        def forward(self, x):
            q, k, v = self.qkv(x).view(x.shape[0], x.shape[1], 3, 4, 16).permute(2, 0, 3, 1, 4)
            pos = torch.arange(x.shape[1], device=x.device)
            bias = -(pos[:, None] - pos[None, :]).abs().to(x.dtype)            # an explicit additive mask
            return F.scaled_dot_product_attention(q, k, v, attn_mask=bias).sum()

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.randn(8, 32, 64), mesh_1d, pattern_ops=False) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    rt = pm.__dict__["_apb200_runtime"]
    aten = torch.ops.aten
    before = {n.target for g in (rt.fw, rt.bw) for n in g.graph.nodes if n.op == "call_function"}
    assert aten._scaled_dot_product_flash_attention_for_cpu.default in before
    # reference run with the host's operators
    pm.to_empty(device="cpu")
    with torch.no_grad():
        for p_ in pm.parameters():
            p_.to_local().normal_(std=0.2)
    x = torch.randn(8 // mesh_1d.size(0), 32, 64)
    ref = pm(x)
    ref.backward()
    ref_grad = pm.qkv.weight.grad.to_local().clone()
    pm.qkv.weight.grad = None
    rt._retarget(torch.device("cuda", 0))                                       # graph surgery only: nothing is run
    after = {n.target for g in (rt.fw, rt.bw, rt.fwd_only) for n in g.graph.nodes if n.op == "call_function"}
    assert aten._scaled_dot_product_flash_attention_for_cpu.default not in after
    assert aten._scaled_dot_product_flash_attention_for_cpu_backward.default not in after
    assert portable_ops.sdpa_forward in after and portable_ops.sdpa_backward in after
    devs = {n.kwargs["device"] for g in (rt.fw, rt.bw) for n in g.graph.nodes if n.op == "call_function" and "device" in n.kwargs}
    assert devs == {torch.device("cuda", 0)}
    # the swapped graphs compute the same thing (run here on the CPU again, with the stand-ins' generic path forced)
    rt._retarget(torch.device("cpu"))
    portable_ops.FORCE_GENERIC = True
    try:
        for formulas in (False, True):
            portable_ops.FORMULAS_ONLY = formulas
            out = pm(x)
            out.backward()
            assert torch.allclose(out, ref, rtol=1e-5, atol=1e-3)
            assert torch.allclose(pm.qkv.weight.grad.to_local(), ref_grad, rtol=1e-4, atol=1e-3)  # values up to a few hundred, fp32
            pm.qkv.weight.grad = None
    finally:
        portable_ops.FORCE_GENERIC = portable_ops.FORMULAS_ONLY = False


def test_tensor_constants_created_in_the_forward_follow_the_graphs(mesh_1d):
    """``torch.tensor([...])`` inside ``forward`` becomes a constant attribute of the traced graphs, materialised on the planning
    host; it moves with the graphs when they are retargeted (a CPU constant next to device tensors is an error otherwise)."""
    import torch.nn as nn

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(4, 4)

        def forward(self, x):
            return self.l(x) * torch.tensor([0.5, 2.0, 1.0, -1.0]) + torch.tensor(3.0)

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.randn(16, 4), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    rt = pm.__dict__["_apb200_runtime"]
    consts = [b for g in (rt.fw, rt.bw, rt.fwd_only) for _, b in g.named_buffers()]
    assert consts and all(b.device.type == "cpu" for b in consts)
    rt._retarget(torch.device("meta"))
    consts = [b for g in (rt.fw, rt.bw, rt.fwd_only) for _, b in g.named_buffers()]
    assert consts and all(b.device.type == "meta" for b in consts)
