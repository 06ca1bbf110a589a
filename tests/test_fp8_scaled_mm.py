"""fp8 projections with scales: the operator, its sharding rule, the pattern rewrite of ``torch._scaled_mm``, the fused
collective forms and two-rank numerics.  (Reference: autoparallel/graph_passes/async_tp/asynctp_ops.py:363-393, 948-1026,
1189-1424 - scale modes and the scaled fused ops; tests/test_ops.py for the operator-level checks.)"""
import os

import pytest
import torch
import torch.distributed as dist
import torch.fx as fx
import torch.multiprocessing as mp
import torch.nn as nn
from conftest import free_port

from autoparallel_b200.ops import library  # noqa: F401  (registers apb200::*)
from autoparallel_b200.runtime import comm_ops

apb = torch.ops.apb200
C = comm_ops.ops
F8 = torch.float8_e4m3fn


def quant_rows(t):
    amax = t.abs().amax(dim=-1, keepdim=True).clamp(min=1e-6)
    scale = amax / 448.0
    return (t / scale).to(F8), scale


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("rowwise", [True, False])
def test_scaled_mm_reference_matches_dequantised_product(trans_b, rowwise):
    torch.manual_seed(0)
    x, w = torch.randn(2, 6, 32), torch.randn(16, 32)
    if rowwise:
        xq, sx = quant_rows(x)
        wq, sw = quant_rows(w)
    else:
        sx, sw = x.abs().max() / 448.0, w.abs().max() / 448.0
        xq, wq = (x / sx).to(F8), (w / sw).to(F8)
    b = wq if trans_b else wq.t().contiguous()
    sb = sw if trans_b or not rowwise else sw.t()
    y = apb.scaled_mm(xq, b, sx, sb, trans_b, torch.float32)
    ref = (xq.float() * sx) @ (wq.float() * sw).t()
    assert y.shape == (2, 6, 16) and torch.allclose(y, ref, atol=1e-5, rtol=1e-5)
    # and the product is a usable approximation of the unquantised one (e4m3: 3 mantissa bits)
    assert (y - x @ w.t()).abs().max() < 0.15 * (x @ w.t()).abs().max()


def test_scaled_mm_rule_shards_scales_with_their_rows(mesh_1d):
    from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

    from autoparallel_b200 import AutoParallel

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("wq", torch.zeros(64, 32).to(F8))
            self.register_buffer("sw", torch.ones(64, 1))
            self.head = nn.Linear(64, 16, bias=False)

        def forward(self, x):
            with torch.no_grad():
                xq, sx = quant_rows(x)
            y = torch._scaled_mm(xq, self.wq.t(), scale_a=sx, scale_b=self.sw.t(), out_dtype=torch.float32)
            return self.head(torch.relu(y)).sum()

    with torch.device("meta"):
        m = M()
    with AutoParallel(m, lambda: torch.randn(32, 32), mesh_1d) as ap:
        assert ap.joint.pattern_stats["scaled_mm"] == 1
        node = next(n for n in ap.joint.gm.graph.nodes if n.op == "call_function" and n.target is apb.scaled_mm.default)
        assert node.args[4] is True  # ``w.t()`` folded: the weight is read as stored
        strat = ap.sharding_optimizer.strats[node]
        seen = set()
        for s in strat.strategies:
            out = s.output_specs.placements[0]
            ins = tuple(i.placements[0] for i in s.input_specs)
            seen.add((out, ins))
        S, R, P = Shard, Replicate(), Partial()
        assert (S(0), (S(0), R, S(0), R)) in seen        # rows of x with their row-wise scale
        assert (S(1), (R, S(0), R, S(0))) in seen        # columns of the result = rows of the stored weight, with their scale
        assert (P, (S(1), S(1), R, R)) in seen           # contraction split: scales whole, partial sums
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        low = ap.lower()
        assert any(n.op == "call_function" and n.target is apb.scaled_mm.default for n in low.gm.graph.nodes)


def _graph_for_fusion(kind):
    g = fx.Graph()

    def ph(name, *shape, dtype=torch.float32):
        n = g.placeholder(name)
        n.meta["val"] = torch.empty(*shape, dtype=dtype)
        return n

    def call(target, args, val):
        n = g.call_function(target, args)
        n.meta["val"] = val
        return n

    if kind == "ag_act":      # sequence-sharded fp8 activation + its row-wise scale, gathered in front of the projection
        x, sx = ph("x", 1, 8, 32, dtype=F8), ph("sx", 1, 8, 1)
        w, sw = ph("w", 16, 32, dtype=F8), ph("sw", 16, 1)
        xf = call(C.all_gather.default, (x, 1, "g", 4), torch.empty(1, 32, 32, dtype=F8))
        sxf = call(C.all_gather.default, (sx, 1, "g", 4), torch.empty(1, 32, 1))
        y = call(apb.scaled_mm.default, (xf, w, sxf, sw, True, torch.bfloat16), torch.empty(1, 32, 16, dtype=torch.bfloat16))
    elif kind == "ag_weight":  # FSDP-style weight shard + row-wise scale
        x, sx = ph("x", 1, 8, 32, dtype=F8), ph("sx", 1, 8, 1)
        w, sw = ph("w", 4, 32, dtype=F8), ph("sw", 4, 1)
        wf = call(C.all_gather.default, (w, 0, "g", 4), torch.empty(16, 32, dtype=F8))
        swf = call(C.all_gather.default, (sw, 0, "g", 4), torch.empty(16, 1))
        y = call(apb.scaled_mm.default, (x, wf, sx, swf, True, torch.bfloat16), torch.empty(1, 8, 16, dtype=torch.bfloat16))
    else:                      # row-parallel projection, sequence-sharded result
        x, sx = ph("x", 1, 32, 8, dtype=F8), ph("sx", 1, 32, 1)
        w, sw = ph("w", 16, 8, dtype=F8), ph("sw", 16, 1)
        full = call(apb.scaled_mm.default, (x, w, sx, sw, True, torch.float32), torch.empty(1, 32, 16))
        y = call(C.reduce_scatter.default, (full, 1, "g", 4), torch.empty(1, 8, 16))
    g.output((y,))
    return fx.GraphModule(nn.Module(), g)


@pytest.mark.parametrize("kind,key,mode", [("ag_act", "ag_scaled_mm", 2), ("ag_weight", "ag_scaled_mm", 0), ("rs", "scaled_mm_rs", 0)])
def test_fusion_pass_builds_the_scaled_forms(kind, key, mode):
    from autoparallel_b200.parallel.passes.fuse_collectives import fuse_collectives

    gm = _graph_for_fusion(kind)
    stats = fuse_collectives(gm)
    assert stats[key] == 1
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    fused = next(n for n in gm.graph.nodes if n.op == "call_function" and n.target in comm_ops.SCALED_FUSED_OPS)
    assert fused.args[4] == mode
    # the separate collectives (of the operand and of its scale) are gone
    assert C.all_gather.default not in targets and C.reduce_scatter.default not in targets and apb.scaled_mm.default not in targets
    # the scale handed to the fused node is the un-gathered one
    if kind == "ag_act":
        assert fused.args[2].name == "sx" and fused.args[5] == 1
    if kind == "ag_weight":
        assert fused.args[3].name == "sw"


def _fused_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    name = dist.group.WORLD.group_name
    torch.manual_seed(0)
    x, w = torch.randn(1, 8 * ws, 32), torch.randn(16, 32)
    xq, sx = quant_rows(x)
    wq, sw = quant_rows(w)
    ref = apb.scaled_mm(xq, wq, sx, sw, True, torch.float32)
    rows = slice(8 * rank, 8 * rank + 8)
    # gathered activation rows (mode 2) and gathered weight rows (mode 0)
    y2, xf = C.ag_scaled_mm(xq[:, rows].contiguous(), wq, sx[:, rows].contiguous(), sw, 2, 1, torch.float32, name, ws)
    nr = 16 // ws
    y0, wf = C.ag_scaled_mm(xq, wq[nr * rank : nr * rank + nr].contiguous(), sx, sw[nr * rank : nr * rank + nr].contiguous(), 0, 0,
                            torch.float32, name, ws)
    # row-parallel: every rank holds a slice of the contraction dim; per-tensor scales (row-wise scales would differ per slice)
    st, swt = x.abs().max() / 448.0, w.abs().max() / 448.0
    xt, wt = (x / st).to(F8), (w / swt).to(F8)
    ks = slice(32 // ws * rank, 32 // ws * (rank + 1))
    yr = C.scaled_mm_rs(xt[..., ks].contiguous(), wt[:, ks].contiguous(), st, swt, 0, 1, torch.float32, name, ws)
    ref_t = apb.scaled_mm(xt, wt, st, swt, True, torch.float32)
    ok = (torch.allclose(y2, ref, atol=1e-5) and torch.equal(xf.float(), xq.float()) and torch.allclose(y0, ref, atol=1e-5)
          and torch.equal(wf.float(), wq.float()) and torch.allclose(yr, ref_t[:, rows], atol=1e-4))
    if rank == 0:
        q.put(bool(ok))
    dist.destroy_process_group()


def test_scaled_fused_ops_match_the_unsharded_product_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_fused_worker, args=(2, free_port(), q), nprocs=2, join=True)
    assert q.get() is True


class _Fp8Block(nn.Module):
    """A frozen fp8 projection (weight quantised once, activations quantised on the fly) feeding a trainable head."""

    def __init__(self):
        super().__init__()
        self.register_buffer("wq", torch.zeros(64, 32).to(F8))
        self.register_buffer("sw", torch.ones(64, 1))
        self.head = nn.Linear(64, 16, bias=False)

    def init_weights(self):
        g = torch.Generator().manual_seed(3)
        wq, sw = quant_rows(torch.randn(64, 32, generator=g))
        with torch.no_grad():
            self.wq.copy_(wq)
            self.sw.copy_(sw)
            self.head.weight.copy_(torch.randn(16, 64, generator=g) * 0.1)

    def forward(self, x):
        with torch.no_grad():
            xq, sx = quant_rows(x)
        y = self.mm(xq, sx)
        return self.head(torch.relu(y)).square().mean()

    def mm(self, xq, sx):
        return torch._scaled_mm(xq, self.wq.t(), scale_a=sx, scale_b=self.sw.t(), out_dtype=torch.float32)


class _Fp8BlockEager(_Fp8Block):
    """The single-device comparison: eager ``torch._scaled_mm`` has no row-wise scales on CPU, so the product is written out."""

    def mm(self, xq, sx):
        return (xq.float() * sx) @ (self.wq.float() * self.sw).t()


def _model_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Shard

    from autoparallel_b200 import AutoParallel

    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with torch.device("meta"):
        m = _Fp8Block()
    with AutoParallel(m, lambda: torch.randn(16, 32), mesh) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    pm.init_weights()
    torch.manual_seed(5)
    x = torch.randn(16, 32)
    loss = pm(x.chunk(ws, 0)[rank])
    loss.backward()
    ref = _Fp8BlockEager()
    ref.init_weights()
    rl = ref(x)
    rl.backward()
    gerr = (pm.head.weight.grad.full_tensor() - ref.head.weight.grad).abs().max().item()
    if rank == 0:
        q.put((loss.item(), rl.item(), gerr))
    dist.destroy_process_group()


def test_model_with_fp8_projection_matches_single_device_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_model_worker, args=(2, free_port(), q), nprocs=2, join=True)
    loss, ref, gerr = q.get()
    assert abs(loss - ref) < 1e-5 * max(1.0, abs(ref)) and gerr < 1e-5
