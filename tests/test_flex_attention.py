"""Flex attention in the planner: option enumeration for the two higher-order operators, planning and
shape-level execution on fake ranks, numerics on gloo ranks against plain causal attention.
(The reference covers the same ground in tests/test_flex_attention.py:261-583.)"""
import os

import pytest
from conftest import free_port
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Replicate, Shard

flex = pytest.importorskip("torch.nn.attention.flex_attention")


def _causal(b, h, q, kv):
    return q >= kv


class FlexBlock(nn.Module):
    def __init__(self, d=64, heads=4, kv_heads=2):
        super().__init__()
        self.h, self.kvh, self.hd = heads, kv_heads, d // heads
        self.wq = nn.Linear(d, d, bias=False)
        self.wk = nn.Linear(d, kv_heads * self.hd, bias=False)
        self.wv = nn.Linear(d, kv_heads * self.hd, bias=False)
        self.wo = nn.Linear(d, d, bias=False)

    def qkv(self, x):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, self.h, self.hd).transpose(1, 2)
        k = self.wk(x).view(B, S, self.kvh, self.hd).transpose(1, 2)
        v = self.wv(x).view(B, S, self.kvh, self.hd).transpose(1, 2)
        return q, k, v

    def forward(self, x):
        B, S, _ = x.shape
        q, k, v = self.qkv(x)
        mask = flex.create_block_mask(_causal, None, None, S, S, device=x.device)
        o = flex.flex_attention(q, k, v, block_mask=mask, enable_gqa=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))

    def reference(self, x):
        B, S, _ = x.shape
        q, k, v = self.qkv(x)
        rep = self.h // self.kvh
        o = torch.nn.functional.scaled_dot_product_attention(
            q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), is_causal=True
        )
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))


def _planned(mesh, in_pl, batch=8, seq=128, **model_kw):
    from autoparallel_b200 import AutoParallel, ForwardInputs

    with torch.device("meta"):
        model = FlexBlock(**model_kw)
    ap = AutoParallel(model, lambda: ForwardInputs((torch.randn(batch, seq, 64),), {}), mesh)
    ap.__enter__()
    ap.add_input_constraints([in_pl])
    return ap


def _flex_nodes(ap):
    from autoparallel_b200.parallel.strategies.flex_rules import is_flex_attention_node

    return [n for n in ap.joint.gm.graph.nodes if is_flex_attention_node(n)]


def _pl(spec):
    return tuple(spec.placements)


def test_options_split_batch_or_heads_and_keep_the_block_mask_replicated(mesh_2d):
    ap = _planned(mesh_2d, (Shard(0), Replicate()))
    try:
        fwd, bwd = _flex_nodes(ap)
        strats = ap.sharding_optimizer.strats
        rep = (Replicate(), Replicate())
        for node in (fwd, bwd):
            options = strats[node].strategies
            firsts = {_pl(o.input_specs[0]) for o in options}  # placements of q
            # 4 query heads, 2 key/value heads, mesh 2 x 4: heads split over dp only; batch over either or both
            assert (Shard(1), Replicate()) in firsts and (Shard(0), Shard(0)) in firsts and (Shard(1), Shard(0)) in firsts
            assert not any(p[1] == Shard(1) for p in firsts), "two key/value heads cannot be split four ways"
            for o in options:
                q = _pl(o.input_specs[0])
                for s in o.input_specs:
                    shape = tuple(s.tensor_meta.shape)
                    if len(shape) >= 2 and shape[0] == 1 and shape[1] == 1:
                        assert _pl(s) == rep  # block-mask index tensors built with B=None, H=None
                    elif len(shape) >= 3 and shape[0] == 8:
                        assert _pl(s) == q  # k, v, out, log-sum-exp, gradients follow q
                outs = [s for s in o.output_specs if s is not None]
                assert all(_pl(s) == q for s in outs)
            # no two options are the same
            keys = [(tuple(_pl(s) for s in o.input_specs), tuple(None if s is None else _pl(s) for s in o.output_specs)) for o in options]
            assert len(set(keys)) == len(keys)
    finally:
        ap.__exit__(None, None, None)


def test_single_key_value_head_stays_replicated_under_head_sharding(mesh_2d):
    ap = _planned(mesh_2d, (Shard(0), Replicate()), kv_heads=1)
    try:
        fwd = _flex_nodes(ap)[0]
        options = ap.sharding_optimizer.strats[fwd].strategies
        hit = [o for o in options if _pl(o.input_specs[0]) == (Replicate(), Shard(1))]
        assert hit, "four query heads over tp=4 with one shared key/value head is a valid option"
        assert _pl(hit[0].input_specs[1]) == (Replicate(), Replicate())
    finally:
        ap.__exit__(None, None, None)


def test_plan_lowers_and_runs_on_fake_ranks(mesh_2d):
    ap = _planned(mesh_2d, (Shard(0), Replicate()), batch=8, seq=256)
    try:
        ap.add_output_constraints([(Shard(0), Replicate())])
        ap.optimize_placement()
        pm = ap.apply_placement()
    finally:
        ap.__exit__(None, None, None)
    pm.to_empty(device="cpu")
    with torch.no_grad():
        for p in pm.parameters():
            p._local_tensor.normal_(std=0.05)
    y = pm(torch.randn(4, 256, 64))
    assert y.shape == (4, 256, 64)
    y.sum().backward()
    assert all(p.grad is not None for p in pm.parameters())


def _numerics_worker(rank, ws, how, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh

    from autoparallel_b200 import AutoParallel, ForwardInputs
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    from autoparallel_b200.parallel.strategies.flex_rules import is_flex_attention_node

    torch.manual_seed(0)
    ref = FlexBlock()
    with torch.device("meta"):
        model = FlexBlock()
    B, S = 4, 128
    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    with AutoParallel(model, lambda: ForwardInputs((torch.randn(B, S, 64),), {}), mesh) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        if how == "heads":  # pin the attention call to head sharding: inputs arrive batch-sharded and are moved
            for n in ap.joint.gm.graph.nodes:
                if is_flex_attention_node(n):
                    ap.sharding_optimizer.add_node_constraint(n, (Shard(1),))
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    ref_state = dict(ref.named_parameters())
    with torch.no_grad():
        for n, t in pm.named_parameters():
            t._local_tensor.copy_(_distribute(ref_state[n].detach(), mesh, t.placements)._local_tensor)
    torch.manual_seed(1)
    x = torch.randn(B, S, 64)
    w = torch.linspace(-1, 1, 64)
    y = pm(x.chunk(ws, 0)[rank])
    (y * w).sum().backward()
    y_ref = ref.reference(x)
    (y_ref * w).sum().backward()
    err = (y - y_ref.chunk(ws, 0)[rank]).abs().max().item()
    worst = 0.0
    for n, p in pm.named_parameters():
        g, rg = p.grad.full_tensor(), ref_state[n].grad
        worst = max(worst, ((g - rg).abs().max() / (rg.abs().max() + 1e-12)).item())
    if rank == 0:
        q.put((err, worst))
    dist.destroy_process_group()


@pytest.mark.parametrize("how", ["auto", "heads"])
def test_matches_plain_causal_attention_on_two_ranks(how):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_numerics_worker, args=(2, how, free_port(), q), nprocs=2, join=True)
    err, worst = q.get()
    assert err < 1e-4 and worst < 1e-3
