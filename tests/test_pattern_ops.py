"""The pattern pass puts a model written in stock PyTorch on the framework's operators.

The model below uses the idioms of the reference's own Llama (autoparallel/_testing/models/llama3.py:187-213,
355-356, 396-397): ``nn.RMSNorm``, rotary embedding by complex multiplication, ``repeat_kv`` + heads-first
``F.scaled_dot_product_attention``, ``F.silu(w1(x)) * w3(x)``.  A second block uses the hand-written RMSNorm of
the Hugging Face Llama family."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F
from conftest import free_port
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel

apb = torch.ops.apb200
aten = torch.ops.aten


class ManualRMSNorm(nn.Module):
    def __init__(self, d, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        dt = x.dtype
        h = x.to(torch.float32)
        var = h.pow(2).mean(-1, keepdim=True)
        h = h * torch.rsqrt(var + self.eps)
        return self.weight * h.to(dt)


def precompute_freqs_cis(dim, end, theta=10000.0):
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].float() / dim))
    t = torch.arange(end)
    return torch.polar(torch.ones(end, dim // 2), torch.outer(t, freqs))


class Attention(nn.Module):
    def __init__(self, d, h, hkv):
        super().__init__()
        self.h, self.hkv, self.hd = h, hkv, d // h
        self.wq = nn.Linear(d, h * self.hd, bias=False)
        self.wk = nn.Linear(d, hkv * self.hd, bias=False)
        self.wv = nn.Linear(d, hkv * self.hd, bias=False)
        self.wo = nn.Linear(h * self.hd, d, bias=False)

    def forward(self, x, freqs_cis):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, -1, self.hd)
        k = self.wk(x).view(B, S, -1, self.hd)
        v = self.wv(x).view(B, S, -1, self.hd)
        q_ = torch.view_as_complex(q.float().reshape(B, S, self.h, -1, 2))
        k_ = torch.view_as_complex(k.float().reshape(B, S, self.hkv, -1, 2))
        f = freqs_cis[0:S].view(1, S, 1, self.hd // 2)
        q = torch.view_as_real(q_ * f).flatten(3).type_as(q)
        k = torch.view_as_real(k_ * f).flatten(3).type_as(k)
        rep = self.h // self.hkv
        k = torch.unsqueeze(k, dim=3).expand(B, S, self.hkv, rep, self.hd).reshape(B, S, self.h, self.hd)
        v = torch.unsqueeze(v, dim=3).expand(B, S, self.hkv, rep, self.hd).reshape(B, S, self.h, self.hd)
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        return self.wo(out.transpose(1, 2).contiguous().view(B, S, -1))


class Block(nn.Module):
    def __init__(self, d, h, hkv, f, manual_norm):
        super().__init__()
        self.attention = Attention(d, h, hkv)
        self.w1, self.w2, self.w3 = nn.Linear(d, f, bias=False), nn.Linear(f, d, bias=False), nn.Linear(d, f, bias=False)
        norm = (lambda: ManualRMSNorm(d)) if manual_norm else (lambda: nn.RMSNorm(d, eps=1e-5))
        self.attention_norm, self.ffn_norm = norm(), norm()

    def forward(self, x, freqs_cis):
        h = x + self.attention(self.attention_norm(x), freqs_cis)
        y = self.ffn_norm(h)
        return h + self.w2(F.silu(self.w1(y)) * self.w3(y))


class PlainLlama(nn.Module):
    def __init__(self, vocab=256, d=64, h=4, hkv=2, f=128, seq=32):
        super().__init__()
        self.tok = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList([Block(d, h, hkv, f, manual_norm=False), Block(d, h, hkv, f, manual_norm=True)])
        self.norm = nn.RMSNorm(d, eps=1e-5)
        self.out = nn.Linear(d, vocab, bias=False)
        self.register_buffer("freqs_cis", precompute_freqs_cis(d // h, seq), persistent=False)

    def forward(self, ids):
        x = self.tok(ids)
        for layer in self.layers:
            x = layer(x, self.freqs_cis)
        return self.out(self.norm(x))


def _targets(gm):
    return [n.target for n in gm.graph.nodes if n.op == "call_function"]


def test_plain_pytorch_llama_traces_into_framework_operators(mesh_1d):
    with torch.device("meta"):
        model = PlainLlama()
    with AutoParallel(model, lambda: torch.randint(0, 256, (8, 32)), mesh_1d) as ap:
        stats = ap.joint.pattern_stats
        assert stats == {"rms_norm": 5, "swiglu": 2, "attention": 2, "rope": 4, "embedding": 1, "scaled_mm": 0}
        t = _targets(ap.gm)
        assert t.count(apb.rms_norm.default) == 5 and t.count(apb.rms_norm_bwd.default) == 5
        assert t.count(apb.attention.default) == 2 and t.count(apb.attention_bwd.default) == 2
        assert t.count(apb.swiglu.default) == 2 and t.count(apb.swiglu_bwd.default) == 2
        assert t.count(apb.rope.default) == 8  # four forward, four (conjugate) in the backward
        # nothing of the decomposed forms is left: no rsqrt, no sigmoid, no complex view of activations, no ATen attention
        assert aten.rsqrt.default not in t and aten.sigmoid.default not in t and aten.view_as_complex.default not in t
        assert not any("scaled_dot_product" in str(x) for x in t)
        # grouped-query keys / values reach the operator unexpanded
        att = next(n for n in ap.gm.graph.nodes if n.target is apb.attention.default)
        assert att.args[0].meta["val"].shape[2] == 4 and att.args[1].meta["val"].shape[2] == 2
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        ap.apply_placement()


def test_pattern_pass_can_be_switched_off(mesh_1d):
    with torch.device("meta"):
        model = PlainLlama()
    with AutoParallel(model, lambda: torch.randint(0, 256, (8, 32)), mesh_1d, pattern_ops=False) as ap:
        t = _targets(ap.gm)
        assert ap.joint.pattern_stats == {} and apb.rms_norm.default not in t and aten.rsqrt.default in t


def test_idioms_that_do_not_match_exactly_are_left_alone(mesh_1d):
    class Odd(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Linear(64, 64, bias=False)

        def forward(self, x):
            a = self.w(x)
            s = F.silu(a)
            y = s * a + s  # silu has two users: not a gated unit
            q = y.view(8, 32, 4, 16).transpose(1, 2)
            mask = torch.ones(32, 32, dtype=torch.bool).tril()
            return F.scaled_dot_product_attention(q, q, q, attn_mask=mask)  # explicit mask: not rewritten

    with torch.device("meta"):
        model = Odd()
    with AutoParallel(model, lambda: torch.rand(8, 32, 64), mesh_1d) as ap:
        assert not any(ap.joint.pattern_stats.values())


def _numerics_worker(rank, ws, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import distribute_tensor

    mesh = init_device_mesh("cpu", (ws,), mesh_dim_names=("dp",))
    torch.manual_seed(0)
    ref = PlainLlama()
    with torch.device("meta"):
        model = PlainLlama()
    with AutoParallel(model, lambda: torch.randint(0, 256, (8, 32)), mesh) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.add_output_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    with torch.no_grad():
        for (n, p), (_, rp) in zip(pm.named_parameters(), ref.named_parameters()):
            p.copy_(distribute_tensor(rp.detach(), mesh, p.placements))
        pm.freqs_cis.copy_(ref.freqs_cis) if not hasattr(pm.freqs_cis, "placements") else pm.freqs_cis.copy_(
            distribute_tensor(ref.freqs_cis, mesh, pm.freqs_cis.placements))
    torch.manual_seed(1)
    ids = torch.randint(0, 256, (8, 32))
    out = pm(ids.chunk(ws, 0)[rank])
    out.square().mean().backward()
    ro = ref(ids)
    (ro.square().mean()).backward()
    fwd = (out - ro.chunk(ws, 0)[rank]).abs().max().item()
    # the parallel loss is the mean over this rank's half: gradients are averages over ranks of per-rank means
    worst = max(((p.grad.full_tensor() / ws - rp.grad).abs().max() / (rp.grad.abs().max() + 1e-12)).item()
                for (_, p), (_, rp) in zip(pm.named_parameters(), ref.named_parameters()))
    if rank == 0:
        q.put((fwd, worst))
    dist.destroy_process_group()


def test_rewritten_model_matches_the_plain_model_on_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(_numerics_worker, args=(2, free_port(), q), nprocs=2, join=True)
    fwd, worst = q.get()
    assert fwd < 1e-4 and worst < 1e-4, (fwd, worst)
