"""Structurally unusual models against their single-device copy on two gloo ranks: tied and twice-used parameters, in-place
operators, no-grad sections, nested outputs, outputs that are inputs / parameters products / returned twice, a sub-module
used at two depths, scalar parameters and integer buffers, a small conv net.  (Reference: tests/test_correctness.py.)"""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F
from conftest import free_port

class Tied(nn.Module):
    def __init__(s):
        super().__init__(); s.emb = nn.Embedding(32, 16); s.mid = nn.Linear(16, 16); s.out = nn.Linear(16, 32, bias=False); s.out.weight = s.emb.weight
    def forward(s, ids): return s.out(torch.tanh(s.mid(s.emb(ids))))
class Twice(nn.Module):
    def __init__(s):
        super().__init__(); s.l = nn.Linear(16, 16)
    def forward(s, x): return s.l(torch.relu(s.l(x))) + s.l.weight.sum()
class InPlace(nn.Module):
    def __init__(s):
        super().__init__(); s.l = nn.Linear(16, 16)
    def forward(s, x):
        y = s.l(x); y.add_(1.0); y = F.relu_(y); z = y.clone(); z[:, 0] = 0.0; z.mul_(2.0)
        return z
class NoGradPart(nn.Module):
    def __init__(s):
        super().__init__(); s.a = nn.Linear(16, 16); s.b = nn.Linear(16, 16)
    def forward(s, x):
        with torch.no_grad(): h = s.a(x)
        return s.b(h + s.a(x).detach()) + s.a(x)
class MultiOut(nn.Module):
    def __init__(s):
        super().__init__(); s.a = nn.Linear(16, 16); s.b = nn.Linear(16, 8)
    def forward(s, x):
        h = s.a(x); return {"h": h, "pair": (s.b(h), h.mean(-1))}
class Chunks(nn.Module):
    def __init__(s):
        super().__init__(); s.qkv = nn.Linear(16, 48)
    def forward(s, x):
        q, k, v = s.qkv(x).chunk(3, -1)
        a = torch.softmax(q @ k.transpose(-1, -2) / 4.0, -1)
        return a @ v
class Scalars(nn.Module):
    def __init__(s):
        super().__init__(); s.l = nn.Linear(16, 16); s.scale = nn.Parameter(torch.tensor(0.5)); s.register_buffer("step", torch.tensor(3))
    def forward(s, x): return s.l(x) * s.scale + s.step.float()
class ConvNet(nn.Module):
    def __init__(s):
        super().__init__(); s.c = nn.Conv2d(2, 4, 3, padding=1); s.bn = nn.BatchNorm2d(4); s.fc = nn.Linear(4, 3)
    def forward(s, x): return s.fc(F.adaptive_avg_pool2d(F.relu(s.bn(s.c(x))), 1).flatten(1))
class RetInput(nn.Module):
    def __init__(s):
        super().__init__(); s.l = nn.Linear(16, 16)
    def forward(s, x): return x, s.l(x), x * 2
class RetParam(nn.Module):
    def __init__(s):
        super().__init__(); s.l = nn.Linear(16, 16)
    def forward(s, x): y = s.l(x); return y, y, s.l.weight.t() @ s.l.weight
class SharedSub(nn.Module):
    def __init__(s):
        super().__init__(); blk = nn.Sequential(nn.Linear(16, 16), nn.GELU()); s.blocks = nn.ModuleList([blk, blk, nn.Sequential(nn.Linear(16, 16))])
    def forward(s, x):
        for b in s.blocks: x = b(x) + x
        return x
class Residual3D(nn.Module):
    def __init__(s):
        super().__init__(); s.n = nn.LayerNorm(16); s.f = nn.Linear(16, 64); s.g = nn.Linear(64, 16); s.drop = nn.Dropout(0.0)
    def forward(s, x): return x + s.drop(s.g(F.gelu(s.f(s.n(x)))))
CASES = {
 "retinput": (RetInput, lambda: torch.randn(8, 16), True),
 "retparam": (RetParam, lambda: torch.randn(8, 16), True),
 "sharedsub": (SharedSub, lambda: torch.randn(8, 16), True),
 "residual3d": (Residual3D, lambda: torch.randn(8, 5, 16), True),
 "tied": (Tied, lambda: torch.randint(0, 32, (8, 6)), False),
 "twice": (Twice, lambda: torch.randn(8, 16), True),
 "inplace": (InPlace, lambda: torch.randn(8, 16), True),
 "nograd": (NoGradPart, lambda: torch.randn(8, 16), True),
 "multiout": (MultiOut, lambda: torch.randn(8, 16), True),
 "chunks": (Chunks, lambda: torch.randn(8, 5, 16), True),
 "scalars": (Scalars, lambda: torch.randn(8, 16), True),
 "convnet": (ConvNet, lambda: torch.randn(8, 2, 6, 6), True),
}
def flat(o):
    from torch.utils._pytree import tree_flatten
    return [t for t in tree_flatten(o)[0] if isinstance(t, torch.Tensor)]
def worker(rank, ws, port, names, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Shard
    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    from torch.distributed.tensor.placement_types import Replicate
    shape = (ws,)
    mesh = init_device_mesh("cpu", shape, mesh_dim_names=("dp", "tp")[:len(shape)])
    rest = (Replicate(),) * (len(shape) - 1)
    dp = shape[0]; me = mesh.get_coordinate()[0]
    results = {}
    for name in names:
        cls, mk, _ = CASES[name]
        try:
            torch.manual_seed(0); ref = cls()
            with torch.device("meta"): m = cls()
            torch.manual_seed(1); x = mk()
            with AutoParallel(m, mk, mesh, activation_checkpointing=mode.get("ac", "none"), bucket_collectives=mode.get("bucket", False), fuse_collectives=mode.get("fuse")) as ap:
                ap.add_parameter_memory_constraint()
                ap.add_input_constraints([(Shard(0),) + rest])
                nout = ap.joint.num_user_outputs
                ap.add_output_constraints([(Shard(0),) + rest if name != 'retparam' or i < 2 else None for i in range(nout)])
                ap.optimize_placement(); pm = ap.apply_placement(executor=mode.get("executor", "graph"))
            pm.to_empty(device="cpu")
            state = dict(ref.named_parameters()); state.update(dict(ref.named_buffers()))
            with torch.no_grad():
                for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
                    t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
            out = flat(pm(x.chunk(dp, 0)[me])); rout = flat(ref(x))
            loss = sum((o.float() * (i + 1)).sum() for i, o in enumerate(out)); loss.backward()
            rloss = sum((o.float() * (i + 1)).sum() for i, o in enumerate(rout)); rloss.backward()
            err = max((o - (r.chunk(dp, 0)[me] if o.shape != r.shape else r)).abs().max().item() for o, r in zip(out, rout))
            gerr = 0.0
            for n, p in pm.named_parameters():
                rg = state[n].grad
                g = p.grad.full_tensor() if p.grad is not None else None
                if rg is None and g is None: continue
                if rg is None: rg = torch.zeros_like(g)
                if g is None: g = torch.zeros_like(rg)
                gerr = max(gerr, ((g - rg).abs().max() / (rg.abs().max() + 1e-3)).item())
            results[name] = (err, gerr)
        except Exception as e:
            results[name] = f"{type(e).__name__}: {str(e)[:300]}"
    if rank == 0:
        q.put(results)
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", [
    {},
    {"ac": "selective"},                              # recomputed operators read buffers the forward has since overwritten
    {"ac": "full"},
    {"executor": "streams", "bucket": True},          # buckets must not mix forward gathers with backward-only ones
    {"bucket": "auto"},
    {"fuse": "all"},                                  # GEMM + collective nodes (compositions on CPU ranks)
], ids=["plain", "selective-ac", "full-ac", "streams+buckets", "priced-buckets", "fused-nodes"])
def test_structural_cases_match_single_device_on_two_ranks(mode):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    mp.spawn(worker, args=(2, free_port(), list(CASES), mode, q), nprocs=2, join=True)
    results = q.get()
    bad = {k: v for k, v in results.items() if isinstance(v, str) or v[0] > 1e-4 or v[1] > 1e-3}
    assert len(results) == len(CASES) and not bad, bad
