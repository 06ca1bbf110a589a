"""This framework's NVLink collectives (symmetric-memory kernels) against NCCL, on 2+ GPUs.

Runs as child processes (one per GPU) so the pytest process itself never joins a process group.
NVLS is off in NCCL for these tests and the kernels use plain peer loads only.
"""
import os
import subprocess
import sys

import pytest
import torch

from conftest import free_port

pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, torch, torch.distributed as dist
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from autoparallel_b200.runtime import symm, comm_ops
from autoparallel_b200.ops import cuda_impl
g = symm.enable_for_group(dist.group.WORLD, workspace_bytes=256 << 20)
name = dist.group.WORLD.group_name
def nccl(fn, *a):
    be = comm_ops._symm_backends.pop(name)
    try: return fn(*a)
    finally: comm_ops._symm_backends[name] = be
torch.manual_seed(rank)
errs = []
for it in range(3):
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(64 * world, 96, 40, device="cuda", dtype=dtype)
        for dim in (0, 1, 2):
            shape = list(x.shape); 
            a = comm_ops.ops.all_gather(x, dim, name, world); b = nccl(comm_ops._all_gather, x, dim, name, world)
            errs.append(("ag", dim, dtype, (a.float() - b.float()).abs().max().item()))
        for dim in (0, 1):
            xs = torch.randn(64 * world, 96 * world, 40, device="cuda", dtype=dtype)
            a = comm_ops.ops.reduce_scatter(xs, dim, name, world); b = nccl(comm_ops._reduce_scatter, xs, dim, name, world)
            tol = 0.1 if dtype == torch.bfloat16 else 1e-4
            errs.append(("rs", dim, dtype, (a.float() - b.float()).abs().max().item() / tol * 1e-6))
        xs = torch.randn(16 * world, 24 * world, 8, device="cuda", dtype=dtype)
        a = comm_ops.ops.all_to_all(xs, 1, 0, name, world); b = nccl(comm_ops._all_to_all, xs, 1, 0, name, world)
        errs.append(("a2a", 1, dtype, (a.float() - b.float()).abs().max().item()))
        a = comm_ops.ops.all_reduce(x, name, world); b = nccl(comm_ops._all_reduce, x, name, world)
        errs.append(("ar", 0, dtype, (a.float() - b.float()).abs().max().item() / (0.1 if dtype == torch.bfloat16 else 1e-4) * 1e-6))
    # split-phase
    x = torch.randn(1024, 512, device="cuda")
    h = comm_ops.ops.all_gather_start(x, 0, name, world); y = comm_ops.ops.comm_wait(h)
    errs.append(("ag_async", 0, torch.float32, (y - nccl(comm_ops._all_gather, x, 0, name, world)).abs().max().item()))
torch.cuda.synchronize(); cuda_impl.check_status()
bad = [e for e in errs if e[3] > 1e-6]
print("RESULT", rank, "bad", bad[:5], "n", len(errs), flush=True)
dist.barrier(); dist.destroy_process_group()
sys.exit(1 if bad else 0)
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symm_collectives_match_nccl(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
         "--master-port", str(free_port()), str(script)],
        env=env, capture_output=True, text=True, timeout=300,
    )
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "bad [(" not in r.stdout and r.stdout.count("RESULT") == n, r.stdout[-2000:]


FUSED_WORKER = r'''
import os, sys, torch, torch.distributed as dist
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from autoparallel_b200.runtime import symm
from autoparallel_b200.ops import cuda_impl
g = symm.enable_for_group(dist.group.WORLD, workspace_bytes=256 << 20)
bad = []
def gather(t):
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous()); return torch.cat(out, 0)
def check(name, got, ref, tol):
    err = (got.float() - ref.float()).abs().max().item()
    if not err <= tol: bad.append((name, err))
for it in range(3):
    torch.manual_seed(100 * it + rank)
    M, K, R = 512 + 128 * it, 320, 384
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(R, K, device="cuda", dtype=torch.bfloat16) * 0.1
    wf = gather(w)
    y, w_full = g.ag_gemm_b(x, w)
    check("ag_b w_full", w_full, wf, 0.0); check("ag_b y", y, x.float() @ wf.float().t(), 0.25)
    dy = torch.randn(M, world * R, device="cuda", dtype=torch.bfloat16)
    dx, w_full2 = g.ag_gemm_bk(dy, w)
    check("ag_bk w_full", w_full2, wf, 0.0); check("ag_bk dx", dx, dy.float() @ wf.float(), 0.5)
    xs = torch.randn(256, K, device="cuda", dtype=torch.bfloat16)
    w2 = torch.randn(512, K, device="cuda", dtype=torch.bfloat16) * 0.1
    ya, x_full = g.ag_gemm_a(xs, w2)
    xf = gather(xs)
    check("ag_a x_full", x_full, xf, 0.0); check("ag_a y", ya, xf.float() @ w2.float().t(), 0.25)
    # GEMM -> reduce-scatter: weight-gradient shape (both operands MN-major) and row-parallel shape
    T = 1024
    dyl = torch.randn(T, 256 * world, device="cuda", dtype=torch.bfloat16)
    xl = torch.randn(T, 320, device="cuda", dtype=torch.bfloat16)
    full = (dyl.float().t() @ xl.float()); dist.all_reduce(full)
    out = g.gemm_rs(dyl, xl, True, True, torch.float32)
    check("wgrad_rs", out, full[rank * 256:(rank + 1) * 256], 0.05)
    a = torch.randn(128 * world * 2, 192, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(264, 192, device="cuda", dtype=torch.bfloat16)
    full = a.float() @ b.float().t(); dist.all_reduce(full)
    out = g.gemm_rs(a, b, False, False, torch.bfloat16, scale=0.5)
    rows = a.shape[0] // world
    check("mm_rs", out, 0.5 * full[rank * rows:(rank + 1) * rows], 0.5)
torch.cuda.synchronize(); cuda_impl.check_status()
print("RESULT", rank, "bad", bad[:6], flush=True)
dist.barrier(); dist.destroy_process_group()
sys.exit(1 if bad else 0)
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_gemm_collectives(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    script = tmp_path / "worker.py"
    script.write_text(FUSED_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
         "--master-port", str(free_port()), str(script)],
        env=env, capture_output=True, text=True, timeout=300,
    )
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "bad [(" not in r.stdout and r.stdout.count("RESULT") == n, r.stdout[-2000:]


DMA_WORKER = r'''
import os, sys, torch, torch.distributed as dist
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from torch.distributed.device_mesh import init_device_mesh
from autoparallel_b200.runtime import dma, comm_ops
from autoparallel_b200.ops import cuda_impl
mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
slot = 4 << 20
arena = dma.enable_for_mesh(mesh, arena_bytes=(64 << 20) + 3 * world * slot, ring=3, slot_bytes=slot, sum_ctas=16)
name = mesh.get_group(0).group_name
g = dma._groups[name]
def nccl(fn, *a):
    be = comm_ops._dma_backends.pop(name)
    try: return fn(*a)
    finally: comm_ops._dma_backends[name] = be
bad = []
torch.manual_seed(rank)
# parameter shards live in the arena; the writer is bracketed by two barriers, as the optimizer does
shards = [arena.alloc((256, 512), torch.bfloat16), arena.alloc((3, 40, 64), torch.bfloat16), arena.alloc((1000,), torch.float32)]
for it in range(3):
    arena.barrier()
    for s in shards: s.copy_(torch.randn(s.shape, device="cuda").to(s.dtype))
    arena.barrier()
    for s in shards:
        for dim in range(s.dim()):
            if not g.can_gather(s, dim): bad.append(("not eligible", tuple(s.shape), dim)); continue
            a = comm_ops.ops.all_gather(s, dim, name, world); b = nccl(comm_ops._all_gather, s, dim, name, world)
            if not torch.equal(a, b): bad.append(("ag", tuple(s.shape), dim))
    h = comm_ops.ops.all_gather_start(shards[0], 0, name, world); y = comm_ops.ops.comm_wait(h)
    if not torch.equal(y, nccl(comm_ops._all_gather, shards[0], 0, name, world)): bad.append(("ag_async", it))
# a tensor outside the arena takes the ordinary path
x = torch.randn(64, 32, device="cuda")
if g.can_gather(x, 0): bad.append(("outside tensor accepted",))
# reduce-scatter: more calls than ring entries, sizes up to one slot, split-phase with several in flight
outs = []
for it in range(8):
    rows = world * (16 + 48 * it)
    xs = torch.randn(rows, 1024, device="cuda")
    ref = nccl(comm_ops._reduce_scatter, xs, 0, name, world)
    h = comm_ops.ops.reduce_scatter_start(xs, 0, name, world)
    outs.append((h, ref))
for h, ref in outs:
    y = comm_ops.ops.comm_wait(h)
    if not torch.allclose(y, ref, rtol=1e-5, atol=1e-4): bad.append(("rs", tuple(ref.shape), (y - ref).abs().max().item()))
big = torch.randn(world * 2048, 1024, device="cuda")  # 8 MiB per chunk > slot: not eligible, falls back
if g.can_reduce(big, 0): bad.append(("oversized reduce accepted",))
torch.cuda.synchronize(); cuda_impl.check_status()
print("RESULT", rank, "bad", bad[:6], "stats", dma.stats(), flush=True)
dist.barrier(); dist.destroy_process_group()
sys.exit(1 if bad else 0)
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_copy_engine_collectives_match_nccl(tmp_path):
    """All-gather of arena-resident shards and fp32 reduce-scatter through the copy engines against NCCL."""
    n = min(torch.cuda.device_count(), 4)
    script = tmp_path / "worker.py"
    script.write_text(DMA_WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
         "--master-port", str(free_port()), str(script)],
        env=env, capture_output=True, text=True, timeout=300,
    )
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "bad [(" not in r.stdout and r.stdout.count("RESULT") == n, r.stdout[-2000:]
