"""Timing of the fused GEMM+collective nodes and the stand-alone NVLink collectives against their
unfused NCCL compositions and against the roofline (the slower of FLOPs at the measured GEMM peak
and bytes over NVLink at the measured peer-copy bandwidth).

    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        -m autoparallel_b200.runtime.bench_fused [--out fused.json]

Shapes are the Llama-3 8B projections at 8192 tokens per rank.  CUDA events on the launching
stream, 3 warm-ups, median of 8, max over ranks."""
import os, sys, json, torch, torch.distributed as dist
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
from autoparallel_b200.runtime import symm, comm_ops
from autoparallel_b200.ops import cuda_impl
g = symm.enable_for_group(dist.group.WORLD)
name = dist.group.WORLD.group_name
C = comm_ops.ops
bf, f32 = torch.bfloat16, torch.float32
def R(*s, dt=bf): return (torch.randn(*s, device="cuda", dtype=f32) * 0.05).to(dt)
def unfused(fn):
    def run():
        be = comm_ops._symm_backends.pop(name)
        try: return fn()
        finally: comm_ops._symm_backends[name] = be
    return run
def timeit(fn, iters=8):
    for _ in range(3): fn()
    torch.cuda.synchronize(); dist.barrier()
    evs = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); evs.append((s, e))
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in evs)
    t = torch.tensor([ts[len(ts)//2]], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()
M = 8192
n = world
rows = []
def case(label, fused_fn, flops, link_bytes):
    tf = timeit(fused_fn); tu = timeit(unfused(fused_fn))
    t_gemm = flops / 1606.1e12 * 1e3; t_link = link_bytes / 770e9 * 1e3
    roof = max(t_gemm, t_link)
    rows.append(dict(case=label, fused_ms=tf, unfused_nccl_ms=tu, roofline_ms=roof, frac_of_roofline=roof / tf, bound="gemm" if t_gemm > t_link else "nvlink"))
    if rank == 0: print(f"{label:34s} fused {tf:7.3f} ms | NCCL+GEMM {tu:7.3f} ms | roofline {roof:6.3f} ms ({'gemm' if t_gemm>t_link else 'link'}) -> {roof/tf:.2f}", flush=True)
for (N_, K_, tag) in ((4096, 4096, "wq"), (14336, 4096, "w1"), (4096, 14336, "w2")):
    x = R(1, M, K_); w = R(N_ // n, K_)
    case(f"F1 fwd ag_mm {tag} [{M}x{N_}x{K_}]", lambda: C.ag_mm(x, w, 0, 0, bf, name, n), 2.0*M*N_*K_, (n-1)/n*N_*K_*2)
    dy = R(1, M, N_)
    case(f"F1 bwd ag_mm {tag} dgrad", lambda: C.ag_mm(dy, w, 1, 0, bf, name, n), 2.0*M*N_*K_, (n-1)/n*N_*K_*2)
    xx = R(1, M, K_)
    case(f"F2 wgrad mm_rs {tag}", lambda: C.mm_rs(dy, xx, 2, 0, f32, 1.0, name, n), 2.0*M*N_*K_, (n-1)/n*N_*K_*4)
xs = R(1, M, 4096); w1s = R(14336 // n, 4096)
case("F3 ag_mm act-gather w1/tp", lambda: C.ag_mm(xs, w1s, 2, 0, bf, name, n), 2.0*(M*n)*(14336//n)*4096, (n-1)*M*4096*2)
a = R(n, M, 14336 // n); w2s = R(4096, 14336 // n)
case("F4 mm_rs row-parallel w2/tp", lambda: C.mm_rs(a, w2s, 0, 0, bf, 1.0, name, n), 2.0*(M*n)*4096*(14336//n), (n-1)*M*4096*4)
for nb in (1 << 20, 16 << 20, 128 << 20):
    t = R(nb // 2)
    ta = timeit(lambda: C.all_gather(t, 0, name, n)); tn = timeit(unfused(lambda: C.all_gather(t, 0, name, n)))
    big = R(nb // 2 * n, dt=bf)
    tr = timeit(lambda: C.reduce_scatter(big, 0, name, n)); trn = timeit(unfused(lambda: C.reduce_scatter(big, 0, name, n)))
    if rank == 0: print(f"U1 {nb>>20:4d} MiB/rank: all_gather ours {ta:.3f} ms nccl {tn:.3f} ms | reduce_scatter ours {tr:.3f} ms nccl {trn:.3f} ms", flush=True)
    rows.append(dict(case=f"U1 {nb>>20}MiB", ag_ms=ta, ag_nccl_ms=tn, rs_ms=tr, rs_nccl_ms=trn))
# copy-engine collectives (runtime/dma.py): gathers of arena-resident shards and fp32 reduce-scatters, against NCCL
try:
    from torch.distributed.device_mesh import init_device_mesh
    from autoparallel_b200.runtime import dma
    mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    slot = 128 << 20
    arena = dma.enable_for_mesh(mesh, arena_bytes=(256 << 20) + 3 * world * slot + (1 << 20), ring=3, slot_bytes=slot, sum_ctas=48)
    dname = mesh.get_group(0).group_name
    def no_dma(fn):
        def run():
            be = comm_ops._dma_backends.pop(dname); sb = comm_ops._symm_backends.pop(name, None)
            try: return fn()
            finally:
                comm_ops._dma_backends[dname] = be
                if sb is not None: comm_ops._symm_backends[name] = sb
        return run
    for nb in (1 << 20, 16 << 20, 128 << 20):
        shard = arena.alloc((nb // 2,), bf); shard.copy_(R(nb // 2)); arena.barrier()
        ta = timeit(lambda: C.all_gather(shard, 0, dname, n)); tn = timeit(no_dma(lambda: C.all_gather(shard, 0, dname, n)))
        full = torch.randn(nb // 4 * n, device="cuda", dtype=f32) if nb * n <= (1 << 30) else None
        if full is not None and nb <= slot:
            tr = timeit(lambda: C.reduce_scatter(full, 0, dname, n)); trn = timeit(no_dma(lambda: C.reduce_scatter(full, 0, dname, n)))
        else:
            tr = trn = float("nan")
        if rank == 0: print(f"CE {nb>>20:4d} MiB/rank: all_gather copy-engine {ta:.3f} ms nccl {tn:.3f} ms | reduce_scatter(fp32) copy-engine+sum {tr:.3f} ms nccl {trn:.3f} ms", flush=True)
        rows.append(dict(case=f"CE {nb>>20}MiB", ag_ms=ta, ag_nccl_ms=tn, rs_ms=tr, rs_nccl_ms=trn))
except Exception as e:
    if rank == 0: print("copy-engine rows skipped:", type(e).__name__, str(e)[:200], flush=True)
torch.cuda.synchronize(); cuda_impl.check_status()
out = next((a.split("=", 1)[1] for a in sys.argv if a.startswith("--out=")), None)
if rank == 0 and out: json.dump(rows, open(out, "w"), indent=1)
dist.barrier(); dist.destroy_process_group()
