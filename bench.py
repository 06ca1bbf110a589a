"""Headline benchmark: Llama-3 8B training tokens/s under the auto-chosen plan.

    python bench.py --gpus N --steps K --warmup W            (N=1; for N>1 launch with torchrun)
    python bench.py --impl reference ...                      (the unmodified reference, if installed)

Every rank builds the model on the meta device, plans it with ``AutoParallel`` (parameter-memory
constraint -> FSDP on the 1-D ``dp`` mesh, bf16 compute / fp32 gradient reduction), materialises
its shards, and runs K timed optimizer steps on synthetic tokens (weak scaling: one 8192-token
sequence per GPU).  Rank 0 prints ONE JSON line.  ``value`` is device-timed with CUDA events over
steps whose inputs are already on the device; ``e2e`` repeats the measurement through the public
API with a pinned-host -> device copy of the inputs and a device -> host read of the loss in every
step.  The per-step working set (16 GB of bf16 weights re-read, tens of GB of activations) is far
larger than the 126 MB L2, so no explicit flush is issued between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S = None  # the reference publishes no throughput number


def _free_port() -> int:
    """A TCP port that is free right now (single-process rendezvous on 127.0.0.1; a fixed port collides
    when two jobs share a host).  Under torchrun MASTER_PORT is already set and this is not used."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="benchmark configuration: 2 = Llama-3 8B on a 1-D dp mesh (the headline; default), 3 = Llama-3 8B on "
                         "dp=2 x tp=4 with global batch 4 x 8192, 4 = MoE decoder (64 experts, top-8, shared expert) with expert "
                         "parallelism through local_map and global batch 16 x 4096, 5 = Llama-3 70B on dp=2 x tp=4 with activation "
                         "checkpointing, a parameter-memory budget and global batch 8 x 4096.  3-5 need 8 GPUs and print their own "
                         "metric name, never the headline's")
    ap.add_argument("--prefetch-discount", type=float, default=None,
                    help="scale the planner's price of parameter gathers (0 = free: they are prefetched by the copy engines / the "
                         "overlap scheduler); default: not applied")
    ap.add_argument("--zipf", type=float, default=None, help="config 4: Zipf(s) router bias over the experts (skewed load)")
    ap.add_argument("--ref-mode", default="auto", choices=["auto", "compile", "compile_ac", "eager"],
                    help="reference arm only: auto tries the reference driver's torch.compile backend, then the same with its "
                         "activation-checkpointing pass, then the eager module")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="capture forward + backward + optimizer in one CUDA graph and replay it (runtime/graph_step.py); auto: on "
                         "one GPU; on: also with NCCL collectives or copy-engine gathers inside the graph")
    ap.add_argument("--kernel-table", default=None, metavar="PATH",
                    help="after the timed regions, run ONE more step under torch.profiler and write the device time per "
                         "kernel name (JSON) to PATH; never part of a reported number")
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama3_debug", "llama3_1b"])
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None, help="debugging only: override the layer count (invalidates the metric)")
    ap.add_argument("--ac", default="auto", choices=["auto", "none", "selective", "full"])
    ap.add_argument("--executor", default="streams", choices=["graph", "streams"])
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "symm", "hybrid", "dma", "dma_ag", "dma_fused"],
                    help="nccl: NCCL collectives under the overlap scheduler; symm: own NVLink kernels for everything, GEMMs fused "
                         "with their collective; hybrid: fused GEMM+collective kernels, stand-alone collectives on NCCL; "
                         "dma: parameter gathers and gradient reduce-scatters on the copy engines (no SM); dma_ag: copy-engine "
                         "gathers, NCCL reductions; dma_fused: copy-engine gathers, weight-gradient GEMM fused with its reduce-scatter")
    ap.add_argument("--dma-ring", type=int, default=4, help="copy-engine reduce-scatter: staging entries in flight")
    ap.add_argument("--dma-sum-ctas", type=int, default=48, help="copy-engine reduce-scatter: CTAs of the kernel that adds the slots")
    ap.add_argument("--reduction-group", default="separate", choices=["separate", "shared"],
                    help="separate: gradient reductions run on a second NCCL communicator so that parameter gathers never queue behind them")
    ap.add_argument("--dynamic-tiles", default=None, choices=["on", "off"],
                    help="hand GEMM tiles to the CTA pairs at run time (a pair that shares its SMs with a collective's kernel takes fewer)")
    ap.add_argument("--nccl-priority", default="high", choices=["high", "normal"],
                    help="priority of the NCCL streams: with 'high' a collective's CTAs are placed first whenever SMs free up")
    ap.add_argument("--prefetch-depth", type=int, default=None, help="overlap scheduler: parameter gathers issued ahead of use")
    ap.add_argument("--max-in-flight-gb", type=float, default=None, help="overlap scheduler: gathered-but-unused bytes allowed")
    ap.add_argument("--pending-reductions", type=int, default=None, help="overlap scheduler: gradient reductions left pending before one is waited for")
    ap.add_argument("--yield-pairs", type=int, default=None,
                    help="SM pairs the GEMM kernels give up for each NCCL collective issued beside them (needs --dynamic-tiles on)")
    ap.add_argument("--emit-bf16", default="on", choices=["on", "off"],
                    help="AdamW also writes each updated parameter as bf16 (2 bytes/param more memory); the forward and "
                         "backward casts of the parameters then cost no kernel")
    ap.add_argument("--gemm-stages", type=int, default=None, choices=[4, 5, 6],
                    help="TMA stages of the CTA-pair GEMM; fewer leave shared memory for an NCCL CTA beside each GEMM CTA")
    ap.add_argument("--reserve-sms", type=int, default=None,
                    help="SMs the GEMM kernels leave idle for NCCL kernels on other streams, which are then capped to as many CTAs "
                         "(default 0: measured slower at N=2, 492 ms with 16 and 523 ms with 8 against 468 ms with none)")
    return ap.parse_args()


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons, power = [], [], set(), []
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def write_kernel_table(path, step_fn, rank):
    """One step under torch.profiler (after all timing); device time aggregated per kernel name."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step_fn(0)
        torch.cuda.synchronize()
    if rank != 0:
        return
    agg = collections.defaultdict(lambda: [0, 0.0])
    t_min, t_max = None, None
    for ev in prof.events():
        if ev.device_type.name != "CUDA" and "cuda" not in str(ev.device_type).lower():
            continue
        dur = float(getattr(ev, "device_time_total", 0.0) or getattr(ev, "cuda_time_total", 0.0) or 0.0)
        if dur <= 0:
            continue
        agg[ev.name][0] += 1
        agg[ev.name][1] += dur
    rows = sorted(({"kernel": k, "launches": n, "total_us": round(t, 1)} for k, (n, t) in agg.items()), key=lambda r: -r["total_us"])
    with open(path, "w") as f:
        json.dump({"sum_of_kernel_us": round(sum(r["total_us"] for r in rows), 1), "kernels": rows}, f, indent=1)


def _dma_stats():
    try:
        from autoparallel_b200.runtime import dma

        return dma.stats() if dma.arena() is not None else {}
    except Exception:
        return {}


def _teardown(graphed=None, limit_s: float = 20.0) -> None:
    """Leave the job: release the captured step first (a CUDA graph that holds collective kernels must be gone before
    its communicator is destroyed), then the process group.  The result line has been printed by now; if the
    teardown itself does not finish within ``limit_s`` the process exits anyway instead of holding the GPUs."""
    import threading

    import torch
    import torch.distributed as dist

    sys.stdout.flush()
    sys.stderr.flush()
    timer = threading.Timer(limit_s, lambda: os._exit(0))
    timer.daemon = True
    timer.start()
    try:
        if graphed is not None:
            graphed.release()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.destroy_process_group()
    finally:
        timer.cancel()


def run_ours(args):
    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Shard

    from autoparallel_b200 import AutoParallel, ForwardInputs
    from autoparallel_b200.models import llama3
    from autoparallel_b200.ops import cuda_impl
    from autoparallel_b200.optim import AdamW
    from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}"
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    reserve = args.reserve_sms
    if reserve is None:
        # hybrid: NCCL kernels and peer-waiting fused kernels share the GPU, so NCCL gets SMs of its own
        reserve = int(os.environ.get("APB200_RESERVE_SMS", "16" if args.comm == "hybrid" else "0")) if world > 1 else 0
    if reserve > 0:
        # NCCL kernels get as many CTAs as the GEMM kernels leave SMs free (a persistent GEMM CTA owns
        # its SM's shared memory, so a collective launched beside it would otherwise wait for a GEMM to end)
        os.environ.setdefault("NCCL_MAX_CTAS", str(reserve))
    pg_opts = None
    if world > 1 and args.nccl_priority == "high":
        pg_opts = dist.ProcessGroupNCCL.Options()
        pg_opts.is_high_priority_stream = True
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank), pg_options=pg_opts)
    if args.config in (3, 5):
        # the named mesh is dp=2 x tp=4 (8 GPUs); on 4 GPUs the same configuration runs on dp=2 x tp=2 and says so
        assert world in (4, 8), f"config {args.config} is defined on a dp=2 x tp=4 mesh: launch on 8 GPUs (or 4 for dp=2 x tp=2)"
        mesh = init_device_mesh("cuda", (2, world // 2), mesh_dim_names=("dp", "tp"))
    elif args.config == 4:
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("ep",))
    else:
        mesh = init_device_mesh("cuda", (world,), mesh_dim_names=("dp",))
    data_ranks = mesh.shape[0]            # ranks the batch is split over (the first mesh dim)
    data_rank = mesh.get_local_rank(0)
    cuda_impl.ensure_loaded()
    cuda_impl.extension().gemm_set_reserved_sms(reserve)
    if args.gemm_stages is not None:
        cuda_impl.extension().gemm_set_pair_stages(args.gemm_stages)
    # measured at N=2 on one box: 463.8 ms with dynamic tiles + high-priority NCCL streams, 468.2 ms without
    dynamic_tiles = (args.dynamic_tiles == "on") if args.dynamic_tiles is not None else world > 1
    cuda_impl.extension().gemm_set_dynamic_tiles(dynamic_tiles)
    yield_pairs = args.yield_pairs if args.yield_pairs is not None else 0
    if world > 1 and dynamic_tiles and yield_pairs > 0:
        from autoparallel_b200.runtime import comm_ops as _co

        _co.set_sm_yield(yield_pairs)

    model_name = args.model
    if args.config == 4:
        from autoparallel_b200.models import moe

        S = 4096 if args.seq_len == 8192 else args.seq_len
        cfg = moe.moe_reference_config(max_seq_len=S, ep_axis="ep", router_bias_zipf=args.zipf)
        if args.layers is not None:
            cfg.n_layers = args.layers
        B_global = 2 * world  # 16 sequences of 4096 on 8 ranks
        model_name = "moe_64e_top8" + (f"_zipf{args.zipf:g}" if args.zipf else "")
        with torch.device("meta"):
            model = moe.MoETransformer(cfg)
    else:
        if args.config == 5:
            model_name = "llama3_70b"
            S = 4096 if args.seq_len == 8192 else args.seq_len
            cfg = llama3.llama3_70b(max_seq_len=S)
            B_global = 8
        else:
            cfg = {"llama3_8b": llama3.llama3_8b, "llama3_debug": llama3.llama3_debug,
                   "llama3_1b": lambda **kw: llama3.llama3_8b(dim=2048, n_layers=16, n_heads=16, n_kv_heads=8, ffn_hidden=8192, **kw)}[args.model](
                max_seq_len=args.seq_len)
            S = args.seq_len
            # config 2: one sequence per GPU (weak scaling; dp=8 gives the named global batch of 8); config 3: 4 x 8192
            B_global = 4 if args.config == 3 else world
        if args.layers is not None:
            cfg.n_layers = args.layers
        with torch.device("meta"):
            model = llama3.Transformer(cfg)
    B_local = B_global // data_ranks

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (B_global, S)),),
                             {"labels": torch.randint(0, cfg.vocab_size, (B_global, S))})

    ac = args.ac
    if ac == "auto":
        # one GPU holds fp32 params + grads + Adam moments (16 B/param): recompute cheap ops there
        n_params = sum(p.numel() for p in model.parameters())
        ac = "full" if args.config == 5 else ("selective" if world == 1 and n_params > 4e9 else "none")
    fuse_arg = None
    comm_mode = args.comm
    if comm_mode == "auto":
        # Measured on this model, one box per row (ms/step, NCCL under the overlap scheduler vs copy-engine collectives):
        # N=2 453.1 / 453.7, N=8 477.7 / 460.3.  The copy-engine mode is the default above one GPU: parameter gathers
        # and gradient reduce-scatters move with the copy engines and take no SM from the persistent GEMMs; tensors it
        # does not cover (and a machine without peer access) fall back to NCCL.
        comm_mode = os.environ.get("APB200_COMM", "dma" if world > 1 else "nccl")
    shadow_arena = None
    if world > 1 and comm_mode.startswith("dma"):
        from autoparallel_b200.runtime import dma

        local_param_bytes = sum(p.numel() for p in model.parameters()) * 2 // world + (256 << 10) * len(list(model.parameters()))
        # one staging slot holds one rank's chunk of the largest per-layer weight gradient (fp32)
        layer_max = max((p.numel() for n_, p in model.named_parameters() if "layers." in n_), default=0)
        slot = ((layer_max * 4 // world + 4095) // 4096) * 4096 if comm_mode == "dma" else 0
        arena_bytes = local_param_bytes + (64 << 20) + args.dma_ring * world * slot
        try:
            shadow_arena = dma.enable_for_mesh(mesh, arena_bytes, ring=args.dma_ring, slot_bytes=slot, sum_ctas=args.dma_sum_ctas,
                                               reductions=(comm_mode == "dma"))
        except Exception as e:  # no peer access / symmetric memory on this machine
            if rank == 0:
                print(f"peer arena unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr, flush=True)
            dma.disable_all()
            comm_mode = "nccl"
    if world > 1 and comm_mode in ("symm", "hybrid", "dma_fused"):
        # communicators first: the planner fuses a GEMM with its collective only where they exist
        from autoparallel_b200.runtime import symm

        try:
            symm.enable_for_mesh(mesh)
            symm.route_standalone_collectives(comm_mode == "symm")
            fuse_arg = "reductions" if comm_mode == "dma_fused" else None
        except Exception as e:  # no peer access / symmetric memory on this machine: NCCL carries everything
            if rank == 0:
                print(f"symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr, flush=True)
            symm.disable_all()
            comm_mode = "nccl"
    if world > 1 and args.reduction_group == "separate":
        from autoparallel_b200.runtime import comm_ops

        comm_ops.use_separate_reduction_groups(mesh, pg_options=pg_opts)
    t0 = time.perf_counter()
    with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), activation_checkpointing=ac,
                      fuse_collectives=fuse_arg) as ap:
        from torch.distributed.tensor.placement_types import Replicate

        if args.config == 5:
            # 180 GB per GPU: fp32 master + gradient + two Adam moments (16 B per element held) may take 150 GB of it
            ap.add_parameter_memory_constraint(budget_bytes=150e9, bytes_per_element=16.0)
        else:
            ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)] * 2)
        if args.prefetch_discount is not None:
            ap.sharding_optimizer.apply_prefetch_discount(args.prefetch_discount)
        ap.optimize_placement()
        from autoparallel_b200.parallel.passes.overlap import OverlapConfig

        ocfg = OverlapConfig()
        if args.prefetch_depth is not None:
            ocfg.prefetch_depth = args.prefetch_depth
        if args.max_in_flight_gb is not None:
            ocfg.max_in_flight_bytes = int(args.max_in_flight_gb * 2**30)
        if args.pending_reductions is not None:
            ocfg.max_pending_reductions = args.pending_reductions
        pm = ap.apply_placement(executor=args.executor, overlap_config=ocfg)
        timings = dict(ap.timings)
        solver = ap.sharding_optimizer
        ilp_solve_s = solver.timings.get("solve")
        n_coll = dict(ap.lowered.num_collectives)
        fused_nodes = dict(ap.fusion_stats)
    plan_s = time.perf_counter() - t0
    pm.to_empty(device="cuda")
    pm.init_weights(seed=0)
    # config 5 (70B on 8 GPUs) has no room for a second, bf16 copy of the parameters: 16 B/element already take 140 GB
    emit = args.emit_bf16 == "on" and args.config != 5
    opt = AdamW(pm.parameters(), lr=3e-4, weight_decay=0.1, emit_bf16=emit, shadow_arena=shadow_arena)

    g = torch.Generator(device="cpu").manual_seed(1234 + data_rank)  # ranks that share a batch shard draw the same tokens
    n_sets = 4
    host = [(torch.randint(0, cfg.vocab_size, (B_local, S), generator=g).pin_memory(),
             torch.randint(0, cfg.vocab_size, (B_local, S), generator=g).pin_memory()) for _ in range(n_sets)]
    devs = [(t.cuda(), l.cuda()) for t, l in host]

    def step_device(i):
        tok, lab = devs[i % n_sets]
        loss = pm(tok, labels=lab)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def step_e2e(i):
        t, l = host[i % n_sets]
        tok = t.cuda(non_blocking=True)
        lab = l.cuda(non_blocking=True)
        loss = pm(tok, labels=lab)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.item()  # device -> host read of the step's result

    for i in range(args.warmup):
        step_device(i)
    torch.cuda.synchronize()
    cuda_impl.check_status()

    graphed = None
    # auto: one GPU only.  With collectives inside the graph the device-side gain is under one per cent (the step is
    # energy-bound) and a communicator must not be destroyed while a graph holds its kernels: --graph on asks for it.
    replayable = world == 1
    if args.graph == "on" or (args.graph == "auto" and replayable):
        from autoparallel_b200.runtime.graph_step import GraphedTrainStep

        try:
            graphed = GraphedTrainStep(pm, opt, (devs[0][0],), {"labels": devs[0][1]})
        except Exception as e:  # capture refused (a collective that cannot be replayed, memory): stay eager
            if args.graph == "on":
                raise
            if rank == 0:
                print(f"CUDA-graph capture unavailable ({type(e).__name__}: {str(e)[:200]}); eager step", file=sys.stderr, flush=True)
            graphed = None
        if world > 1:
            ok = torch.tensor([1 if graphed is not None else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                graphed = None
    if graphed is not None:
        def step_device(i):  # noqa: F811
            tok, lab = devs[i % n_sets]
            return graphed(tok, labels=lab)

        def step_e2e(i):  # noqa: F811
            t, l = host[i % n_sets]
            return graphed(t, labels=l).item()  # pinned host -> static device buffers, replay, loss read back

        for i in range(2):
            step_device(i)
        torch.cuda.synchronize()
        cuda_impl.check_status()

    def timed(fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = cuda_impl.launch_count
        s.record()
        last = None
        for i in range(steps):
            last = fn(i)
        e.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([s.elapsed_time(e)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), cuda_impl.launch_count - l0, last

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev, launches, last = timed(step_device, args.steps)
    ms_e2e, _, last_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    cuda_impl.check_status()
    peak_mem = torch.cuda.max_memory_allocated() / 2**30
    tokens = B_global * S * args.steps
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    if rank == 0:
        flops_tok = cfg.flops_per_token(S) if hasattr(cfg, "flops_per_token") else 0
        headline = args.config == 2 and args.model == "llama3_8b" and args.layers is None
        mesh_desc = " x ".join(f"{n}={s_}" for n, s_ in zip(mesh.mesh_dim_names, mesh.shape))
        out = {
            "metric": "Llama-3-8B train tokens/s (auto plan)" if headline else f"{model_name} train tokens/s on {mesh_desc} (auto plan; config {args.config}, NOT the headline config)",
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_dev / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16",
            "data": "synthetic",
            "impl": "ours",
            "config": {
                "model": model_name if args.layers is None else f"{model_name}[{args.layers} layers]",
                "global_batch": B_global,
                "seq_len": S,
                "parallelism": (f"dp{world} (plan chosen by the ILP: FSDP, bf16 compute, fp32 grad reduce)" if args.config == 2
                                else f"{mesh_desc} (plan chosen by the ILP, bf16 compute, fp32 grad reduce)"),
                "optimizer": "AdamW (fp32 state, in the timed region)",
                "activation_checkpointing": ac,
                "executor": args.executor + (" + whole-step CUDA graph" if graphed is not None else ""),
                "comm": comm_mode if world > 1 else "none",
                "reserved_sms_for_comm": reserve,
                "overlap": {"prefetch_depth": ocfg.prefetch_depth, "max_in_flight_gib": round(ocfg.max_in_flight_bytes / 2**30, 2),
                            "pending_reductions": ocfg.max_pending_reductions},
                "planner_prefetch_discount": args.prefetch_discount,
                "sm_pairs_yielded_per_collective": yield_pairs if world > 1 and dynamic_tiles else 0,
                "optimizer_emits_bf16_params": emit,
                "gemm_stages": cuda_impl.extension().gemm_get_pair_stages(),
                "gemm_dynamic_tiles": bool(cuda_impl.extension().gemm_get_dynamic_tiles()),
                "nccl_stream_priority": args.nccl_priority if world > 1 else "none",
                "reduction_group": args.reduction_group if world > 1 else "none",
                "fused_nodes": fused_nodes,
                "collectives_in_graph": n_coll,
                "copy_engine_collectives": _dma_stats(),
                "l2": "no explicit flush: per-step working set (>=16 GB of weights + activations) >> 126 MB L2",
            },
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 2 * B_local * S * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "library_fallbacks": dict(cuda_impl.library_fallbacks),
            "clocks": clocks,
            "ilp_solve_s": ilp_solve_s,
            "plan_s": {k: round(v, 3) for k, v in timings.items()},
            "plan_total_s": round(plan_s, 2),
            "mfu_vs_nominal_2250": (value / world * flops_tok / 2.25e15) if flops_tok else None,
            "peak_mem_gib": round(peak_mem, 1),
            "final_loss": float(last_e2e),
        }
        print(json.dumps(out), flush=True)
    if args.kernel_table:
        write_kernel_table(args.kernel_table, step_device, rank)
    _teardown(graphed)


def run_reference(args):
    from baseline.reference_arm import run

    run(args)


if __name__ == "__main__":
    a = parse()
    if a.comm.startswith("dma") or a.comm == "auto":
        # one hardware queue per stream: a bounded flag wait on a communication stream must never sit in front
        # of compute kernels of another stream in a shared queue (read once, when the CUDA context is created)
        os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
