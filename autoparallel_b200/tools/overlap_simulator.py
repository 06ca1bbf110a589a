"""Offline what-if tool for the overlap scheduler.

    python -m autoparallel_b200.tools.overlap_simulator --model llama3_8b --mesh 8 [--layers 4]
        [--prefetch-depth 12] [--max-in-flight-gb 2] [--bucket] [--table colls.json] [--trace out.json]
        [--save-capture step.capture.json]
    python -m autoparallel_b200.tools.overlap_simulator --replay step.capture.json [--table colls16_8.table] ...

The second form needs no model and no process group: it reloads the per-rank graphs a previous run (or a training
job, ``tools.graph_capture.save_capture``) wrote, prices the collectives through the capture's own group-name ->
mesh-dim mapping with the alpha-beta model or a measured table (this framework's JSON tables or the reference's
``colls*.table`` text tables), and reports the same numbers.

Plans the model on fake ranks (no GPU, no process group traffic), lowers it, partitions it, applies
the bucketing / overlap passes with the given knobs and reports, for forward and backward: number
of collectives by kind, simulated total / compute / communication / exposed-communication time and
peak live bytes – before and after scheduling.  Collective times come from the α–β NVLink-5 model or
from a measured table (``--table``, the format written by ``parallel.cost.calibrate``).
Reference: autoparallel/tools/overlap_simulator/run.py (replays captured graphs through Inductor's
scheduler with measured collective tables).
"""
from __future__ import annotations

import argparse
import copy
import json


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama3_70b", "llama3_debug"])
    ap.add_argument("--mesh", default="8", help="comma separated mesh shape, e.g. 8 or 2,4")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prefetch-depth", type=int, default=12)
    ap.add_argument("--max-in-flight-gb", type=float, default=2.0)
    ap.add_argument("--max-pending-reductions", type=int, default=6)
    ap.add_argument("--bucket", nargs="?", const="static", default=None, choices=["static", "auto"],
                    help="merge collectives: static size caps, or 'auto' = plan from priced collectives / compute window / memory headroom")
    ap.add_argument("--table", default=None)
    ap.add_argument("--trace", default=None)
    ap.add_argument("--device", default="B200")
    ap.add_argument("--ac", default="none", choices=["none", "selective", "full"], help="activation checkpointing mode of the plan")
    ap.add_argument("--optimizer-bytes-per-param", type=float, default=30.0,
                    help="HBM traffic of the optimizer step per local parameter element (AdamW on fp32 state with a bf16 copy: "
                         "reads p, g, m, v = 16 B, writes p, m, v + bf16 = 14 B); 0 leaves the optimizer out")
    ap.add_argument("--save-capture", default=None, help="write the partitioned per-rank graphs to this file for later --replay")
    ap.add_argument("--replay", default=None, help="simulate a saved capture instead of planning a model")
    args = ap.parse_args(argv)
    if args.replay:
        return replay(args)

    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Replicate, Shard
    from torch.testing._internal.distributed.fake_pg import FakeStore

    from .. import AutoParallel, ForwardInputs
    from ..models import llama3
    from ..parallel.frontend.mp_cast import MPPolicy
    from ..parallel.lower.partition import partition_joint
    from ..parallel.passes.overlap import OverlapConfig, exposed_collectives, schedule_for_streams
    from ..utils.trace_sim import create_execution_trace, estimate_graph_metrics

    shape = tuple(int(x) for x in args.mesh.split(","))
    world = 1
    for s in shape:
        world *= s
    if not dist.is_initialized():
        dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=world)
    mesh = init_device_mesh("cpu", shape, mesh_dim_names=("dp", "tp", "cp")[: len(shape)])
    cfg = getattr(llama3, args.model)(max_seq_len=args.seq_len)
    if args.layers:
        cfg.n_layers = args.layers
    batch = args.batch or shape[0]
    with torch.device("meta"):
        model = llama3.Transformer(cfg)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (batch, args.seq_len)),),
                             {"labels": torch.randint(0, cfg.vocab_size, (batch, args.seq_len))})

    with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), plan_device=args.device,
                      cost_model=args.table or "auto",
                      bucket_collectives={None: False, "static": True, "auto": "auto"}[args.bucket], activation_checkpointing=args.ac) as apx:
        apx.add_parameter_memory_constraint()
        apx.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)] * 2)
        apx.optimize_placement()
        lowered = apx.lower()
        parts = partition_joint(lowered.joint)
        if args.save_capture:
            from .graph_capture import save_capture

            save_capture(args.save_capture, parts.fw, parts.bw, mesh, {"model": args.model, "layers": cfg.n_layers, "seq_len": args.seq_len})
        ocfg = OverlapConfig(args.prefetch_depth, int(args.max_in_flight_gb * 2**30), args.max_pending_reductions)
        report = {"plan": {"collectives": lowered.num_collectives, "fused": apx.fusion_stats, "buckets": apx.bucket_stats,
                           "ilp_solve_s": apx.sharding_optimizer.timings.get("solve")}}
        for name, gm in (("forward", parts.fw), ("backward", parts.bw)):
            before = estimate_graph_metrics(gm, mesh, args.device)
            sched = schedule_for_streams(copy.deepcopy(gm), mesh, ocfg)
            after = estimate_graph_metrics(sched, mesh, args.device)
            report[name] = {
                "before": before.__dict__, "after": after.__dict__,
                "exposed_collectives_after": exposed_collectives(sched),
            }
            if args.trace:
                create_execution_trace(sched, mesh, args.trace.replace(".json", f"_{name}.json"), args.device)
        # the optimizer is not part of the traced graphs: a bandwidth-bound pass over the local shards of the state
        from ..parallel.cost.device import DEVICE_LIMITS

        local_params = sum(p.numel() for p in model.parameters()) / world
        opt_us = args.optimizer_bytes_per_param * local_params / DEVICE_LIMITS[args.device].bytes_per_us()
        report["optimizer_us"] = opt_us
        report["step_ms_after"] = (report["forward"]["after"]["total_us"] + report["backward"]["after"]["total_us"] + opt_us) / 1e3
        report["kernel_ms"] = (report["forward"]["after"]["compute_us"] + report["backward"]["after"]["compute_us"] + opt_us) / 1e3
    print(json.dumps(report, indent=1, default=float))
    return report


def replay(args) -> dict:
    """Simulate a saved capture: no model, no process group."""
    from ..parallel.cost import comm as comm_cost
    from ..parallel.passes.overlap import OverlapConfig, exposed_collectives, schedule_for_streams
    from ..utils.trace_sim import make_runtime_estimator, simulate
    from .graph_capture import load_capture, load_colls_table

    cap = load_capture(args.replay)
    topo = comm_cost.Topology([comm_cost.NVLINK5] * len(cap["mesh_shape"]))
    if args.table:
        if args.table.endswith(".table"):
            topo.tables.update(load_colls_table(args.table))
        else:
            topo.load_table(args.table)
    est = make_runtime_estimator(None, args.device, group_dim=cap["group_dim"], topology=topo)
    ocfg = OverlapConfig(args.prefetch_depth, int(args.max_in_flight_gb * 2**30), args.max_pending_reductions)
    report = {"capture": {"mesh_shape": cap["mesh_shape"], "group_dim": cap["group_dim"], **cap.get("extra", {})},
              "table": args.table or "alpha-beta NVLink 5 model"}
    for name, gm in (("forward", cap["forward_gm"]), ("backward", cap["backward_gm"])):
        if gm is None:
            continue
        before = simulate(gm, est)
        sched = schedule_for_streams(copy.deepcopy(gm), None, ocfg)
        events: list = []
        after = simulate(sched, est, events)
        report[name] = {"before": before.__dict__, "after": after.__dict__, "exposed_collectives_after": exposed_collectives(sched)}
        if args.trace:
            with open(args.trace.replace(".json", f"_{name}.json"), "w") as f:
                json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    report["step_ms_after"] = sum(report[k]["after"]["total_us"] for k in ("forward", "backward") if k in report) / 1e3
    print(json.dumps(report, indent=1, default=float))
    return report


if __name__ == "__main__":
    main()
