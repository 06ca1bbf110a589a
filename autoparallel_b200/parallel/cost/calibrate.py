"""Calibration of the communication cost table from this machine's own collectives.

``python -m torch.distributed.run --nproc-per-node N -m autoparallel_b200.parallel.cost.calibrate
--out table.json [--backend symm|nccl]`` times all-gather / reduce-scatter / all-reduce /
all-to-all at a ladder of sizes with CUDA events (3 warm-ups, median of 8, max over ranks) and
writes ``{"collectives": {kind: {n: [[bytes, us], ...]}}}`` which ``Topology.load_table`` (or
``AutoParallel(cost_model=path)``) reads.  The reference calibrates inside its Inductor bucketing
pass and pickles the result (autoparallel/graph_passes/autobucketing_inductor/estimation_utils.py:
91-147, estimation.py:35-41, 176-231).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters=8):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def calibrate(sizes_mib=(0.0625, 0.25, 1, 4, 16, 64, 256), backend: str = "symm") -> dict:
    from ...runtime import comm_ops, symm

    n = dist.get_world_size()
    name = dist.group.WORLD.group_name
    if backend == "symm":
        symm.enable_for_group(dist.group.WORLD)
    C = comm_ops.ops
    table = {k: {str(n): []} for k in ("all_gather", "reduce_scatter", "all_reduce", "all_to_all")}
    for mib in sizes_mib:
        full = int(mib * (1 << 20))  # bytes of the full (gathered / pre-scatter) tensor
        elems = max(full // 2 // (n * 64), 1) * n * 64
        x_full = torch.randn(elems, device="cuda", dtype=torch.bfloat16)
        x_shard = x_full[: elems // n].clone()
        nb = elems * 2
        table["all_gather"][str(n)].append([nb, _time(lambda: C.all_gather(x_shard, 0, name, n))])
        table["reduce_scatter"][str(n)].append([nb, _time(lambda: C.reduce_scatter(x_full, 0, name, n))])
        table["all_reduce"][str(n)].append([nb, _time(lambda: C.all_reduce(x_full, name, n))])
        table["all_to_all"][str(n)].append([nb, _time(lambda: C.all_to_all(x_full.view(n, -1), 0, 0, name, n))])
    return {"backend": backend, "world_size": n, "device": torch.cuda.get_device_name(), "collectives": table}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--backend", default="symm", choices=["symm", "nccl"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    res = calibrate(backend=args.backend)
    if rank == 0:
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
        print(json.dumps(res["collectives"]["all_gather"]))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
