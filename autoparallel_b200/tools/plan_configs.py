"""Plans the benchmark configurations on fake ranks (no GPU) and reports how long each planning stage takes.

    python -m autoparallel_b200.tools.plan_configs [--only 1,2,3] [--json out.json]

Configurations (model, mesh, global batch x sequence):
  1  GPT-2 small (12 layers, d 768), fp32, 1-D mesh of 8, 8 x 256
  2  Llama-3 8B, bf16 compute / fp32 gradient reduction, 1-D mesh dp=8, 8 x 8192
  3  Llama-3 8B, same policy, 2-D mesh dp=2 x tp=4, 4 x 8192
  4  MoE decoder (12 layers, d 2048, 64 experts top-8 + shared expert) through local_map, ep=8, 16 x 4096
  5  Llama-3 70B, 2-D mesh dp=2 x tp=4, 2 x 8192

Each configuration runs in its own process group of fake ranks, one after the other; the numbers are host
seconds of this machine.  Reference counterpart: the "Took N s" print around ``optimize_placement`` in
examples/example_llama3.py.
"""
from __future__ import annotations

import argparse
import json
import time


def _configs():
    import torch

    from ..models import gpt2, llama3, moe
    from ..parallel.frontend.mp_cast import MPPolicy

    bf16 = MPPolicy(torch.bfloat16, torch.float32)

    def gpt2_small():
        cfg = gpt2.gpt2_small() if hasattr(gpt2, "gpt2_small") else gpt2.GPT2Config()
        return gpt2.GPT2(cfg), cfg.vocab_size, False

    def llama(name):
        def make():
            cfg = getattr(llama3, name)(max_seq_len=8192)
            return llama3.Transformer(cfg), cfg.vocab_size, True

        return make

    def moe_ref():
        cfg = moe.moe_reference_config(max_seq_len=4096, ep_axis="ep")
        return moe.MoETransformer(cfg), cfg.vocab_size, True

    return {
        1: ("GPT-2 small, 1-D mesh 8", gpt2_small, (8,), ("dp",), (8, 256), None),
        2: ("Llama-3 8B, dp=8", llama("llama3_8b"), (8,), ("dp",), (8, 8192), bf16),
        3: ("Llama-3 8B, dp=2 x tp=4", llama("llama3_8b"), (2, 4), ("dp", "tp"), (4, 8192), bf16),
        4: ("MoE 64 experts via local_map, ep=8", moe_ref, (8,), ("ep",), (16, 4096), bf16),
        5: ("Llama-3 70B, dp=2 x tp=4", llama("llama3_70b"), (2, 4), ("dp", "tp"), (2, 8192), bf16),
    }


def plan(idx: int) -> dict:
    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Replicate, Shard
    from torch.testing._internal.distributed.fake_pg import FakeStore

    from .. import AutoParallel, ForwardInputs

    title, make, shape, names, (batch, seq), policy = _configs()[idx]
    world = 1
    for s in shape:
        world *= s
    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=world)
    mesh = init_device_mesh("cpu", shape, mesh_dim_names=names)
    with torch.device("meta"):
        model, vocab, with_labels = make()

    def input_fn():
        ids = torch.randint(0, vocab, (batch, seq))
        return ForwardInputs((ids,), {"labels": torch.randint(0, vocab, (batch, seq))} if with_labels else {})

    t0 = time.perf_counter()
    with AutoParallel(model, input_fn, mesh, policy, plan_device="B200") as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)] * (2 if with_labels else 1))
        ap.optimize_placement()
        t_lower = time.perf_counter()
        lowered = ap.lower()
        t_lower = time.perf_counter() - t_lower
        opt = ap.sharding_optimizer
        row = {
            "config": idx,
            "what": title,
            "trace_s": round(ap.timings["trace"], 2),
            "strategies_s": round(opt.timings["strategies"], 2),
            "costs_s": round(opt.timings["costs"], 2),
            "ilp_build_s": round(opt.timings["build"], 2),
            "ilp_solve_s": round(opt.timings["solve"], 2),
            "lower_s": round(t_lower, 2),
            "total_s": round(time.perf_counter() - t0, 2),
            "ilp": opt.problem_size,
            "collectives": lowered.num_collectives,
            "sharded_params": sum(1 for v in lowered.param_placements.values() if v and any(isinstance(p, Shard) or "Strided" in type(p).__name__ for p in v)),
            "params": len(lowered.param_placements),
        }
    dist.destroy_process_group()
    return row


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--json", default=None)
    a = ap.parse_args(argv)
    ids = [int(x) for x in a.only.split(",")] if a.only else sorted(_configs())
    rows = []
    for i in ids:
        row = plan(i)
        rows.append(row)
        print(json.dumps(row), flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
