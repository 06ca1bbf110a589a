"""MoE decoder with expert parallelism through ``local_map``.  Fake ranks by default; under
torchrun it runs real steps on NCCL (or gloo with --cpu).
(Reference counterpart: examples/example_ds3_local_map.py.)

    python examples/example_moe_local_map.py
    torchrun --nproc-per-node 4 examples/example_moe_local_map.py --real
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models.moe import MoETransformer, moe_debug


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--real", action="store_true")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--zipf", type=float, default=None)
    a = ap.parse_args()
    if a.real:
        backend = "gloo" if a.cpu else "nccl"
        if not a.cpu:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group(backend)
        world = dist.get_world_size()
        mesh = init_device_mesh("cpu" if a.cpu else "cuda", (world,), mesh_dim_names=("ep",))
    else:
        from examples._fake import fake_mesh

        world = 8
        mesh = fake_mesh((8,), ("ep",))
    cfg = moe_debug(num_experts=max(8, world), router_bias_zipf=a.zipf)
    B, S = 2 * world, 64
    with torch.device("meta"):
        model = MoETransformer(cfg)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (B, S)),), {"labels": torch.randint(0, cfg.vocab_size, (B, S))})

    with AutoParallel(model, input_fn, mesh) as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0),)] * 2)
        autop.optimize_placement()
        parallel = autop.apply_placement()
        if not a.real or dist.get_rank() == 0:
            print("collectives:", autop.lowered.num_collectives)
    if a.real:
        dev = "cpu" if a.cpu else "cuda"
        parallel.to_empty(device=dev)
        parallel.init_weights(seed=0)
        tok = torch.randint(0, cfg.vocab_size, (B // world, S), device=dev)
        for step in range(3):
            loss = parallel(tok, labels=tok)
            loss.backward()
            if dist.get_rank() == 0:
                print("step", step, "loss", loss.item())
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
