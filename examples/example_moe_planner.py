"""MoE decoder whose routed experts are ordinary graph nodes (``expert_mode="planner"``): the solver itself decides
where the token buffer moves to the experts.  Prints the placements it chose for one layer's MoE operators.
(Reference counterpart: examples/native_ds3/, where the expert ops are visible to the ILP.)

    python examples/example_moe_planner.py [--mesh 8] [--dim 1024]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models.moe import MoETransformer, moe_debug
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
from examples._fake import fake_mesh


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mesh", default="8")
    ap.add_argument("--dim", type=int, default=1024)
    ap.add_argument("--seq-len", type=int, default=1024)
    a = ap.parse_args()
    shape = tuple(int(x) for x in a.mesh.split(","))
    mesh = fake_mesh(shape, ("dp", "ep")[: len(shape)])
    cfg = moe_debug(expert_mode="planner", num_experts=8, dispatch_blocks=8, dim=a.dim, expert_hidden=a.dim // 2, n_heads=8,
                    max_seq_len=a.seq_len)
    B = 8
    with torch.device("meta"):
        model = MoETransformer(cfg)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (B, a.seq_len)),),
                             {"labels": torch.randint(0, cfg.vocab_size, (B, a.seq_len))})

    with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), plan_device="B200") as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)] * 2)
        sol = autop.optimize_placement()
        seen = set()
        for n in autop.gm.graph.nodes:
            t = str(n.target)
            if n.op == "call_function" and ("moe_" in t or "grouped_mm" in t) and t not in seen:
                seen.add(t)
                spec = sol[n]
                outs = spec.output_specs
                print(f"{t.split('.')[1]:18s} in {[str(tuple(i.placements)) for i in spec.input_specs]} -> "
                      f"{tuple(outs.placements) if not isinstance(outs, (tuple, list)) else [tuple(o.placements) for o in outs]}")
        lowered = autop.lower()
        print("collectives:", lowered.num_collectives)


if __name__ == "__main__":
    main()
