"""Plan Llama-3 8B / 70B on 64 fake ranks, 1-D or 2-D, optionally with a vocab-parallel output
constraint; print the plan summary, simulated step metrics and write the HTML report.
(Reference counterpart: examples/example_llama3.py.)

    python examples/example_llama3.py --model llama3_8b --mesh 8,8 --vocab-parallel --layers 4
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models import llama3
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
from autoparallel_b200.utils.trace_sim import estimate_graph_metrics
from autoparallel_b200.utils.visualizer import generate_visualization_html
from examples._fake import fake_mesh


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--mesh", default="64")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--vocab-parallel", action="store_true")
    ap.add_argument("--html", default=None)
    a = ap.parse_args()
    shape = tuple(int(x) for x in a.mesh.split(","))
    mesh = fake_mesh(shape, ("dp", "tp")[: len(shape)])
    cfg = getattr(llama3, a.model)(max_seq_len=a.seq_len)
    cfg.n_layers = a.layers
    with torch.device("meta"):
        model = llama3.Transformer(cfg)
    batch = shape[0] * 2

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (batch, a.seq_len)),))

    with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), plan_device="B200") as autop:
        autop.add_parameter_memory_constraint()
        x_pl = (Shard(0),) + (Replicate(),) * (mesh.ndim - 1)
        autop.add_input_constraints([x_pl])
        out_pl = (Shard(0), Shard(2)) if (a.vocab_parallel and mesh.ndim == 2) else x_pl
        autop.add_output_constraints([out_pl])
        autop.optimize_placement()
        opt = autop.sharding_optimizer
        print("ILP:", opt.problem_size, {k: round(v, 2) for k, v in opt.timings.items()})
        print("cost:", opt.total_cost_breakdown())
        lowered = autop.lower()
        print("collectives:", lowered.num_collectives, "fused:", autop.fusion_stats)
        print("simulated joint graph:", estimate_graph_metrics(lowered.gm, mesh, "B200"))
        if a.html:
            with open(a.html, "w") as f:
                f.write(generate_visualization_html(opt.get_json(), f"{a.model} on mesh {shape}"))
            print("wrote", a.html)


if __name__ == "__main__":
    main()
