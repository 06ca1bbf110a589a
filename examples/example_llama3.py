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
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models import llama3
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
from autoparallel_b200.utils.trace_sim import estimate_graph_metrics
from autoparallel_b200.utils.visualizer import generate_visualization_html
from examples._fake import fake_mesh


def force_tp_constraints(autop) -> int:
    """Megatron-style tensor parallelism by hand: in every block wq / wk / wv / w1 / w3 are column-parallel
    (output features split over "tp"), wo / w2 row-parallel (partial sums over "tp").  Forward projections are
    found through the module path recorded on their nodes.  (Reference counterpart: the helper of the same
    purpose in examples/example_llama3.py.)"""
    apb = torch.ops.apb200
    col, row = ("wq", "wk", "wv", "w1", "w3"), ("wo", "w2")
    pinned = 0
    for node in autop.gm.graph.nodes:
        if node.op != "call_function" or node.target is not apb.mm_nd.default:
            continue
        stack = node.meta.get("nn_module_stack")
        if not stack:
            continue  # backward nodes carry the forward stack under another key
        leaf = str(list(stack.values())[-1][0]).split(".")[-1] if isinstance(stack, dict) else ""
        if leaf in col:
            autop.sharding_optimizer.add_node_constraint(node, (Shard(0), Shard(2)))
            pinned += 1
        elif leaf in row:
            autop.sharding_optimizer.add_node_constraint(node, (Shard(0), Partial()))
            pinned += 1
    return pinned


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b")
    ap.add_argument("--mesh", default="64")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--vocab-parallel", action="store_true")
    ap.add_argument("--manual-tp", action="store_true", help="pin the Megatron pattern on every block (2-D mesh)")
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
        if a.manual_tp and mesh.ndim == 2:
            n = force_tp_constraints(autop)
            print("pinned", n, "projections")
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
