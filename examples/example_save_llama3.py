"""Save a solved plan (full optimizer state and the small placements file), reload both without a
model or process group, and re-apply the placements to a fresh optimizer.
(Reference counterpart: examples/example_save_llama3.py, docs/save_load.md.)"""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models import llama3
from autoparallel_b200.parallel.solver.ilp import ShardingOptimizer
from examples._fake import fake_mesh


def plan(mesh, cfg):
    with torch.device("meta"):
        model = llama3.Transformer(cfg)
    return AutoParallel(model, lambda: ForwardInputs((torch.randint(0, cfg.vocab_size, (16, 256)),)), mesh, plan_device="B200")


def main():
    mesh = fake_mesh((8,), ("dp",))
    cfg = llama3.llama3_debug(n_layers=4)
    d = tempfile.mkdtemp()
    with plan(mesh, cfg) as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0),)])
        autop.optimize_placement()
        autop.sharding_optimizer.save(os.path.join(d, "optimizer.pt"))
        autop.sharding_optimizer.save_placements(os.path.join(d, "placements.json"))
        obj = autop.sharding_optimizer.objective_value
    for f in os.listdir(d):
        print(f, os.path.getsize(os.path.join(d, f)), "bytes")
    loaded = ShardingOptimizer.load(os.path.join(d, "optimizer.pt"))
    print("reloaded objective", loaded.objective_value, "== saved", obj, "; re-solve:", round(loaded.total_cost(), 2))
    loaded.resolve()
    with plan(mesh, cfg) as autop2:  # same graph, no solve: just apply the stored placements
        autop2.add_parameter_memory_constraint()
        sol = autop2.sharding_optimizer.load_placements(os.path.join(d, "placements.json"))
        parallel = autop2.apply_placement(sol)
    print("applied stored placements:", type(parallel).__name__, len(list(parallel.parameters())), "parameters")


if __name__ == "__main__":
    main()
