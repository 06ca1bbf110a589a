"""Plan a Hugging Face causal LM built from a config (no download): GPT-2 by default.
(Reference counterpart: examples/example_hf.py / run_hf_eval.sh.)

    python examples/example_hf.py --model gpt2 --mesh 8
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from examples._fake import fake_mesh

CONFIGS = {
    "gpt2": lambda T: T.GPT2Config(),
    "gpt2-medium": lambda T: T.GPT2Config(n_embd=1024, n_layer=24, n_head=16),
    "llama-tiny": lambda T: T.LlamaConfig(hidden_size=512, intermediate_size=1376, num_hidden_layers=4, num_attention_heads=8,
                                          num_key_value_heads=4, vocab_size=32000),
    "qwen2-tiny": lambda T: T.Qwen2Config(hidden_size=512, intermediate_size=1376, num_hidden_layers=4, num_attention_heads=8,
                                          num_key_value_heads=4, vocab_size=32000),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2", choices=list(CONFIGS))
    ap.add_argument("--mesh", default="8")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=256)
    a = ap.parse_args()
    import transformers as T

    shape = tuple(int(x) for x in a.mesh.split(","))
    mesh = fake_mesh(shape, ("dp", "tp")[: len(shape)])
    cfg = CONFIGS[a.model](T)
    cfg.use_cache = False
    cfg._attn_implementation = "sdpa"
    with torch.device("meta"):
        model = T.AutoModelForCausalLM.from_config(cfg)

    def input_fn():
        return ForwardInputs((), {"input_ids": torch.randint(0, cfg.vocab_size, (a.batch, a.seq_len))})

    with AutoParallel(model, input_fn, mesh) as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)])
        autop.optimize_placement()
        print(a.model, "ILP", autop.sharding_optimizer.problem_size, autop.sharding_optimizer.total_cost_breakdown())
        lowered = autop.lower()
        print("collectives:", lowered.num_collectives)


if __name__ == "__main__":
    main()
