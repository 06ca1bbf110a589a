"""Plan and lower one small instance of every Hugging Face architecture family the reference's model-zoo
script covers (examples/run_hf_eval.sh there: decoder-only, encoder-decoder and encoder-only models on a
1-D and a 2-D mesh), built from configs so nothing is downloaded.

    python examples/run_hf_zoo.py [--mesh 8] [--only gpt2,t5] [--execute]

``--execute`` also runs rank 0's forward + backward on CPU with fake ranks (shapes only).
"""
import argparse
import os
import sys
import time
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from torch.distributed.tensor.placement_types import Replicate, Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from examples._fake import fake_mesh

D, L, H, V = 256, 2, 8, 4096  # hidden, layers, heads, vocab of every tiny instance


def _dec(cls, **kw):
    return ("causal-lm", lambda T: getattr(T, cls)(**kw))


ZOO = {
    "gpt2": _dec("GPT2Config", n_embd=D, n_layer=L, n_head=H, vocab_size=V, n_positions=512),
    "gpt_neo": _dec("GPTNeoConfig", hidden_size=D, num_layers=L, num_heads=H, vocab_size=V, attention_types=[[["global", "local"], 1]],
                    max_position_embeddings=512, window_size=64),
    "gptj": _dec("GPTJConfig", n_embd=D, n_layer=L, n_head=H, vocab_size=V, rotary_dim=16, n_positions=512),
    "gpt_neox": _dec("GPTNeoXConfig", hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D, vocab_size=V,
                     max_position_embeddings=512),
    "bloom": _dec("BloomConfig", hidden_size=D, n_layer=L, n_head=H, vocab_size=V),
    "qwen2": _dec("Qwen2Config", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                  vocab_size=V, max_position_embeddings=512),
    "phi": _dec("PhiConfig", hidden_size=D, intermediate_size=4 * D, num_hidden_layers=L, num_attention_heads=H, vocab_size=V,
                max_position_embeddings=512),
    "llama": _dec("LlamaConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                  vocab_size=V, max_position_embeddings=512),
    "stablelm": _dec("StableLmConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H,
                     num_key_value_heads=4, vocab_size=V, max_position_embeddings=512),
    "mistral": _dec("MistralConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                    vocab_size=V, max_position_embeddings=512, sliding_window=128),
    "falcon": _dec("FalconConfig", hidden_size=D, num_hidden_layers=L, num_attention_heads=H, vocab_size=V),
    "t5": ("seq2seq", lambda T: T.T5Config(d_model=D, d_ff=4 * D, num_layers=L, num_decoder_layers=L, num_heads=H, d_kv=D // H, vocab_size=V)),
    "bert": ("masked-lm", lambda T: T.BertConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                                 vocab_size=V, max_position_embeddings=512)),
    "roberta": ("masked-lm", lambda T: T.RobertaConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                                       vocab_size=V, max_position_embeddings=514)),
    "distilbert": ("masked-lm", lambda T: T.DistilBertConfig(dim=D, n_layers=L, n_heads=H, hidden_dim=4 * D, vocab_size=V,
                                                             max_position_embeddings=512)),
}


def plan_one(name, mesh, batch, seq, execute, bf16=False):
    import transformers as T

    task, make = ZOO[name]
    cfg = make(T)
    cfg.use_cache = False
    auto = {"causal-lm": T.AutoModelForCausalLM, "seq2seq": T.AutoModelForSeq2SeqLM, "masked-lm": T.AutoModelForMaskedLM}[task]
    with torch.device("meta"):
        try:
            cfg._attn_implementation = "sdpa"
            model = auto.from_config(cfg)
        except ValueError:  # architectures without a fused-attention path: explicit softmax(QK^T)V
            cfg._attn_implementation = "eager"
            model = auto.from_config(cfg)

    def ids():
        return torch.randint(0, cfg.vocab_size, (batch, seq))

    def input_fn():
        kw = {"input_ids": ids()}
        if task == "seq2seq":
            kw["decoder_input_ids"] = ids()
        return ForwardInputs((), kw)

    n_in = 2 if task == "seq2seq" else 1
    t0 = time.perf_counter()
    policy = None
    if bf16:
        from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy

        policy = MPPolicy(torch.bfloat16, torch.float32)
    with AutoParallel(model, input_fn, mesh, policy) as autop:
        autop.add_parameter_memory_constraint()
        autop.add_input_constraints([(Shard(0),) + (Replicate(),) * (mesh.ndim - 1)] * n_in)
        autop.optimize_placement()
        cost = autop.sharding_optimizer.total_cost_breakdown()
        if execute:
            pm = autop.apply_placement()
            lowered = autop.lowered
        else:
            lowered = autop.lower()
    secs = time.perf_counter() - t0
    if execute:
        pm.to_empty(device="cpu")
        with torch.no_grad():  # no checkpoint to load: small random weights, zeroed index buffers
            for t in list(pm.parameters()) + list(pm.buffers()):
                loc = t._local_tensor if hasattr(t, "_local_tensor") else t
                loc.normal_(0.0, 0.02) if loc.dtype.is_floating_point else loc.zero_()
        local = {k: v[: batch // mesh.shape[0]] for k, v in input_fn().kwargs.items()}
        out = pm(**local)
        logits = out.logits if hasattr(out, "logits") else out[0]
        logits.float().sum().backward()
    return secs, cost, lowered.num_collectives


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mesh", default="8")
    ap.add_argument("--only", default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--execute", action="store_true")
    ap.add_argument("--bf16", action="store_true", help="bf16 compute with fp32 gradient reduction")
    a = ap.parse_args()
    shape = tuple(int(x) for x in a.mesh.split(","))
    mesh = fake_mesh(shape, ("dp", "tp")[: len(shape)])
    names = a.only.split(",") if a.only else list(ZOO)
    failed = []
    for name in names:
        try:
            secs, cost, coll = plan_one(name, mesh, a.batch, a.seq_len, a.execute, a.bf16)
            print(f"PASS {name:12s} {secs:6.1f}s  total {cost['total_us']:10.1f} us  collectives {coll}", flush=True)
        except Exception as e:  # keep going: the point is the list of families that plan
            failed.append(name)
            print(f"FAIL {name:12s} {type(e).__name__}: {str(e)[:300]}", flush=True)
            if os.environ.get("ZOO_TRACEBACK"):
                traceback.print_exc()
    print(f"{len(names) - len(failed)}/{len(names)} planned" + (f"; failed: {failed}" if failed else ""))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
