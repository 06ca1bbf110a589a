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
    "opt": _dec("OPTConfig", hidden_size=D, ffn_dim=4 * D, num_hidden_layers=L, num_attention_heads=H, vocab_size=V, word_embed_proj_dim=D,
                max_position_embeddings=512),
    "gpt_bigcode": _dec("GPTBigCodeConfig", n_embd=D, n_layer=L, n_head=H, vocab_size=V, n_positions=512),
    "gemma": _dec("GemmaConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                  head_dim=32, vocab_size=V, max_position_embeddings=512),
    "gemma2": _dec("Gemma2Config", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                   head_dim=32, vocab_size=V, max_position_embeddings=512, sliding_window=128),
    "phi3": _dec("Phi3Config", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                 vocab_size=V, max_position_embeddings=512, original_max_position_embeddings=512, pad_token_id=0),
    "qwen3": _dec("Qwen3Config", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                  head_dim=32, vocab_size=V, max_position_embeddings=512),
    "olmo": _dec("OlmoConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, vocab_size=V,
                 max_position_embeddings=512),
    "olmo2": _dec("Olmo2Config", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                  vocab_size=V, max_position_embeddings=512),
    "starcoder2": _dec("Starcoder2Config", hidden_size=D, intermediate_size=4 * D, num_hidden_layers=L, num_attention_heads=H,
                       num_key_value_heads=4, vocab_size=V, max_position_embeddings=512, sliding_window=128),
    "granite": _dec("GraniteConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                    vocab_size=V, max_position_embeddings=512),
    "cohere": _dec("CohereConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                   vocab_size=V, max_position_embeddings=512),
    "mpt": _dec("MptConfig", d_model=D, n_layers=L, n_heads=H, vocab_size=V, max_seq_len=512),
    "codegen": _dec("CodeGenConfig", n_embd=D, n_layer=L, n_head=H, vocab_size=V, rotary_dim=16, n_positions=512),
    "bart": ("seq2seq", lambda T: T.BartConfig(d_model=D, encoder_layers=L, decoder_layers=L, encoder_attention_heads=H, decoder_attention_heads=H,
                                               encoder_ffn_dim=4 * D, decoder_ffn_dim=4 * D, vocab_size=V, max_position_embeddings=512)),
    "electra": ("masked-lm", lambda T: T.ElectraConfig(hidden_size=D, embedding_size=D, num_hidden_layers=L, num_attention_heads=H,
                                                       intermediate_size=4 * D, vocab_size=V, max_position_embeddings=512)),
    "albert": ("masked-lm", lambda T: T.AlbertConfig(hidden_size=D, embedding_size=128, num_hidden_layers=L, num_attention_heads=H,
                                                     intermediate_size=4 * D, vocab_size=V, max_position_embeddings=512)),
    "vit": ("image-cls", lambda T: T.ViTConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                               image_size=64, patch_size=8, num_labels=16)),
    "deit": ("image-cls", lambda T: T.DeiTConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                                 image_size=64, patch_size=8, num_labels=16)),
    "resnet": ("image-cls", lambda T: T.ResNetConfig(embedding_size=32, hidden_sizes=[32, 64], depths=[1, 1], layer_type="basic", num_labels=16)),
    "convnext": ("image-cls", lambda T: T.ConvNextConfig(num_stages=2, hidden_sizes=[32, 64], depths=[1, 1], num_labels=16)),
    "whisper": ("speech", lambda T: T.WhisperConfig(d_model=D, encoder_layers=L, decoder_layers=L, encoder_attention_heads=H,
                                                    decoder_attention_heads=H, encoder_ffn_dim=4 * D, decoder_ffn_dim=4 * D,
                                                    vocab_size=V, num_mel_bins=16, max_source_positions=64, max_target_positions=512,
                                                    pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)),
    "distilbert": ("masked-lm", lambda T: T.DistilBertConfig(dim=D, n_layers=L, n_heads=H, hidden_dim=4 * D, vocab_size=V,
                                                             max_position_embeddings=512)),
    # further families: decoders, encoders, seq2seq and vision models with less common building blocks (grouped linear layers,
    # relative-position attention, shifted windows, depthwise convolutions, spatial-reduction attention, pooling mixers)
    "openai_gpt": _dec("OpenAIGPTConfig", n_embd=D, n_layer=L, n_head=H, vocab_size=V, n_positions=512),
    "ctrl": _dec("CTRLConfig", n_embd=D, n_layer=L, n_head=H, dff=4 * D, vocab_size=V, n_positions=512),
    "glm": _dec("GlmConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                head_dim=32, vocab_size=V, max_position_embeddings=512, pad_token_id=0),
    "nemotron": _dec("NemotronConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H,
                     num_key_value_heads=4, head_dim=32, vocab_size=V, max_position_embeddings=512),
    "helium": _dec("HeliumConfig", hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=4,
                   head_dim=32, vocab_size=V, max_position_embeddings=512),
    "smollm3": _dec("SmolLM3Config", pad_token_id=0, hidden_size=D, intermediate_size=704, num_hidden_layers=L, num_attention_heads=H,
                    num_key_value_heads=4, vocab_size=V, max_position_embeddings=512),
    "biogpt": _dec("BioGptConfig", hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D, vocab_size=V,
                   max_position_embeddings=512),
    "xglm": _dec("XGLMConfig", d_model=D, num_layers=L, attention_heads=H, ffn_dim=4 * D, vocab_size=V, max_position_embeddings=512),
    "mt5": ("seq2seq", lambda T: T.MT5Config(d_model=D, d_ff=4 * D, num_layers=L, num_decoder_layers=L, num_heads=H, d_kv=D // H, vocab_size=V)),
    "mbart": ("seq2seq", lambda T: T.MBartConfig(d_model=D, encoder_layers=L, decoder_layers=L, encoder_attention_heads=H,
                                                 decoder_attention_heads=H, encoder_ffn_dim=4 * D, decoder_ffn_dim=4 * D, vocab_size=V,
                                                 max_position_embeddings=512)),
    "pegasus": ("seq2seq", lambda T: T.PegasusConfig(d_model=D, encoder_layers=L, decoder_layers=L, encoder_attention_heads=H,
                                                     decoder_attention_heads=H, encoder_ffn_dim=4 * D, decoder_ffn_dim=4 * D, vocab_size=V,
                                                     max_position_embeddings=512)),
    "marian": ("seq2seq", lambda T: T.MarianConfig(d_model=D, encoder_layers=L, decoder_layers=L, encoder_attention_heads=H,
                                                   decoder_attention_heads=H, encoder_ffn_dim=4 * D, decoder_ffn_dim=4 * D, vocab_size=V,
                                                   max_position_embeddings=512, pad_token_id=0, decoder_start_token_id=0)),
    "deberta_v2": ("masked-lm", lambda T: T.DebertaV2Config(hidden_size=D, num_hidden_layers=L, num_attention_heads=H,
                                                            intermediate_size=4 * D, vocab_size=V, max_position_embeddings=512)),
    "mobilebert": ("masked-lm", lambda T: T.MobileBertConfig(hidden_size=D, embedding_size=128, num_hidden_layers=L, num_attention_heads=4,
                                                             intermediate_size=4 * D, intra_bottleneck_size=128, vocab_size=V,
                                                             max_position_embeddings=512)),
    "squeezebert": ("masked-lm", lambda T: T.SqueezeBertConfig(hidden_size=D, embedding_size=D, num_hidden_layers=L, num_attention_heads=H,
                                                               intermediate_size=4 * D, vocab_size=V, max_position_embeddings=512,
                                                               q_groups=2, k_groups=2, v_groups=2, post_attention_groups=1,
                                                               intermediate_groups=2, output_groups=2)),
    "xlm_roberta": ("masked-lm", lambda T: T.XLMRobertaConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H,
                                                              intermediate_size=4 * D, vocab_size=V, max_position_embeddings=514)),
    "mpnet": ("masked-lm", lambda T: T.MPNetConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                                   vocab_size=V, max_position_embeddings=514)),
    "roformer": ("masked-lm", lambda T: T.RoFormerConfig(hidden_size=D, embedding_size=D, num_hidden_layers=L, num_attention_heads=H,
                                                         intermediate_size=4 * D, vocab_size=V, max_position_embeddings=512)),
    "beit": ("image-cls", lambda T: T.BeitConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                                 image_size=64, patch_size=8, num_labels=16)),
    "swin": ("image-cls", lambda T: T.SwinConfig(image_size=64, patch_size=4, embed_dim=32, depths=[1, 1], num_heads=[2, 4], window_size=4,
                                                 num_labels=16)),
    "mobilenet_v2": ("image-cls", lambda T: T.MobileNetV2Config(image_size=64, num_labels=16, depth_multiplier=0.35)),
    "regnet": ("image-cls", lambda T: T.RegNetConfig(embedding_size=32, hidden_sizes=[32, 64], depths=[1, 1], groups_width=8, num_labels=16)),
    "segformer": ("image-cls", lambda T: T.SegformerConfig(num_encoder_blocks=2, depths=[1, 1], sr_ratios=[2, 1], hidden_sizes=[32, 64],
                                                           patch_sizes=[7, 3], strides=[4, 2], num_attention_heads=[1, 2], num_labels=16)),
    "clip": ("contrastive", lambda T: T.CLIPConfig(
        text_config=T.CLIPTextConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D, vocab_size=V,
                                     max_position_embeddings=128, projection_dim=64).to_dict(),
        vision_config=T.CLIPVisionConfig(hidden_size=D, num_hidden_layers=L, num_attention_heads=H, intermediate_size=4 * D,
                                         image_size=64, patch_size=8, projection_dim=64).to_dict(),
        projection_dim=64)),
    "poolformer": ("image-cls", lambda T: T.PoolFormerConfig(num_encoder_blocks=2, depths=[1, 1], hidden_sizes=[32, 64], patch_sizes=[7, 3],
                                                             strides=[4, 2], padding=[2, 1], num_labels=16)),
}


# LayerDrop draws a random number per layer and branches on it in Python while training: not capturable as one
# graph.  These families are planned in eval mode (the branch is skipped; dropout is off).
EVAL_MODE = {"opt", "bart", "whisper", "biogpt", "xglm", "mbart", "pegasus", "marian"}


def plan_one(name, mesh, batch, seq, execute, bf16=False, uneven=False):
    import transformers as T

    task, make = ZOO[name]
    cfg = make(T)
    cfg.use_cache = False
    if name == "deit":
        cfg.architectures = ["DeiTForImageClassification"]  # the auto class maps this config to two heads
    auto = {"causal-lm": T.AutoModelForCausalLM, "seq2seq": T.AutoModelForSeq2SeqLM, "masked-lm": T.AutoModelForMaskedLM,
            "image-cls": T.AutoModelForImageClassification, "speech": T.AutoModelForSpeechSeq2Seq, "contrastive": T.AutoModel}[task]
    with torch.device("meta"):
        try:
            cfg._attn_implementation = "sdpa"
            model = auto.from_config(cfg)
        except ValueError:  # architectures without a fused-attention path: explicit softmax(QK^T)V
            cfg._attn_implementation = "eager"
            model = auto.from_config(cfg)
    if name in EVAL_MODE:
        model.eval()

    def ids():
        return torch.randint(0, cfg.vocab_size, (batch, seq))

    def input_fn():
        if task == "image-cls":
            return ForwardInputs((), {"pixel_values": torch.randn(batch, 3, 64, 64)})
        if task == "speech":  # log-mel frames in (two per encoder position), decoder tokens
            return ForwardInputs((), {"input_features": torch.randn(batch, 16, 128), "decoder_input_ids": ids()})
        if task == "contrastive":  # one caption per image
            return ForwardInputs((), {"input_ids": torch.randint(0, V, (batch, min(seq, 64))), "pixel_values": torch.randn(batch, 3, 64, 64)})
        kw = {"input_ids": ids()}
        if task == "seq2seq":
            kw["decoder_input_ids"] = ids()
        return ForwardInputs((), kw)

    n_in = 2 if task in ("seq2seq", "speech", "contrastive") else 1
    t0 = time.perf_counter()
    policy = None
    if bf16:
        from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy

        policy = MPPolicy(torch.bfloat16, torch.float32)
    with AutoParallel(model, input_fn, mesh, policy, uneven_sharding=uneven) as autop:
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
        logits = out.logits if hasattr(out, "logits") else (out.logits_per_image if hasattr(out, "logits_per_image") else out[0])
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
    ap.add_argument("--uneven", action="store_true", help="allow shards of unequal size (try --seq-len 100)")
    a = ap.parse_args()
    shape = tuple(int(x) for x in a.mesh.split(","))
    mesh = fake_mesh(shape, ("dp", "tp")[: len(shape)])
    names = a.only.split(",") if a.only else list(ZOO)
    failed = []
    for name in names:
        try:
            secs, cost, coll = plan_one(name, mesh, a.batch, a.seq_len, a.execute, a.bf16, a.uneven)
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
