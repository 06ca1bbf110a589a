"""Numerics of the Hugging Face zoo on real ranks (gloo, CPU): every family of ``run_hf_zoo.py`` is planned on the
given mesh, loaded with the weights of a single-device copy, and one forward / backward is compared with that copy
(largest absolute output error, largest gradient error relative to the gradient's size).  Models run in eval mode
so that dropout does not draw different masks.

    python examples/run_hf_numerics.py 2          # 1-D mesh of two ranks, all families
    python examples/run_hf_numerics.py 2,2 llama,t5,vit

(Reference counterpart: examples/run_hf_eval.sh, which checks that the models plan; numerics are checked here.)"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch.distributed.tensor.placement_types import Replicate, Shard

def worker(rank, ws, names, port, mesh_shape):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    import transformers as T
    from torch.distributed.device_mesh import init_device_mesh
    from autoparallel_b200 import AutoParallel, ForwardInputs
    from autoparallel_b200.parallel.lower.init_weights import _distribute
    from examples.run_hf_zoo import ZOO
    mesh = init_device_mesh("cpu", mesh_shape, mesh_dim_names=("dp", "tp")[:len(mesh_shape)])
    dp = mesh_shape[0]; me = mesh.get_coordinate()[0]
    for name in names:
        try:
            task, make = ZOO[name]
            cfg = make(T); cfg.use_cache = False
            if name == "deit": cfg.architectures = ["DeiTForImageClassification"]
            auto = {"causal-lm": T.AutoModelForCausalLM, "seq2seq": T.AutoModelForSeq2SeqLM, "masked-lm": T.AutoModelForMaskedLM,
                    "image-cls": T.AutoModelForImageClassification, "speech": T.AutoModelForSpeechSeq2Seq, "contrastive": T.AutoModel}[task]
            try:
                cfg._attn_implementation = "sdpa"; torch.manual_seed(0); ref = auto.from_config(cfg)
            except ValueError:
                cfg._attn_implementation = "eager"; torch.manual_seed(0); ref = auto.from_config(cfg)
            ref.eval()
            with torch.device("meta"):
                model = auto.from_config(cfg)
            model.eval()
            B, S = 4, 32
            torch.manual_seed(1)
            if task == "image-cls":
                full = {"pixel_values": torch.randn(B, 3, 64, 64)}
            elif task == "speech":
                full = {"input_features": torch.randn(B, 16, 128), "decoder_input_ids": torch.randint(0, cfg.vocab_size, (B, S))}
            elif task == "contrastive":
                full = {"input_ids": torch.randint(0, cfg.text_config.vocab_size, (B, S)), "pixel_values": torch.randn(B, 3, 64, 64)}
            else:
                full = {"input_ids": torch.randint(0, cfg.vocab_size, (B, S))}
                if task == "seq2seq": full["decoder_input_ids"] = torch.randint(0, cfg.vocab_size, (B, S))
            rest = (Replicate(),) * (len(mesh_shape) - 1)
            with AutoParallel(model, lambda: ForwardInputs((), {k: (torch.randn(v.shape) if v.is_floating_point() else torch.randint(0, 16, v.shape)) for k, v in full.items()}), mesh) as ap:
                ap.add_parameter_memory_constraint()
                ap.add_input_constraints([(Shard(0),) + rest] * len(full))
                ap.add_output_constraints([(Shard(0),) + rest] + [None] * (ap.joint.num_user_outputs - 1))
                ap.optimize_placement(); pm = ap.apply_placement()
            pm.to_empty(device="cpu")
            state = dict(ref.named_parameters()); state.update(dict(ref.named_buffers()))
            with torch.no_grad():
                for n, t in list(pm.named_parameters()) + list(pm.named_buffers()):
                    t._local_tensor.copy_(_distribute(state[n].detach().clone(), mesh, t.placements)._local_tensor)
            out = pm(**{k: v.chunk(dp, 0)[me] for k, v in full.items()})
            logits = out.logits if hasattr(out, "logits") else out.logits_per_image
            w = torch.linspace(-1, 1, logits.shape[-1])
            (logits.float() * w).mean().backward()
            ro = ref(**full)
            rl = ro.logits if hasattr(ro, "logits") else ro.logits_per_image
            (rl.float() * w).mean().backward()
            err = (logits - rl.chunk(dp, 0)[me]).abs().max().item()
            worst, who = 0.0, ""
            for n, p in pm.named_parameters():
                if p.grad is None: continue
                g = p.grad.full_tensor() * (1.0 / dp); rg = state[n].grad
                if rg is None:  # a parameter the single-device model's loss does not reach: its gradient here must be zero
                    rg = torch.zeros_like(g)
                e = ((g - rg).abs().max() / (rg.abs().max() + 1e-6)).item()
                if e > worst: worst, who = e, n
            if rank == 0: print(f"{name:12s} out {err:.2e} grad {worst:.2e} ({who})", flush=True)
        except Exception as e:
            if rank == 0: print(f"{name:12s} EXC {type(e).__name__}: {str(e)[:200]}", flush=True)
    dist.destroy_process_group()

if __name__ == "__main__":
    shape = tuple(int(x) for x in sys.argv[1].split(","))
    from examples.run_hf_zoo import ZOO as _ZOO

    names = sys.argv[2].split(",") if len(sys.argv) > 2 else list(_ZOO)
    ws = 1
    for s in shape: ws *= s
    mp.spawn(worker, args=(ws, names, 29500 + os.getpid() % 400, shape), nprocs=ws, join=True)
