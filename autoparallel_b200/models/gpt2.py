"""GPT-2 decoder (learned positions, LayerNorm, GELU FFN, tied embedding / LM head).

This is the CPU planning/benchmark model: 12 layers, d_model 768, 12 heads, FFN 3072,
vocab 50257, fp32, N(0, 0.02) weights.  It is written with plain ATen ops so that it
exercises the planner's generic path (DTensor rules, ``addmm`` decomposition, un-decomposed
``native_layer_norm``, aliased parameters) the way the reference's Hugging Face example does
(examples/example_hf.py:114-126).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int = 3072
    layer_norm_eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = True


def gpt2_small(**kw) -> GPT2Config:
    return GPT2Config(**kw)


def gpt2_debug(**kw) -> GPT2Config:
    base = dict(vocab_size=512, n_positions=64, n_embd=64, n_layer=2, n_head=4, n_inner=128)
    base.update(kw)
    return GPT2Config(**base)


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head = cfg.n_head
        self.ln_1 = nn.LayerNorm(cfg.n_embd, eps=cfg.layer_norm_eps)
        self.c_attn = nn.Linear(cfg.n_embd, 3 * cfg.n_embd)
        self.c_proj = nn.Linear(cfg.n_embd, cfg.n_embd)
        self.ln_2 = nn.LayerNorm(cfg.n_embd, eps=cfg.layer_norm_eps)
        self.c_fc = nn.Linear(cfg.n_embd, cfg.n_inner)
        self.c_out = nn.Linear(cfg.n_inner, cfg.n_embd)

    def forward(self, x):
        b, s, d = x.shape
        qkv = self.c_attn(self.ln_1(x))
        q, k, v = qkv.split(d, dim=2)
        hd = d // self.n_head
        q = q.view(b, s, self.n_head, hd).transpose(1, 2)
        k = k.view(b, s, self.n_head, hd).transpose(1, 2)
        v = v.view(b, s, self.n_head, hd).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.c_proj(a.transpose(1, 2).reshape(b, s, d))
        return x + self.c_out(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = nn.Embedding(cfg.n_positions, cfg.n_embd)
        self.h = nn.ModuleList([GPT2Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.n_embd, eps=cfg.layer_norm_eps)
        self.lm_head = nn.Linear(cfg.n_embd, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.wte.weight

    def forward(self, tokens, labels=None):
        s = tokens.shape[1]
        pos = torch.arange(s, device=tokens.device)
        x = self.wte(tokens) + self.wpe(pos)
        for blk in self.h:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        if labels is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))

    def init_weights(self, seed=None):
        if seed is not None:
            torch.manual_seed(seed)
        std = self.cfg.init_std
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=std)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, mean=0.0, std=std)
            elif isinstance(m, nn.LayerNorm):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
