"""Llama-3 family decoder written on the framework's operator library.

Architecture parity with the reference test model (autoparallel/_testing/models/llama3.py:
``TransformerModelArgs`` :75-135, ``Attention`` :228-317, ``FeedForward`` :320-361,
``TransformerBlock`` :364-429, ``Transformer`` :432-547): pre-norm blocks, GQA, interleaved
RoPE, SwiGLU FFN whose hidden size is rounded up to ``multiple_of``, untied output head,
depth-scaled init.  Differences that are deliberate:

* tensors stay ``[batch, seq, heads, head_dim]`` end to end – the attention kernel is
  GQA-native, so there is neither ``repeat_kv`` nor a transpose around it;
* RoPE uses real ``cos``/``sin`` tables (fp32 buffers) instead of a complex buffer;
* every non-GEMM hot op is an ``apb200`` operator (one planner rule + one sm_100a kernel each).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops as K


@dataclass
class LlamaConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = 8
    vocab_size: int = 128256
    ffn_hidden: Optional[int] = None  # explicit hidden size; else derived Llama-style
    multiple_of: int = 1024
    ffn_dim_multiplier: Optional[float] = 1.3
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 8192
    init_std: float = 0.02
    depth_init: bool = False

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def kv_heads(self) -> int:
        return self.n_kv_heads if self.n_kv_heads is not None else self.n_heads

    def hidden_dim(self) -> int:
        if self.ffn_hidden is not None:
            return self.ffn_hidden
        h = int(2 * (4 * self.dim) / 3)
        if self.ffn_dim_multiplier is not None:
            h = int(self.ffn_dim_multiplier * h)
        return self.multiple_of * ((h + self.multiple_of - 1) // self.multiple_of)

    def num_params(self) -> int:
        d, h, hd = self.dim, self.hidden_dim(), self.head_dim
        per_layer = d * (self.n_heads * hd) * 2 + d * (self.kv_heads * hd) * 2 + 3 * d * h + 2 * d
        return self.n_layers * per_layer + 2 * self.vocab_size * d + d

    def flops_per_token(self, seq_len: int) -> int:
        """Training FLOPs per token (6·N_nonembedding + causal-unaware attention term)."""
        d, h, hd = self.dim, self.hidden_dim(), self.head_dim
        dense = self.n_layers * (d * (self.n_heads * hd) * 2 + d * (self.kv_heads * hd) * 2 + 3 * d * h)
        dense += self.vocab_size * d
        return 6 * dense + 12 * self.n_layers * self.n_heads * hd * seq_len


def llama3_8b(**kw) -> LlamaConfig:
    base = dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_hidden=14336)
    base.update(kw)
    return LlamaConfig(**base)


def llama3_70b(**kw) -> LlamaConfig:
    base = dict(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_hidden=28672, max_seq_len=4096)
    base.update(kw)
    return LlamaConfig(**base)


def llama3_debug(**kw) -> LlamaConfig:
    base = dict(dim=256, n_layers=2, n_heads=8, n_kv_heads=4, ffn_hidden=512, vocab_size=1024, max_seq_len=256)
    base.update(kw)
    return LlamaConfig(**base)


def rope_tables(head_dim: int, max_seq_len: int, theta: float, device=None, yarn: Optional[dict] = None):
    """cos / sin tables ``[max_seq_len, head_dim / 2]``.  ``yarn``: context extension of a model trained at
    ``original_max_seq_len`` by ``factor``: rotary pairs that turn more than ``beta_fast`` times over the
    original context keep their frequency, pairs that turn fewer than ``beta_slow`` times are slowed down by
    ``factor`` (position interpolation), the ones in between blend linearly; both tables are scaled by the
    attention temperature ``0.1 * mscale * ln(factor) + 1`` (the reference's DeepSeek-V3 model precomputes its
    rotary frequencies this way, autoparallel/_testing/models/dsv3.py:62-135)."""
    half = torch.arange(0, head_dim, 2, device=device, dtype=torch.float32)
    inv = 1.0 / (theta ** (half / head_dim))
    scale = 1.0
    if yarn is not None and yarn.get("factor", 1.0) > 1.0:
        factor = float(yarn["factor"])
        orig = int(yarn.get("original_max_seq_len", max_seq_len))
        beta_fast, beta_slow = float(yarn.get("beta_fast", 32.0)), float(yarn.get("beta_slow", 1.0))

        def pair_with_rotations(r):  # index of the rotary pair that completes ``r`` turns over the original context
            return head_dim * math.log(orig / (r * 2 * math.pi)) / (2 * math.log(theta))

        lo = max(math.floor(pair_with_rotations(beta_fast)), 0)
        hi = min(math.ceil(pair_with_rotations(beta_slow)), head_dim // 2 - 1)
        ramp = ((torch.arange(head_dim // 2, device=device, dtype=torch.float32) - lo) / max(hi - lo, 1e-3)).clamp(0.0, 1.0)
        inv = inv * (1.0 - ramp) + (inv / factor) * ramp
        scale = 0.1 * float(yarn.get("mscale", 1.0)) * math.log(factor) + 1.0
    ang = torch.outer(torch.arange(max_seq_len, device=device, dtype=torch.float32), inv)
    return ang.cos() * scale, ang.sin() * scale


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return K.rms_norm(x, self.weight, self.eps)

    def init_weights(self):
        nn.init.ones_(self.weight)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.n_heads, self.n_kv, self.hd = cfg.n_heads, cfg.kv_heads, cfg.head_dim
        self.wq = nn.Linear(cfg.dim, self.n_heads * self.hd, bias=False)
        self.wk = nn.Linear(cfg.dim, self.n_kv * self.hd, bias=False)
        self.wv = nn.Linear(cfg.dim, self.n_kv * self.hd, bias=False)
        self.wo = nn.Linear(self.n_heads * self.hd, cfg.dim, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        q = self.wq(x).view(b, s, self.n_heads, self.hd)
        k = self.wk(x).view(b, s, self.n_kv, self.hd)
        v = self.wv(x).view(b, s, self.n_kv, self.hd)
        q = K.rope(q, cos, sin)
        k = K.rope(k, cos, sin)
        o = K.attention(q, k, v, causal=True)
        return self.wo(o.view(b, s, self.n_heads * self.hd))

    def init_weights(self, std: float, out_std: float):
        for lin in (self.wq, self.wk, self.wv):
            nn.init.normal_(lin.weight, mean=0.0, std=std)
        nn.init.normal_(self.wo.weight, mean=0.0, std=out_std)


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)

    def forward(self, x):
        return self.w2(K.swiglu(self.w1(x), self.w3(x)))

    def init_weights(self, std: float, out_std: float):
        nn.init.normal_(self.w1.weight, mean=0.0, std=std)
        nn.init.normal_(self.w3.weight, mean=0.0, std=std)
        nn.init.normal_(self.w2.weight, mean=0.0, std=out_std)


class TransformerBlock(nn.Module):
    def __init__(self, layer_id: int, cfg: LlamaConfig):
        super().__init__()
        self.attention = Attention(cfg)
        self.feed_forward = FeedForward(cfg.dim, cfg.hidden_dim())
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        depth = (layer_id + 1) if cfg.depth_init else cfg.n_layers
        self.std = cfg.init_std
        self.out_std = cfg.init_std / (2 * depth) ** 0.5 if cfg.depth_init else cfg.init_std

    def forward(self, x, cos, sin):
        h = x + self.attention(self.attention_norm(x), cos, sin)
        return h + self.feed_forward(self.ffn_norm(h))

    def init_weights(self):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.std, self.out_std)
        self.feed_forward.init_weights(self.std, self.out_std)


class Transformer(nn.Module):
    """Decoder-only LM.  ``forward(tokens)`` returns logits ``[B, S, vocab]``;
    ``forward(tokens, labels)`` returns the mean next-token cross-entropy (scalar)."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleDict({str(i): TransformerBlock(i, cfg) for i in range(cfg.n_layers)})
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.output = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        cos, sin = rope_tables(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def forward(self, tokens, labels=None):
        s = tokens.shape[1]
        cos, sin = self.rope_cos[:s], self.rope_sin[:s]
        h = self.tok_embeddings(tokens)
        for layer in self.layers.values():
            h = layer(h, cos, sin)
        logits = self.output(self.norm(h))
        if labels is None:
            return logits
        return K.cross_entropy(logits, labels)

    def init_weights(self, seed: Optional[int] = None):
        if seed is not None:
            torch.manual_seed(seed)
        cfg = self.cfg
        dev = self.rope_cos.device
        cos, sin = rope_tables(cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, device=dev)
        self.rope_cos = cos
        self.rope_sin = sin
        nn.init.normal_(self.tok_embeddings.weight, mean=0.0, std=cfg.init_std)
        for layer in self.layers.values():
            layer.init_weights()
        self.norm.init_weights()
        nn.init.normal_(self.output.weight, mean=0.0, std=cfg.init_std)
