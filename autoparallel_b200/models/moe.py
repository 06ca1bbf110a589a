"""Mixture-of-experts decoder with expert parallelism through ``local_map`` or through
planner-visible MoE operators (``MoEConfig.expert_mode``).

Config of record: 12 layers, d_model 2048, 16 query / 4 KV heads, RoPE, RMSNorm, vocab 102400;
every FFN is MoE with 64 routed SwiGLU experts (hidden 1408), softmax top-8 router, plus one
always-on shared expert.  The dense parts (attention, shared expert, norms, embeddings) are sharded
by the planner; the routed-expert block is one ``local_map`` region – route → dispatch all-to-all →
expert FFN on the local experts → combine all-to-all → weighted scatter-add – with tokens
``Shard(0)`` and expert weights ``Shard(0)`` on the expert-parallel mesh axis.

Dispatch is **capacity based**: each (source rank, expert) pair owns a fixed slot count
``C = ceil(capacity_factor · tokens · top_k / num_experts)``; assignments beyond the slot count are
dropped (their gate weight contributes nothing).  ``capacity_factor=None`` is the **dropless** setting: every
(source rank, expert) pair gets as many slots as the rank has tokens - the most it can ever need, since a token
names an expert at most once - so no assignment is ever dropped and the numerics equal the single-device model
under any routing skew, at the price of moving and multiplying the padding (exact, not fast: a transport and a
grouped GEMM that skip the padding through device-side counts are not built).  ``MoEFFN.dropped_assignments``
counts what a given batch would lose under the configured capacity.  Shapes are therefore static – no device→host
sync for split sizes in any layer and the step is CUDA-graph capturable – where the reference
exchanges counts and then syncs to the host for variable all-to-all splits
(autoparallel/_testing/models/dsv3.py:552-616; routing :388-444; region :620-703).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.distributed.tensor.placement_types import Shard

from .. import ops as K
from ..collectives import all_to_all, axis_size, local_map
from .llama3 import Attention, LlamaConfig, RMSNorm, rope_tables


@dataclass
class MoEConfig:
    dim: int = 2048
    n_layers: int = 12
    n_heads: int = 16
    n_kv_heads: int = 4
    vocab_size: int = 102400
    num_experts: int = 64
    top_k: int = 8
    expert_hidden: int = 1408
    shared_hidden: int = 1408
    capacity_factor: Optional[float] = 1.25  # None: dropless (capacity = tokens per rank)
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 4096
    init_std: float = 0.02
    ep_axis: str = "ep"
    router_bias_zipf: Optional[float] = None  # s of a Zipf(s) bias over experts (skewed-load runs)
    #: "local_map": the routed block is one opaque region with hand-written all-to-alls on ``ep_axis``;
    #: "planner": the block is built from the apb200 MoE operators (ops/moe_ops.py) and the solver
    #: chooses where the token buffer moves to the experts (no mesh axis is named in the model)
    #: "gqa": grouped-query attention as in the Llama model; "mla": multi-head latent attention (low-rank
    #: compressed keys / values with a rotary part shared by all heads, optional low-rank queries)
    attention: str = "gqa"
    q_lora_rank: int = 0
    kv_lora_rank: int = 64
    qk_nope_head_dim: int = 32
    qk_rope_head_dim: int = 16
    v_head_dim: int = 32
    #: YaRN context extension of the rotary tables, e.g. {"factor": 4.0, "original_max_seq_len": 1024}
    rope_yarn: Optional[dict] = None
    expert_mode: str = "local_map"
    dispatch_blocks: int = 8  # planner mode: token blocks with their own per-expert capacity (a multiple of the shard count)

    def rope_dim(self) -> int:
        """Width of the rotated part of a query / key head."""
        return self.qk_rope_head_dim if self.attention == "mla" else self.dim // self.n_heads

    def attn_cfg(self) -> LlamaConfig:
        return LlamaConfig(dim=self.dim, n_layers=self.n_layers, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                           vocab_size=self.vocab_size, norm_eps=self.norm_eps, rope_theta=self.rope_theta,
                           max_seq_len=self.max_seq_len, init_std=self.init_std)


def moe_reference_config(**kw) -> MoEConfig:
    return MoEConfig(**kw)


def moe_debug(**kw) -> MoEConfig:
    base = dict(dim=128, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=512, num_experts=8, top_k=2, expert_hidden=64,
                shared_hidden=64, max_seq_len=64)
    base.update(kw)
    return MoEConfig(**base)


def _expert_region(x, gate_w, gate_idx, w1, w3, w2, *, ep_axis: str, num_experts: int, capacity: int):
    """Runs on local shards.  x [T, d] tokens of this rank; gate_w / gate_idx [T, k]; w1, w3
    [E_loc, d, h], w2 [E_loc, h, d] local experts.  Returns [T, d]."""
    T, d = x.shape
    n = axis_size(ep_axis)
    e_loc = num_experts // n
    # slot of every (token, choice) in this rank's [E * C] send buffer (E * C = beyond the capacity: dropped), the rows
    # written expert-major, and after the expert FFN read back weighted by the gate: three operators with kernels and
    # gradients of their own (ops/moe_ops.py) instead of a sort, a dozen index operators and a [T * k, d] intermediate
    slot = K.moe_slots(gate_idx, num_experts, capacity, 1)
    send = K.moe_dispatch(x, slot, num_experts, capacity, 1)        # [E, 1, C, d]
    recv = all_to_all(send.reshape(n * e_loc * capacity, d), ep_axis, 0, 0).view(n, e_loc, capacity, d)
    h = recv.permute(1, 0, 2, 3).reshape(e_loc, n * capacity, d)    # expert-major
    y = K.grouped_mm(K.swiglu(K.grouped_mm(h, w1), K.grouped_mm(h, w3)), w2)   # [E_loc, n*C, d]: one grouped GEMM launch each
    back = y.view(e_loc, n, capacity, d).permute(1, 0, 2, 3).reshape(n * e_loc * capacity, d)
    got = all_to_all(back, ep_axis, 0, 0)                           # [E*C, d] in this rank's slot order
    return K.moe_combine(got.view(num_experts, 1, capacity, d), slot, gate_w)


class MLAttention(nn.Module):
    """Multi-head latent attention (the attention of the reference's DeepSeek-V3 test model,
    autoparallel/_testing/models/dsv3.py:1382-1530): keys and values are projected down to ``kv_lora_rank``
    (+ one rotary key of ``qk_rope_head_dim`` shared by all heads), normalised, and projected up per head;
    queries optionally take the same detour.  Query / key heads are ``qk_nope + qk_rope`` wide, value heads
    ``v_head_dim``; values are zero-padded to the query width for the attention operator and the padding is
    dropped from its output."""

    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.h = cfg.n_heads
        self.nope, self.rope, self.vd = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk = self.nope + self.rope
        self.kv_rank, self.q_rank = cfg.kv_lora_rank, cfg.q_lora_rank
        if self.q_rank == 0:
            self.wq = nn.Linear(cfg.dim, self.h * self.qk, bias=False)
        else:
            self.wq_a = nn.Linear(cfg.dim, self.q_rank, bias=False)
            self.q_norm = RMSNorm(self.q_rank, cfg.norm_eps)
            self.wq_b = nn.Linear(self.q_rank, self.h * self.qk, bias=False)
        self.wkv_a = nn.Linear(cfg.dim, self.kv_rank + self.rope, bias=False)
        self.kv_norm = RMSNorm(self.kv_rank, cfg.norm_eps)
        self.wkv_b = nn.Linear(self.kv_rank, self.h * (self.nope + self.vd), bias=False)
        self.wo = nn.Linear(self.h * self.vd, cfg.dim, bias=False)

    def forward(self, x, cos, sin):
        b, s, _ = x.shape
        q = self.wq(x) if self.q_rank == 0 else self.wq_b(self.q_norm(self.wq_a(x)))
        q = q.view(b, s, self.h, self.qk)
        q_nope, q_pe = q[..., : self.nope], q[..., self.nope:]
        kv = self.wkv_a(x)
        kv_c, k_pe = kv[..., : self.kv_rank], kv[..., self.kv_rank:]
        k_pe = K.rope(k_pe.reshape(b, s, 1, self.rope), cos, sin)            # one rotary key for all heads
        q_pe = K.rope(q_pe.contiguous(), cos, sin)
        kvu = self.wkv_b(self.kv_norm(kv_c)).view(b, s, self.h, self.nope + self.vd)
        k_nope, v = kvu[..., : self.nope], kvu[..., self.nope:]
        q = torch.cat([q_nope, q_pe], dim=-1)
        k = torch.cat([k_nope, k_pe.expand(b, s, self.h, self.rope)], dim=-1)
        v = F.pad(v, (0, self.qk - self.vd)) if self.qk > self.vd else v
        o = K.attention(q, k, v, causal=True, scale=self.qk ** -0.5)[..., : self.vd]
        return self.wo(o.reshape(b, s, self.h * self.vd))

    def init_weights(self, std: float, out_std: float):
        for name in ("wq", "wq_a", "wq_b", "wkv_a", "wkv_b"):
            lin = getattr(self, name, None)
            if lin is not None:
                nn.init.normal_(lin.weight, mean=0.0, std=std)
        nn.init.normal_(self.wo.weight, mean=0.0, std=out_std)
        self.kv_norm.init_weights()
        if self.q_rank:
            self.q_norm.init_weights()


class MoEFFN(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.cfg = cfg
        E, d, h = cfg.num_experts, cfg.dim, cfg.expert_hidden
        self.router = nn.Linear(d, E, bias=False)
        self.register_buffer("router_bias", torch.zeros(E), persistent=True)
        self.w1 = nn.Parameter(torch.empty(E, d, h))
        self.w3 = nn.Parameter(torch.empty(E, d, h))
        self.w2 = nn.Parameter(torch.empty(E, h, d))
        self.shared_w1 = nn.Linear(d, cfg.shared_hidden, bias=False)
        self.shared_w3 = nn.Linear(d, cfg.shared_hidden, bias=False)
        self.shared_w2 = nn.Linear(cfg.shared_hidden, d, bias=False)

    def forward(self, x):
        cfg = self.cfg
        b, s, d = x.shape
        scores = torch.softmax((self.router(x).float() + self.router_bias), dim=-1)
        gate_w, gate_idx = torch.topk(scores, cfg.top_k, dim=-1)
        gate_w = gate_w / gate_w.sum(-1, keepdim=True)
        shared = self.shared_w2(K.swiglu(self.shared_w1(x), self.shared_w3(x)))
        if cfg.expert_mode == "planner":
            return shared + self._routed_planner(x.reshape(b * s, d), gate_w.to(x.dtype).reshape(b * s, -1),
                                                 gate_idx.reshape(b * s, -1)).view(b, s, d)
        tokens_per_rank = (b * s) // axis_size(cfg.ep_axis)
        capacity = self.capacity(tokens_per_rank)

        # Argument order = order of first use inside the region: the graph capture lists the region's
        # inputs in that order and insists that the declared placements line up with it.
        def region(gi, xf, w1, w3, w2, gw):
            return _expert_region(xf, gw, gi, w1, w3, w2, ep_axis=cfg.ep_axis, num_experts=cfg.num_experts, capacity=capacity)

        tok_pl = (Shard(0),)
        routed = local_map(region, out_placements=(tok_pl,), in_placements=(tok_pl,) * 6)(
            gate_idx.reshape(b * s, -1), x.reshape(b * s, d), self.w1, self.w3, self.w2, gate_w.to(x.dtype).reshape(b * s, -1))
        return shared + routed.view(b, s, d)

    def capacity(self, tokens: int) -> int:
        """Slots of one (token block, expert) pair; ``tokens`` = tokens of the block (a rank, or a dispatch block)."""
        cfg = self.cfg
        if cfg.capacity_factor is None:
            return max(1, tokens)  # dropless: a block never sends more than one assignment per token to an expert
        return max(1, math.ceil(cfg.capacity_factor * tokens * cfg.top_k / cfg.num_experts))

    @torch.no_grad()
    def dropped_assignments(self, x: torch.Tensor, blocks: int) -> int:
        """How many of the ``tokens x top_k`` assignments of ``x`` [b, s, d] the configured capacity drops when the
        tokens are split into ``blocks`` equal blocks (ranks of the expert-parallel axis, or dispatch blocks)."""
        cfg = self.cfg
        scores = torch.softmax(self.router(x).float() + self.router_bias, dim=-1)
        idx = torch.topk(scores, cfg.top_k, dim=-1).indices.reshape(blocks, -1)          # [blocks, tokens/block * k]
        cap = self.capacity(idx.shape[1] // cfg.top_k)
        counts = torch.zeros(blocks, cfg.num_experts, dtype=torch.long, device=x.device).scatter_add_(1, idx, torch.ones_like(idx))
        return int((counts - cap).clamp_min(0).sum().item())

    def _routed_planner(self, xf, gate_w, gate_idx):
        """Routed experts as graph nodes the solver places: slots -> scatter -> 3 grouped GEMMs -> gather."""
        cfg = self.cfg
        T, d = xf.shape
        E, nb = cfg.num_experts, cfg.dispatch_blocks
        capacity = self.capacity(T // nb)
        slot = K.moe_slots(gate_idx, E, capacity, nb)
        h = K.moe_dispatch(xf, slot, E, capacity, nb).view(E, nb * capacity, d)
        y = K.grouped_mm(K.swiglu(K.grouped_mm(h, self.w1), K.grouped_mm(h, self.w3)), self.w2)
        return K.moe_combine(y.view(E, nb, capacity, d), slot, gate_w)

    def init_weights(self, std: float):
        nn.init.normal_(self.router.weight, mean=0.0, std=std)
        for w in (self.w1, self.w3, self.w2):
            nn.init.normal_(w, mean=0.0, std=std)
        for lin in (self.shared_w1, self.shared_w3, self.shared_w2):
            nn.init.normal_(lin.weight, mean=0.0, std=std)
        if self.cfg.router_bias_zipf:
            ranks = torch.arange(1, self.cfg.num_experts + 1, dtype=torch.float32, device=self.router_bias.device)
            p = ranks.pow(-self.cfg.router_bias_zipf)
            self.router_bias = (p / p.sum()).log() - (p / p.sum()).log().mean()
        else:
            self.router_bias = torch.zeros_like(self.router_bias)


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.attention = MLAttention(cfg) if cfg.attention == "mla" else Attention(cfg.attn_cfg())
        self.moe = MoEFFN(cfg)
        self.attention_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.std = cfg.init_std

    def forward(self, x, cos, sin):
        h = x + self.attention(self.attention_norm(x), cos, sin)
        return h + self.moe(self.ffn_norm(h))

    def init_weights(self):
        self.attention_norm.init_weights()
        self.ffn_norm.init_weights()
        self.attention.init_weights(self.std, self.std)
        self.moe.init_weights(self.std)


class MoETransformer(nn.Module):
    def __init__(self, cfg: MoEConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.dim)
        self.layers = nn.ModuleDict({str(i): MoEBlock(cfg) for i in range(cfg.n_layers)})
        self.norm = RMSNorm(cfg.dim, cfg.norm_eps)
        self.output = nn.Linear(cfg.dim, cfg.vocab_size, bias=False)
        cos, sin = rope_tables(cfg.rope_dim(), cfg.max_seq_len, cfg.rope_theta, yarn=cfg.rope_yarn)
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
        cos, sin = rope_tables(cfg.rope_dim(), cfg.max_seq_len, cfg.rope_theta, device=self.rope_cos.device, yarn=cfg.rope_yarn)
        self.rope_cos, self.rope_sin = cos, sin
        nn.init.normal_(self.tok_embeddings.weight, mean=0.0, std=cfg.init_std)
        for layer in self.layers.values():
            layer.init_weights()
        self.norm.init_weights()
        nn.init.normal_(self.output.weight, mean=0.0, std=cfg.init_std)
