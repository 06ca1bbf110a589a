"""Device-neutral stand-ins for operators that only the planning host has.

Planning traces the model on CPU fake tensors, so an attention call that the pattern pass does not take over (an explicit
attention mask, ``pattern_ops=False``) is decomposed to ``aten._scaled_dot_product_flash_attention_for_cpu`` and its backward
- operators without a CUDA implementation.  When a runtime's graphs move to another device the executor swaps them for the
functions below.  Off the CPU the forward is ``torch.nn.functional.scaled_dot_product_attention`` itself (whatever fused
kernel the device's library picks, mask included) and the backward recomputes that call under autograd, so nothing of
size L x S is kept; if the library refuses the arguments, the same mathematics runs in ordinary tensor operators with
the score matrix materialised.  (The framework's own attention operator serves the mask-free cases through the pattern
pass.)  Signatures and return values are those of the two ATen operators, so the swap is a change of ``node.target``
only; the log-sum-exp output is exact on the formula path and a placeholder on the library path, whose backward does
not read it.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

aten = torch.ops.aten
#: tests set this to run the device-neutral paths on CPU tensors as well
FORCE_GENERIC = False
#: skip the library call and use the explicit formulas (tests; a device whose library lacks the fused operator)
FORMULAS_ONLY = False


def _acc(t) -> torch.dtype:
    """Accumulation dtype: fp32 for 16-bit operands, the operand's own otherwise."""
    return torch.float32 if t.dtype in (torch.bfloat16, torch.float16) else t.dtype


def _scores(q, k, attn_mask, is_causal, scale):
    a = _acc(q)
    s = (q.to(a) @ k.to(a).transpose(-1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(q.shape[-1]))
    if is_causal:
        L, S = q.shape[-2], k.shape[-2]
        keep = torch.ones(L, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~keep, float("-inf"))
    if attn_mask is not None:
        s = s.masked_fill(~attn_mask, float("-inf")) if attn_mask.dtype == torch.bool else s + attn_mask.to(a)
    return s


def sdpa_forward(q, k, v, dropout_p: float = 0.0, is_causal: bool = False, *, attn_mask: Optional[torch.Tensor] = None,
                 scale: Optional[float] = None):
    """(output [B, H, L, Dv], logsumexp [B, H, L]) of softmax(q k^T * scale + mask) v."""
    if q.device.type == "cpu" and not FORCE_GENERIC:
        return aten._scaled_dot_product_flash_attention_for_cpu(q, k, v, dropout_p, is_causal, attn_mask=attn_mask, scale=scale)
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout inside the traced attention operator is not supported off the planning device")
    if not FORMULAS_ONLY:
        try:
            out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, is_causal=is_causal, scale=scale)
            return out, q.new_zeros(q.shape[:-1], dtype=torch.float32)
        except RuntimeError:
            pass
    s = _scores(q, k, attn_mask, is_causal, scale)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)  # rows that are masked out entirely
    return (p @ v.to(p.dtype)).to(q.dtype), lse


def sdpa_backward(grad_out, q, k, v, out, lse, dropout_p: float, is_causal: bool, *, attn_mask: Optional[torch.Tensor] = None,
                  scale: Optional[float] = None):
    """(dq, dk, dv) from the saved output and log-sum-exp."""
    if q.device.type == "cpu" and not FORCE_GENERIC:
        return aten._scaled_dot_product_flash_attention_for_cpu_backward(grad_out, q, k, v, out, lse, dropout_p, is_causal,
                                                                       attn_mask=attn_mask, scale=scale)
    if not FORMULAS_ONLY:
        try:
            with torch.enable_grad():
                qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
                o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, attn_mask=attn_mask, is_causal=is_causal, scale=scale)
                return torch.autograd.grad(o, (qq, kk, vv), grad_out)
        except RuntimeError:
            pass
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = _scores(q, k, attn_mask, is_causal, scale)
    p = torch.nan_to_num(torch.exp(s - lse.unsqueeze(-1)), nan=0.0)
    a = p.dtype
    do = grad_out.to(a)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.to(a).transpose(-1, -2)
    delta = (do * out.to(a)).sum(-1, keepdim=True)
    ds = p * (dp - delta) * sc
    dq = ds @ k.to(a)
    dk = ds.transpose(-1, -2) @ q.to(a)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


#: operators of the planning host -> stand-ins that run anywhere
SWAPS = {
    aten._scaled_dot_product_flash_attention_for_cpu.default: sdpa_forward,
    aten._scaled_dot_product_flash_attention_for_cpu_backward.default: sdpa_backward,
}
