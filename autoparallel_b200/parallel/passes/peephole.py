"""Local rewrites on the lowered graph that remove memory round trips.

* ``dtype_cast(gemm_like(a, b, .., bf16), fp32)`` with a single consumer becomes the GEMM with an
  fp32 epilogue: the weight-gradient GEMM writes the fp32 gradient the reduce-scatter wants
  directly (one full read+write of every gradient less, and no bf16 rounding before the
  reduction).
"""
from __future__ import annotations

import torch
import torch.fx as fx

apb = torch.ops.apb200

_GEMM_OUT_DTYPE_POS = {apb.mm_wgrad.default: 2, apb.mm_nd.default: 3, apb.gemm.default: 4}


def fuse_cast_into_gemm(gm: fx.GraphModule) -> int:
    n_fused = 0
    for n in list(gm.graph.nodes):
        if n.op != "call_function" or n.target is not apb.dtype_cast.default:
            continue
        src = n.args[0]
        if not (isinstance(src, fx.Node) and src.op == "call_function" and src.target in _GEMM_OUT_DTYPE_POS):
            continue
        if len(src.users) != 1 or n.args[1] not in (torch.float32, torch.bfloat16):
            continue
        pos = _GEMM_OUT_DTYPE_POS[src.target]
        args = list(src.args)
        args[pos] = n.args[1]
        src.args = tuple(args)
        src.meta["val"] = n.meta["val"]
        n.replace_all_uses_with(src)
        gm.graph.erase_node(n)
        n_fused += 1
    if n_fused:
        gm.graph.lint()
        gm.recompile()
    return n_fused
