"""Pattern pass: puts plain-PyTorch models on this framework's operators.

Models written against ``autoparallel_b200.ops`` already trace into kernel-sized nodes.  A model
written in stock PyTorch - the reference's own Llama, the Hugging Face zoo, user code - would
otherwise run node by node on decomposed ATen kernels (and its fused attention would be traced as
the CPU variant of the planning device, which cannot run on a GPU at all).  This pass rewrites the
graph Dynamo captures, *before* AOTAutograd differentiates it, so the backward falls out of the
operators' own autograd formulas:

* ``torch.rms_norm`` / ``F.rms_norm`` over the last dim, and the hand-written idiom
  ``w * (x.float() * rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)).to(dtype)``  ->  ``apb200::rms_norm``
* ``F.silu(a) * b`` (either operand order)                                 ->  ``apb200::swiglu``
* ``F.scaled_dot_product_attention(q, k, v, is_causal=...)`` without mask or dropout, heads-first
  layout; transposes from the ``[B, S, H, D]`` layout and ``repeat_kv`` expansions of grouped-query
  keys / values are looked through                                        ->  ``apb200::attention``
* ``F.embedding`` / ``nn.Embedding`` without padding index or norm clipping  ->  ``apb200::embedding`` (own gather kernel,
  gradient through ``apb200::embedding_bwd``)
* rotary embedding by complex multiplication, ``view_as_real(view_as_complex(x.float().reshape(..., -1, 2)) * f)
  .flatten(3).type_as(x)``                                                 ->  ``apb200::rope``

Every rewrite is local and keeps the value (same dtype, same shape); anything that does not match
exactly is left as it is.  Reference counterpart: the reference gets operator fusion from Inductor
(autoparallel/compile.py:259-310) and runs its model's ``nn.RMSNorm`` / complex RoPE / ``F.silu`` /
SDPA as traced (autoparallel/_testing/models/llama3.py:187-213, 355-356, 396-397).
"""
from __future__ import annotations

import math
import operator

import torch
import torch.fx as fx
import torch.nn.functional as F

apb = torch.ops.apb200


def _val(n):
    v = n.meta.get("example_value", n.meta.get("val")) if isinstance(n, fx.Node) else None
    return v if isinstance(v, torch.Tensor) else None


def _is_method(n, name):
    return isinstance(n, fx.Node) and n.op == "call_method" and n.target == name


def _is_fn(n, *fns):
    return isinstance(n, fx.Node) and n.op == "call_function" and any(n.target is f for f in fns)


def _arg(n, i, name=None, default=None):
    if len(n.args) > i:
        return n.args[i]
    return n.kwargs.get(name, default) if name else default


def _copy_meta(dst: fx.Node, src: fx.Node):
    for k in ("example_value", "val", "stack_trace", "nn_module_stack", "source_fn_stack", "custom"):
        if k in src.meta:
            dst.meta[k] = src.meta[k]


# ------------------------------------------------------------------------------------------ RMSNorm
def _rewrite_rms_norm(g: fx.Graph) -> int:
    count = 0
    for n in list(g.nodes):
        if not _is_fn(n, torch.rms_norm, F.rms_norm):
            continue
        x, shape, w, eps = _arg(n, 0, "input"), _arg(n, 1, "normalized_shape"), _arg(n, 2, "weight"), _arg(n, 3, "eps")
        xv = _val(x)
        if w is None or xv is None or not isinstance(shape, (tuple, list, torch.Size)) or len(shape) != 1 or xv.shape[-1] % 8:
            continue
        if eps is None:
            eps = torch.finfo(xv.dtype).eps
        with g.inserting_before(n):
            pair = g.call_function(apb.rms_norm.default, (x, w, float(eps)))
            y = g.call_function(operator.getitem, (pair, 0))
        _copy_meta(y, n)
        n.replace_all_uses_with(y)
        g.erase_node(n)
        count += 1
    return count


def _strip_casts(n):
    """x.float() / x.to(torch.float32) -> x (the operators compute in fp32 themselves)."""
    while isinstance(n, fx.Node) and n.op == "call_method" and (
            n.target == "float" or (n.target == "to" and len(n.args) == 2 and n.args[1] in (torch.float32,))):
        n = n.args[0]
    return n


def _rewrite_manual_rms_norm(g: fx.Graph) -> int:
    """``weight * (h * rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)`` with ``h = x.to(float32)``."""
    count = 0
    for rs in list(g.nodes):
        if not _is_fn(rs, torch.rsqrt):
            continue
        add = rs.args[0]
        if not _is_fn(add, operator.add) or not isinstance(add.args[1], (int, float)):
            continue
        mean, eps = add.args[0], float(add.args[1])
        if not (_is_method(mean, "mean") and _arg(mean, 1, "dim") in (-1, (-1,), [-1]) and mean.kwargs.get("keepdim", _arg(mean, 2)) is True):
            continue
        pw = mean.args[0]
        if not (_is_method(pw, "pow") and pw.args[1] == 2):
            continue
        h = pw.args[0]
        scaled = [u for u in rs.users if _is_fn(u, operator.mul) and (u.args[0] is h or u.args[1] is h)]
        if len(scaled) != 1 or len(rs.users) != 1:
            continue
        y = scaled[0]
        # optional cast back to the input dtype, then multiplication by the weight
        nxt = y
        if len(y.users) == 1 and _is_method(next(iter(y.users)), "to"):
            nxt = next(iter(y.users))
        if len(nxt.users) != 1:
            continue
        wm = next(iter(nxt.users))
        if not _is_fn(wm, operator.mul):
            continue
        w = wm.args[0] if wm.args[1] is nxt else wm.args[1]
        x = _strip_casts(h)
        xv, wv, outv = _val(x), _val(w), _val(wm)
        if xv is None or wv is None or outv is None or wv.ndim != 1 or wv.shape[0] != xv.shape[-1] or xv.shape[-1] % 8:
            continue
        if outv.dtype != xv.dtype or outv.shape != xv.shape:
            continue
        with g.inserting_before(wm):
            pair = g.call_function(apb.rms_norm.default, (x, w, eps))
            out = g.call_function(operator.getitem, (pair, 0))
        _copy_meta(out, wm)
        wm.replace_all_uses_with(out)
        count += 1
    if count:
        g.eliminate_dead_code()
    return count


# ------------------------------------------------------------------------------------------ SwiGLU
def _rewrite_swiglu(g: fx.Graph) -> int:
    count = 0
    for n in list(g.nodes):
        if not _is_fn(n, operator.mul, torch.mul):
            continue
        a, b = n.args[0], n.args[1]
        for s, other in ((a, b), (b, a)):
            if _is_fn(s, F.silu) and len(s.users) == 1 and isinstance(other, fx.Node):
                sv, ov = _val(s.args[0]), _val(other)
                if sv is None or ov is None or sv.shape != ov.shape or sv.dtype != ov.dtype or sv.numel() % 8:
                    continue
                with g.inserting_before(n):
                    y = g.call_function(apb.swiglu.default, (s.args[0], other))
                _copy_meta(y, n)
                n.replace_all_uses_with(y)
                g.erase_node(n)
                g.erase_node(s)
                count += 1
                break
    return count


# ------------------------------------------------------------------------------------------ attention
def _through_transpose_12(n):
    """heads-first [B, H, S, D] value that is ``t.transpose(1, 2)`` of a [B, S, H, D] tensor -> t."""
    if _is_method(n, "transpose") and set(n.args[1:3]) == {1, 2}:
        return n.args[0]
    if _is_method(n, "permute") and tuple(n.args[1:]) in ((0, 2, 1, 3),):
        return n.args[0]
    return None


def _through_repeat_kv(n):
    """[B, S, Hkv * rep, D] built as ``x.unsqueeze(3).expand(B, S, Hkv, rep, D).reshape(B, S, H, D)`` -> x."""
    if not (_is_method(n, "reshape") or _is_method(n, "view")):
        return None
    e = n.args[0]
    if not _is_method(e, "expand"):
        return None
    u = e.args[0]
    src = None
    if _is_fn(u, torch.unsqueeze) and (_arg(u, 1, "dim") == 3):
        src = u.args[0]
    elif _is_method(u, "unsqueeze") and u.args[1] == 3:
        src = u.args[0]
    elif _is_fn(u, operator.getitem) and isinstance(u.args[1], tuple) and len(u.args[1]) == 5 and u.args[1][3] is None:
        src = u.args[0]
    sv, nv = _val(src) if src is not None else None, _val(n)
    if sv is None or nv is None or sv.ndim != 4 or nv.ndim != 4:
        return None
    if sv.shape[0] == nv.shape[0] and sv.shape[1] == nv.shape[1] and sv.shape[3] == nv.shape[3] and nv.shape[2] % sv.shape[2] == 0:
        return src
    return None


def _rewrite_sdpa(g: fx.Graph) -> int:
    count = 0
    for n in list(g.nodes):
        if not _is_fn(n, F.scaled_dot_product_attention):
            continue
        q, k, v = n.args[0], n.args[1], n.args[2]
        mask = _arg(n, 3, "attn_mask")
        drop = _arg(n, 4, "dropout_p", 0.0)
        causal = bool(_arg(n, 5, "is_causal", False))
        scale = _arg(n, 6, "scale")
        if mask is not None or drop not in (0, 0.0) or n.kwargs.get("enable_gqa", False):
            continue
        qv, kv = _val(q), _val(k)
        if qv is None or kv is None or qv.ndim != 4 or qv.shape[-1] % 8:
            continue
        if scale is None:
            scale = 1.0 / math.sqrt(qv.shape[-1])
        with g.inserting_before(n):
            def to_bshd(t):
                src = _through_transpose_12(t)
                return src if src is not None else g.call_method("transpose", (t, 1, 2))

            qb, kb, vb = to_bshd(q), to_bshd(k), to_bshd(v)
            # grouped-query heads: the operator reads them in place, the expansion is not needed
            ks, vs = _through_repeat_kv(kb), _through_repeat_kv(vb)
            if ks is not None and vs is not None:
                kb, vb = ks, vs
            pair = g.call_function(apb.attention.default, (qb, kb, vb, causal, float(scale)))
            out = g.call_function(operator.getitem, (pair, 0))
            back = g.call_method("transpose", (out, 1, 2))
        _copy_meta(back, n)
        n.replace_all_uses_with(back)
        g.erase_node(n)
        count += 1
    if count:
        g.eliminate_dead_code()
    return count


# ------------------------------------------------------------------------------------------ RoPE (complex form)
def _rewrite_complex_rope(g: fx.Graph) -> int:
    count = 0
    tables: dict = {}  # frequency node -> (cos, sin) nodes
    for vr in list(g.nodes):
        if not _is_fn(vr, torch.view_as_real):
            continue
        m = vr.args[0]
        if not _is_fn(m, operator.mul, torch.mul):
            continue
        xc, f = m.args
        if not _is_fn(xc, torch.view_as_complex):
            xc, f = f, xc
        if not _is_fn(xc, torch.view_as_complex) or not isinstance(f, fx.Node):
            continue
        rs = xc.args[0]
        if not (_is_method(rs, "reshape") or _is_method(rs, "view")) or rs.args[-1] != 2:
            continue
        x = _strip_casts(rs.args[0])
        xv, fv = _val(x), _val(f)
        if xv is None or fv is None or xv.ndim != 4 or not fv.is_complex() or xv.shape[-1] % 8:
            continue
        B, S, H, D = xv.shape
        # the frequencies broadcast over batch and heads: [1, S, 1, D/2] (or [S, D/2] before a view)
        if fv.numel() != S * (D // 2):
            continue
        # consumers: flatten(3) then an optional type_as / to
        if len(vr.users) != 1:
            continue
        fl = next(iter(vr.users))
        if not (_is_method(fl, "flatten") and fl.args[1] == 3):
            continue
        end = fl
        if len(fl.users) == 1:
            u = next(iter(fl.users))
            if _is_method(u, "type_as") or _is_method(u, "to"):
                end = u
        ev = _val(end)
        if ev is None or ev.dtype != xv.dtype or ev.shape != xv.shape:
            continue
        if f not in tables:
            with g.inserting_after(f):
                fr = g.call_function(torch.view_as_real, (f,))
            with g.inserting_after(fr):
                flat = g.call_method("reshape", (fr, S, D // 2, 2))
            with g.inserting_after(flat):
                cos = g.call_function(operator.getitem, (flat, (slice(None), slice(None), 0)))
            with g.inserting_after(cos):
                sin = g.call_function(operator.getitem, (flat, (slice(None), slice(None), 1)))
            tables[f] = (cos, sin)
        cos, sin = tables[f]
        with g.inserting_before(end):
            y = g.call_function(apb.rope.default, (x, cos, sin, False))
        _copy_meta(y, end)
        end.replace_all_uses_with(y)
        count += 1
    if count:
        g.eliminate_dead_code()
    return count


# ------------------------------------------------------------------------------------------ embedding
def _rewrite_embedding(g: fx.Graph) -> int:
    count = 0
    for n in list(g.nodes):
        if not _is_fn(n, F.embedding):
            continue
        ids, w = _arg(n, 0, "input"), _arg(n, 1, "weight")
        plain = (_arg(n, 2, "padding_idx") is None and _arg(n, 3, "max_norm") is None and not _arg(n, 5, "scale_grad_by_freq", False)
                 and not _arg(n, 6, "sparse", False))
        wv, iv = _val(w), _val(ids)
        if not plain or wv is None or iv is None or wv.ndim != 2 or iv.dtype != torch.long:
            continue
        with g.inserting_before(n):
            y = g.call_function(apb.embedding.default, (w, ids))
        _copy_meta(y, n)
        n.replace_all_uses_with(y)
        g.erase_node(n)
        count += 1
    return count


# ------------------------------------------------------------------------------------------ fp8 projection
def _rewrite_scaled_mm(g: fx.Graph) -> int:
    """``torch._scaled_mm(a, b, scale_a, scale_b, out_dtype=..)`` without bias or result scale -> ``apb200::scaled_mm``.
    A second operand written as ``w.t()`` (how float8 linears pass a row-major weight) is folded into ``trans_b``, so
    the planner sees the weight as stored and its row-wise scale [N, 1] as a per-row tensor of it."""
    count = 0
    for n in list(g.nodes):
        if not _is_fn(n, torch._scaled_mm):
            continue
        a, b, sa, sb = _arg(n, 0, "self"), _arg(n, 1, "mat2"), _arg(n, 2, "scale_a"), _arg(n, 3, "scale_b")
        if _arg(n, 4, "bias") is not None or _arg(n, 5, "scale_result") is not None:
            continue
        out_dtype = _arg(n, 6, "out_dtype")
        av, bv, sav, sbv = _val(a), _val(b), _val(sa), _val(sb)
        if av is None or bv is None or sav is None or sbv is None or av.ndim != 2 or bv.ndim != 2:
            continue
        if out_dtype is None:
            out_dtype = av.dtype
        trans_b = False
        if _is_method(b, "t") or (_is_method(b, "transpose") and set(b.args[1:]) in ({0, 1}, {-1, -2}, {0, -1}, {1, -2})):
            src = b.args[0]
            if _val(src) is not None and _val(src).ndim == 2:
                # scale_b [1, N] belongs to the columns of b = rows of the stored weight: hand it over as [N, 1]
                with g.inserting_before(n):
                    sb_t = g.call_method("reshape", (sb, -1, 1)) if sbv.numel() > 1 else sb
                if sb_t is not sb and "example_value" in sb.meta:
                    sb_t.meta["example_value"] = sbv.reshape(-1, 1)
                b, sb, trans_b = src, sb_t, True
        with g.inserting_before(n):
            y = g.call_function(apb.scaled_mm.default, (a, b, sa, sb, trans_b, out_dtype))
        _copy_meta(y, n)
        n.replace_all_uses_with(y)
        g.erase_node(n)
        count += 1
    return count


def rewrite_to_framework_ops(gm: fx.GraphModule) -> dict:
    """Apply every pattern to a Dynamo-level (torch IR) graph in place; returns how many of each were rewritten."""
    g = gm.graph
    stats = {
        "rms_norm": _rewrite_rms_norm(g) + _rewrite_manual_rms_norm(g),
        "swiglu": _rewrite_swiglu(g),
        "attention": _rewrite_sdpa(g),
        "rope": _rewrite_complex_rope(g),
        "embedding": _rewrite_embedding(g),
        "scaled_mm": _rewrite_scaled_mm(g),
    }
    if any(stats.values()):
        g.lint()
        gm.recompile()
    return stats
