"""Operator library of the framework: schemas, CPU reference kernels, meta kernels, autograd.

Every hot op of the model zoo is a ``torch.library`` operator in the ``apb200``
namespace.  A schema is defined once here; three implementations hang off it:

* ``CPU``  – a plain PyTorch fp32 restatement (the numerics oracle of the test-suite and
  what planner tests execute on machines without a GPU),
* ``Meta`` – shape/dtype propagation, so fake-tensor tracing of the joint graph works,
* ``CUDA`` – the hand-written sm_100a kernels (registered by ``ops.cuda_impl`` once the
  in-tree extension is loaded; a CUDA tensor reaching an op without it raises).

Backward formulas are themselves ``apb200`` ops, so a traced joint forward/backward graph
contains only planner-visible nodes (the planner has a sharding rule per op, see
``parallel/strategies/rules.py``).

The reference reaches the same math through ATen / cuDNN / Inductor instead:
RMSNorm (autoparallel/_testing/models/llama3.py:396), RoPE (llama3.py:187-213), SwiGLU
(llama3.py:355-356), SDPA (llama3.py:49-54), ``autoparallel::dtype_cast``
(autoparallel/cast_parametrization.py:71-100).
"""
from __future__ import annotations

import math

import torch

NS = "apb200"
lib = torch.library.Library(NS, "DEF")  # noqa: TOR901

_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32]


def dtype_to_code(dt: torch.dtype) -> int:
    return _DTYPES.index(dt)


def code_to_dtype(code: int) -> torch.dtype:
    return _DTYPES[code]


# --------------------------------------------------------------------------------------
# schemas
# --------------------------------------------------------------------------------------
lib.define("dtype_cast(Tensor x, ScalarType dtype) -> Tensor")


def _cast_ref(x, dtype):
    from . import shadow

    hit = shadow.lookup(x, dtype) if x.dtype != dtype else None
    return hit if hit is not None else x.to(dtype)

lib.define("rms_norm(Tensor x, Tensor weight, float eps) -> (Tensor, Tensor)")
lib.define("rms_norm_bwd(Tensor dy, Tensor x, Tensor weight, Tensor rstd) -> (Tensor, Tensor)")
lib.define("rope(Tensor x, Tensor cos, Tensor sin, bool conj) -> Tensor")
lib.define("swiglu(Tensor a, Tensor b) -> Tensor")
lib.define("swiglu_bwd(Tensor dy, Tensor a, Tensor b) -> (Tensor, Tensor)")
lib.define("attention(Tensor q, Tensor k, Tensor v, bool causal, float scale) -> (Tensor, Tensor)")
lib.define(
    "attention_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor out, Tensor lse, bool causal, float scale)"
    " -> (Tensor, Tensor, Tensor)"
)
lib.define("cross_entropy(Tensor logits, Tensor labels) -> (Tensor, Tensor)")
lib.define("cross_entropy_bwd(Tensor dloss, Tensor logits, Tensor labels, Tensor lse) -> Tensor")
# C[M,N] = op(A) @ op(B); trans flags are about the *stored* layout (row-major storage).
lib.define("gemm(Tensor a, Tensor b, bool trans_a, bool trans_b, ScalarType out_dtype) -> Tensor")
lib.define("embedding(Tensor weight, Tensor ids) -> Tensor")
lib.define("embedding_bwd(Tensor dy, Tensor ids, int num_rows) -> Tensor")


# --------------------------------------------------------------------------------------
# CPU reference kernels (fp32 math)
# --------------------------------------------------------------------------------------
def _rms_norm_ref(x, weight, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * weight.float()).to(x.dtype)
    return y, rstd.squeeze(-1)


def _rms_norm_bwd_ref(dy, x, weight, rstd):
    xf, dyf, wf = x.float(), dy.float(), weight.float()
    r = rstd.unsqueeze(-1)
    xhat = xf * r
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    g = dyf * wf
    dx = r * (g - xhat * (g * xhat).mean(-1, keepdim=True))
    return dx.to(x.dtype), dw.to(weight.dtype)


def _rope_ref(x, cos, sin, conj):
    # x: [B, S, H, D]; cos/sin: [S, D/2]; pairs are interleaved (x[..., 2i], x[..., 2i+1]).
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c = cos.float()[None, :, None, :]
    s = sin.float()[None, :, None, :]
    if conj:
        s = -s
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack((a * c - b * s, a * s + b * c), dim=-1)
    return out.reshape(x.shape).to(x.dtype)


def _swiglu_ref(a, b):
    return (torch.nn.functional.silu(a.float()) * b.float()).to(a.dtype)


def _swiglu_bwd_ref(dy, a, b):
    af, bf, dyf = a.float(), b.float(), dy.float()
    sig = torch.sigmoid(af)
    silu = af * sig
    da = dyf * bf * (sig * (1 + af * (1 - sig)))
    db = dyf * silu
    return da.to(a.dtype), db.to(b.dtype)


def _attention_ref(q, k, v, causal, scale):
    # q: [B, S, H, D]; k, v: [B, S, Hkv, D] -> out [B, S, H, D], lse [B, H, S] (natural log)
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sk = k.shape[1]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3).contiguous()
    return o.to(q.dtype), lse


def _attention_bwd_ref(dout, q, k, v, out, lse, causal, scale):
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    rep = H // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    dof = dout.float().permute(0, 2, 1, 3)
    of = out.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sk = k.shape[1]
        mask = torch.ones(S, Sk, dtype=torch.bool, device=q.device).tril(Sk - S)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    Sk = k.shape[1]
    dk = dk.reshape(B, Hkv, rep, Sk, D).sum(2)
    dv = dv.reshape(B, Hkv, rep, Sk, D).sum(2)
    return (
        dq.permute(0, 2, 1, 3).contiguous().to(q.dtype),
        dk.permute(0, 2, 1, 3).contiguous().to(k.dtype),
        dv.permute(0, 2, 1, 3).contiguous().to(v.dtype),
    )


def _cross_entropy_ref(logits, labels):
    # logits [..., V], labels [...] -> per-token loss fp32 [...], lse fp32 [...]
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    picked = torch.gather(lf, -1, labels.unsqueeze(-1)).squeeze(-1)
    return lse - picked, lse


def _cross_entropy_bwd_ref(dloss, logits, labels, lse):
    p = torch.exp(logits.float() - lse.unsqueeze(-1))
    p.scatter_add_(-1, labels.unsqueeze(-1), -torch.ones_like(p[..., :1]))
    return (p * dloss.float().unsqueeze(-1)).to(logits.dtype)


def _gemm_ref(a, b, trans_a, trans_b, out_dtype):
    A = a.transpose(-1, -2) if trans_a else a
    Bm = b.transpose(-1, -2) if trans_b else b
    if a.dtype in (torch.bfloat16, torch.float16):
        return torch.matmul(A.float(), Bm.float()).to(out_dtype)
    return torch.matmul(A, Bm).to(out_dtype)


def _embedding_bwd_ref(dy, ids, num_rows):
    out = torch.zeros(num_rows, dy.shape[-1], dtype=torch.float32, device=dy.device)
    out.index_add_(0, ids.reshape(-1), dy.reshape(-1, dy.shape[-1]).float())
    return out.to(dy.dtype)


_CPU_IMPLS = {
    "dtype_cast": lambda x, dtype: _cast_ref(x, dtype),
    "rms_norm": _rms_norm_ref,
    "rms_norm_bwd": _rms_norm_bwd_ref,
    "rope": _rope_ref,
    "swiglu": _swiglu_ref,
    "swiglu_bwd": _swiglu_bwd_ref,
    "attention": _attention_ref,
    "attention_bwd": _attention_bwd_ref,
    "cross_entropy": _cross_entropy_ref,
    "cross_entropy_bwd": _cross_entropy_bwd_ref,
    "gemm": _gemm_ref,
    "embedding": lambda weight, ids: torch.nn.functional.embedding(ids, weight),
    "embedding_bwd": _embedding_bwd_ref,
}
for _name, _fn in _CPU_IMPLS.items():
    lib.impl(_name, _fn, "CPU")

#: reference implementations by op name, used by GPU numerics tests as the oracle.
reference_impls = dict(_CPU_IMPLS)


# --------------------------------------------------------------------------------------
# meta kernels
# --------------------------------------------------------------------------------------
def _meta_like(x, dtype=None, shape=None):
    return torch.empty(shape if shape is not None else x.shape, dtype=dtype or x.dtype, device=x.device)


def _gemm_meta(a, b, trans_a, trans_b, out_dtype):
    m = a.shape[-1] if trans_a else a.shape[-2]
    n = b.shape[-2] if trans_b else b.shape[-1]
    return a.new_empty((*a.shape[:-2], m, n), dtype=out_dtype)


_META_IMPLS = {
    "dtype_cast": lambda x, dtype: _meta_like(x, dtype=dtype),
    "rms_norm": lambda x, w, eps: (_meta_like(x), _meta_like(x, torch.float32, x.shape[:-1])),
    "rms_norm_bwd": lambda dy, x, w, rstd: (_meta_like(x), _meta_like(w)),
    "rope": lambda x, cos, sin, conj: _meta_like(x),
    "swiglu": lambda a, b: _meta_like(a),
    "swiglu_bwd": lambda dy, a, b: (_meta_like(a), _meta_like(b)),
    "attention": lambda q, k, v, causal, scale: (
        _meta_like(q),
        _meta_like(q, torch.float32, (q.shape[0], q.shape[2], q.shape[1])),
    ),
    "attention_bwd": lambda dout, q, k, v, out, lse, causal, scale: (_meta_like(q), _meta_like(k), _meta_like(v)),
    "cross_entropy": lambda logits, labels: (
        _meta_like(logits, torch.float32, logits.shape[:-1]),
        _meta_like(logits, torch.float32, logits.shape[:-1]),
    ),
    "cross_entropy_bwd": lambda dloss, logits, labels, lse: _meta_like(logits),
    "gemm": _gemm_meta,
    "embedding": lambda weight, ids: weight.new_empty((*ids.shape, weight.shape[1])),
    "embedding_bwd": lambda dy, ids, num_rows: dy.new_empty((num_rows, dy.shape[-1])),
}
for _name, _fn in _META_IMPLS.items():
    lib.impl(_name, _fn, "Meta")


# --------------------------------------------------------------------------------------
# CUDA: a guard kernel until ops.cuda_impl installs the sm_100a kernels.
# --------------------------------------------------------------------------------------
_cuda_table: dict[str, object] = {}


def _make_cuda_entry(name):
    def entry(*args):
        fn = _cuda_table.get(name)
        if fn is None:
            from . import cuda_impl

            cuda_impl.ensure_loaded()
            fn = _cuda_table.get(name)
            if fn is None:
                raise RuntimeError(
                    f"apb200::{name} received a CUDA tensor but the sm_100a extension provides no kernel for it"
                )
        return fn(*args)

    return entry


for _name in _CPU_IMPLS:
    lib.impl(_name, _make_cuda_entry(_name), "CUDA")


def register_cuda_impl(name: str, fn) -> None:
    """Install the sm_100a kernel wrapper for ``apb200::<name>``."""
    _cuda_table[name] = fn


# --------------------------------------------------------------------------------------
# autograd
# --------------------------------------------------------------------------------------
ops = getattr(torch.ops, NS)


def _ag(name, backward, setup):
    torch.library.register_autograd(f"{NS}::{name}", backward, setup_context=setup, lib=lib)


def _cast_setup(ctx, inputs, output):
    ctx.src_dtype = inputs[0].dtype


_ag("dtype_cast", lambda ctx, g: (ops.dtype_cast(g, ctx.src_dtype), None), _cast_setup)


def _rms_setup(ctx, inputs, output):
    x, w, _ = inputs
    ctx.save_for_backward(x, w, output[1])


def _rms_bwd(ctx, dy, _drstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = ops.rms_norm_bwd(dy, x, w, rstd)
    return dx, dw, None


_ag("rms_norm", _rms_bwd, _rms_setup)


def _rope_setup(ctx, inputs, output):
    _, cos, sin, conj = inputs
    ctx.save_for_backward(cos, sin)
    ctx.conj = conj


def _rope_bwd(ctx, dy):
    cos, sin = ctx.saved_tensors
    return ops.rope(dy, cos, sin, not ctx.conj), None, None, None


_ag("rope", _rope_bwd, _rope_setup)


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swiglu_bwd(ctx, dy):
    a, b = ctx.saved_tensors
    return ops.swiglu_bwd(dy, a, b)


_ag("swiglu", _swiglu_bwd, _swiglu_setup)


def _attn_setup(ctx, inputs, output):
    q, k, v, causal, scale = inputs
    ctx.save_for_backward(q, k, v, output[0], output[1])
    ctx.causal, ctx.scale = causal, scale


def _attn_bwd(ctx, dout, _dlse):
    q, k, v, out, lse = ctx.saved_tensors
    dq, dk, dv = ops.attention_bwd(dout, q, k, v, out, lse, ctx.causal, ctx.scale)
    return dq, dk, dv, None, None


_ag("attention", _attn_bwd, _attn_setup)


def _ce_setup(ctx, inputs, output):
    logits, labels = inputs
    ctx.save_for_backward(logits, labels, output[1])


def _ce_bwd(ctx, dloss, _dlse):
    logits, labels, lse = ctx.saved_tensors
    return ops.cross_entropy_bwd(dloss, logits, labels, lse), None


_ag("cross_entropy", _ce_bwd, _ce_setup)


def _gemm_setup(ctx, inputs, output):
    a, b, ta, tb, _ = inputs
    ctx.save_for_backward(a, b)
    ctx.ta, ctx.tb = ta, tb


def _gemm_bwd(ctx, dc):
    a, b = ctx.saved_tensors
    ta, tb = ctx.ta, ctx.tb
    # C = op(A) op(B).  dA_op = dC op(B)^T, dB_op = op(A)^T dC, then undo the storage transpose.
    if not ta:
        da = ops.gemm(dc, b, False, not tb, a.dtype)
    else:
        da = ops.gemm(b, dc, tb, True, a.dtype)
    if not tb:
        db = ops.gemm(a, dc, not ta, False, b.dtype)
    else:
        db = ops.gemm(dc, a, True, ta, b.dtype)
    return da, db, None, None, None


_ag("gemm", _gemm_bwd, _gemm_setup)


def _emb_setup(ctx, inputs, output):
    weight, ids = inputs
    ctx.save_for_backward(ids)
    ctx.num_rows = weight.shape[0]


def _emb_bwd(ctx, dy):
    (ids,) = ctx.saved_tensors
    return ops.embedding_bwd(dy, ids, ctx.num_rows), None


_ag("embedding", _emb_bwd, _emb_setup)


# --------------------------------------------------------------------------------------
# thin functional front-ends used by the model zoo
# --------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return ops.rms_norm(x, weight, eps)[0]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return ops.rope(x, cos, sin, False)


def swiglu(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ops.swiglu(a, b)


def attention(q, k, v, causal: bool = True, scale: float | None = None) -> torch.Tensor:
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return ops.attention(q, k, v, causal, float(scale))[0]


def embedding(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Rows ``ids`` of ``weight`` ([V, D]); the gradient is scattered back by ``embedding_bwd``."""
    return ops.embedding(weight, ids)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Mean next-token cross-entropy over all positions of ``labels``."""
    return ops.cross_entropy(logits, labels)[0].mean()


def dtype_cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return ops.dtype_cast(x, dtype)


# --------------------------------------------------------------------------------------
# N-d linear algebra ops that the graph canonicaliser substitutes for
# ``view -> aten.mm -> view`` chains.  Keeping the leading dims un-flattened is what lets the
# planner shard the sequence dim of ``[B, S, K]`` activations through a projection (the
# reference gets the same effect by rewriting to einsum, autoparallel/graph_passes/
# graph_utils.py:270-439).  Both map 1:1 onto one launch of the tcgen05 GEMM kernel.
# --------------------------------------------------------------------------------------
lib.define("mm_nd(Tensor a, Tensor b, bool trans_b, ScalarType out_dtype) -> Tensor")
lib.define("mm_wgrad(Tensor a, Tensor b, ScalarType out_dtype) -> Tensor")


def _mm_nd_ref(a, b, trans_b, out_dtype):
    """``a[..., K] @ (b[N, K]^T if trans_b else b[K, N]) -> [..., N]``."""
    lead = a.shape[:-1]
    out = _gemm_ref(a.reshape(-1, a.shape[-1]), b, False, trans_b, out_dtype)
    return out.reshape(*lead, out.shape[-1])


def _mm_wgrad_ref(a, b, out_dtype):
    """``sum over leading dims of a[..., M]^T b[..., N] -> [M, N]``."""
    return _gemm_ref(a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1]), True, False, out_dtype)


def _mm_nd_meta(a, b, trans_b, out_dtype):
    n = b.shape[0] if trans_b else b.shape[1]
    return a.new_empty((*a.shape[:-1], n), dtype=out_dtype)


lib.impl("mm_nd", _mm_nd_ref, "CPU")
lib.impl("mm_wgrad", _mm_wgrad_ref, "CPU")
lib.impl("mm_nd", _mm_nd_meta, "Meta")
lib.impl("mm_wgrad", lambda a, b, out_dtype: a.new_empty((a.shape[-1], b.shape[-1]), dtype=out_dtype), "Meta")
lib.impl("mm_nd", _make_cuda_entry("mm_nd"), "CUDA")
lib.impl("mm_wgrad", _make_cuda_entry("mm_wgrad"), "CUDA")
reference_impls["mm_nd"] = _mm_nd_ref
reference_impls["mm_wgrad"] = _mm_wgrad_ref


# --------------------------------------------------------------------------------------
# fp8 projection with scales: ``(a * scale_a) @ (b * scale_b)`` accumulated in fp32.  ``a`` [..., K] and ``b``
# ([N, K] when ``trans_b`` else [K, N]) are float8 tensors; a scale is a scalar (tensor-wise) or, row-wise, has the
# operand's shape with the contraction dim reduced to 1 (``scale_a`` [..., 1]; ``scale_b`` [N, 1] / [1, N]).
# The planner sees it like ``mm_nd`` with the scales sharded along with the rows they belong to.  No autograd
# formula: float8 training wraps it in its own autograd function, as with ``torch._scaled_mm`` (reference:
# autoparallel/graph_passes/async_tp/asynctp_ops.py:363-393 for the scale modes).
# --------------------------------------------------------------------------------------
lib.define("scaled_mm(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, bool trans_b, ScalarType out_dtype) -> Tensor")


def _scaled_mm_ref(a, b, scale_a, scale_b, trans_b, out_dtype):
    af = a.float() * scale_a.float()
    bf = b.float() * scale_b.float()
    lead = af.shape[:-1]
    out = af.reshape(-1, af.shape[-1]) @ (bf.t() if trans_b else bf)
    return out.reshape(*lead, out.shape[-1]).to(out_dtype)


def _scaled_mm_meta(a, b, scale_a, scale_b, trans_b, out_dtype):
    n = b.shape[0] if trans_b else b.shape[1]
    return a.new_empty((*a.shape[:-1], n), dtype=out_dtype)


lib.impl("scaled_mm", _scaled_mm_ref, "CPU")
lib.impl("scaled_mm", _scaled_mm_meta, "Meta")
lib.impl("scaled_mm", _make_cuda_entry("scaled_mm"), "CUDA")
reference_impls["scaled_mm"] = _scaled_mm_ref


def _mm_nd_setup(ctx, inputs, output):
    a, b, tb, _ = inputs
    ctx.save_for_backward(a, b)
    ctx.tb = tb


def _mm_nd_bwd(ctx, dc):
    a, b = ctx.saved_tensors
    da = ops.mm_nd(dc, b, not ctx.tb, a.dtype)
    db = ops.mm_wgrad(dc, a, b.dtype) if ctx.tb else ops.mm_wgrad(a, dc, b.dtype)
    return da, db, None, None


_ag("mm_nd", _mm_nd_bwd, _mm_nd_setup)
