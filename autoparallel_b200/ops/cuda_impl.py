"""CUDA implementations of the ``apb200`` operators on the in-tree sm_100a extension.

Loaded on first use of an op with a CUDA tensor.  If the extension is missing on a machine with a
GPU the op raises.  A few inputs are outside what the kernels take and are answered by a library
call instead; each such call is counted in ``library_fallbacks`` (printed by ``bench.py``) and the
first of each kind is logged once, so a run never uses a library path without saying so:

* ``gemm``          operands that are not bf16 (fp32 / fp16 models), or row strides that are not a
                    multiple of 16 bytes (TMA cannot address them) -> ``torch.matmul``
* ``grouped_gemm``  the same conditions for the expert GEMMs -> the PyTorch composition
* ``cast``          dtype pairs other than fp32 <-> bf16, or unaligned / strided inputs -> ``Tensor.to``
* ``attention``     the fused-attention library kernel (cuDNN) when the own kernel is not selected

``APB200_DIAG_LIBRARY_GEMM=1`` sends every GEMM to the library (a diagnostic for comparing power and
time of a whole step; counted like any other fallback).
"""
from __future__ import annotations

import importlib
import os
import threading

import torch

from . import library as L

_C = None
_lock = threading.Lock()
_status: dict[int, torch.Tensor] = {}
_scratch: dict[tuple, torch.Tensor] = {}
launch_count = 0  # kernels of this extension launched since import (bench bookkeeping)
#: calls answered by a library kernel instead of this extension's, by kind
library_fallbacks: dict[str, int] = {}
_DIAG_LIBRARY_GEMM = os.environ.get("APB200_DIAG_LIBRARY_GEMM") == "1"


def _fallback(kind: str, why: str) -> None:
    n = library_fallbacks.get(kind, 0)
    library_fallbacks[kind] = n + 1
    if n == 0:
        import logging

        logging.getLogger("autoparallel_b200").warning("library fallback for %s: %s (counted in cuda_impl.library_fallbacks)", kind, why)

STATUS_NAMES = {
    0: "ok",
    1: "GEMM consumer timed out waiting for a TMA stage",
    2: "GEMM producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for an accumulator",
    4: "MMA issuer timed out waiting for a free accumulator",
    5: "timed out waiting for a peer flag",
    6: "bad argument",
    7: "attention: MMA issuer timed out waiting for a K / V tile",
    8: "attention: loader timed out waiting for a free K / V slot",
    9: "attention: softmax timed out waiting for a score or product accumulator",
    10: "attention: MMA issuer timed out waiting for a probability tile",
}


def extension():
    return _C


def ensure_loaded() -> None:
    global _C
    if _C is not None:
        return
    with _lock:
        if _C is not None:
            return
        from . import build

        if not os.path.exists(build.so_path()):
            if os.environ.get("APB200_NO_JIT_BUILD"):
                raise RuntimeError(
                    "the sm_100a extension is not built: run `python -m autoparallel_b200.ops.build` "
                    "(or __graft_entry__.build())"
                )
            build.build()
        _C = importlib.import_module("autoparallel_b200.ops._C")
        _register()


def status_buffer(device) -> torch.Tensor:
    idx = torch.device(device).index or 0
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device=None) -> None:
    """Raise if any kernel on ``device`` recorded a timed-out wait (synchronises)."""
    for idx, t in _status.items():
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(t[0].item())
        if code != 0:
            t.zero_()
            raise RuntimeError(f"apb200 kernel status {code} on cuda:{idx}: {STATUS_NAMES.get(code, 'unknown')}")


def _scratch_f32(device, n: int) -> torch.Tensor:
    key = (torch.device(device).index or 0, "f32")
    t = _scratch.get(key)
    if t is None or t.numel() < n:
        t = torch.empty(max(n, 16384), dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ----------------------------------------------------------------------------------- GEMM family
def _as2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(-1) != 1 or (t2.stride(0) % 8) != 0 or (t2.data_ptr() % 16) != 0:
        t2 = t2.contiguous()
    return t2


def gemm_raw(a2: torch.Tensor, b2: torch.Tensor, a_mn: bool, b_mn: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """C[M,N] = opA @ opB on the tcgen05 kernel.  a2: [M,K] or [K,M] if a_mn; b2: [N,K] or [K,N] if b_mn."""
    M = a2.shape[1] if a_mn else a2.shape[0]
    N = b2.shape[1] if b_mn else b2.shape[0]
    if (_DIAG_LIBRARY_GEMM or a2.dtype != torch.bfloat16 or b2.dtype != torch.bfloat16 or (a2.shape[1] % 8) or (b2.shape[1] % 8)
            or (N % 8)):
        # fp32 / fp16 operands, or row strides TMA cannot address (not multiples of 16 bytes):
        # library GEMM (not a tensor-core path of this framework)
        _fallback("gemm", f"dtypes {a2.dtype}/{b2.dtype}, shapes {tuple(a2.shape)} {tuple(b2.shape)}"
                  + (" [APB200_DIAG_LIBRARY_GEMM]" if _DIAG_LIBRARY_GEMM else ""))
        A = a2.t() if a_mn else a2
        B = b2 if b_mn else b2.t()
        if out_dtype == torch.float32 and A.dtype != torch.float32:
            return torch.matmul(A.float(), B.float())
        return torch.matmul(A, B).to(out_dtype)
    c = torch.empty((M, N), dtype=out_dtype if out_dtype in (torch.bfloat16, torch.float32) else torch.float32, device=a2.device)
    _C.gemm(a2, b2, c, a_mn, b_mn, status_buffer(a2.device))
    _count()
    return c if c.dtype == out_dtype else c.to(out_dtype)


def _gemm(a, b, trans_a, trans_b, out_dtype):
    a2, b2 = _as2d(a), _as2d(b)
    # op(a): stored [M,K] if not trans_a else [K,M]; op(b): stored [K,N] if not trans_b else [N,K]
    return gemm_raw(a2, b2, bool(trans_a), not trans_b, out_dtype)


def _mm_nd(a, b, trans_b, out_dtype):
    lead = a.shape[:-1]
    out = gemm_raw(_as2d(a), _as2d(b), False, not trans_b, out_dtype)
    return out.view(*lead, out.shape[-1])


def _mm_wgrad(a, b, out_dtype):
    return gemm_raw(_as2d(a), _as2d(b), True, True, out_dtype)


def _scaled_mm(a, b, scale_a, scale_b, trans_b, out_dtype):
    """fp8 operands with tensor-wise or row-wise scales: the library's fp8 GEMM (cuBLASLt through ``torch._scaled_mm``),
    counted as a library call - this framework has no fp8 tensor-core kernel of its own."""
    _fallback("scaled_mm", f"fp8 GEMM {tuple(a.shape)} x {tuple(b.shape)}")
    lead = a.shape[:-1]
    a2 = a.reshape(-1, a.shape[-1])
    if a2.stride(-1) != 1:
        a2 = a2.contiguous()
    bk = b.t() if trans_b else b  # [K, N]; the library wants it column-major
    if bk.stride(0) != 1:
        bk = bk.t().contiguous().t()
    n = bk.shape[1]
    sa = scale_a.float().reshape(-1, 1) if scale_a.numel() > 1 else scale_a.float().reshape(())
    sb = scale_b.float().reshape(1, -1) if scale_b.numel() > 1 else scale_b.float().reshape(())
    if (sa.ndim == 0) != (sb.ndim == 0):  # the library takes both scales tensor-wise or both row-wise
        sa = sa.expand(a2.shape[0], 1).contiguous() if sa.ndim == 0 else sa
        sb = sb.expand(1, n).contiguous() if sb.ndim == 0 else sb
    sa = sa.contiguous() if sa.ndim else sa
    sb = sb.contiguous() if sb.ndim else sb
    want = out_dtype if out_dtype in (torch.bfloat16, torch.float16, torch.float32) else torch.bfloat16
    try:
        out = torch._scaled_mm(a2, bk, scale_a=sa, scale_b=sb, out_dtype=want)
    except RuntimeError:
        if want == torch.bfloat16:
            raise
        out = torch._scaled_mm(a2, bk, scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)  # row-wise scales: bf16 results only
    return out.view(*lead, n).to(out_dtype)


def _grouped_ok(*ts):
    return all(t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0 for t in ts)


def _grouped_mm(a, b, trans_b, out_dtype):
    """[E,M,K] x ([E,N,K] if trans_b else [E,K,N]) -> [E,M,N]: every expert in one launch of the grouped tcgen05 GEMM."""
    n = b.shape[1] if trans_b else b.shape[2]
    if not _grouped_ok(a, b) or n % 8 or out_dtype not in (torch.bfloat16, torch.float32):
        from .moe_ops import _grouped_mm as ref

        _fallback("grouped_gemm", f"dtypes {a.dtype}/{b.dtype}, shapes {tuple(a.shape)} {tuple(b.shape)}")
        return ref(a, b, trans_b, out_dtype)
    c = torch.empty((a.shape[0], a.shape[1], n), dtype=out_dtype, device=a.device)
    _C.gemm_grouped(a.contiguous(), b.contiguous(), c, False, not trans_b, status_buffer(a.device))
    _count()
    return c


def _grouped_mm_wgrad(a, b, out_dtype):
    """sum over rows of a[E,M,Ka]^T b[E,M,Nb] -> [E,Ka,Nb] (both operands read as stored)."""
    if not _grouped_ok(a, b) or out_dtype not in (torch.bfloat16, torch.float32):
        from .moe_ops import _grouped_mm_wgrad as ref

        _fallback("grouped_gemm", f"wgrad dtypes {a.dtype}/{b.dtype}, shapes {tuple(a.shape)} {tuple(b.shape)}")
        return ref(a, b, out_dtype)
    c = torch.empty((a.shape[0], a.shape[2], b.shape[2]), dtype=out_dtype, device=a.device)
    _C.gemm_grouped(a.contiguous(), b.contiguous(), c, True, True, status_buffer(a.device))
    _count()
    return c


# ----------------------------------------------------------------------------------- mixture-of-experts dispatch
_MOE_KERNELS = os.environ.get("APB200_MOE_KERNELS", "1") != "0"


def _moe_ok(*ts) -> bool:
    return _MOE_KERNELS and all(t.is_cuda for t in ts)


def _moe_slots(gate_idx, num_experts, capacity, num_blocks):
    from . import moe_ops

    T, k = gate_idx.shape
    if not (_moe_ok(gate_idx) and gate_idx.dtype == torch.long and T % num_blocks == 0 and T > 0
            and num_experts <= _C.moe_slots_max_experts(T // num_blocks * k) and num_experts * capacity < 2**31):
        _fallback("moe_index", f"moe_slots {tuple(gate_idx.shape)} E={num_experts}")
        return moe_ops._moe_slots(gate_idx, num_experts, capacity, num_blocks)
    slot = torch.empty_like(gate_idx, memory_format=torch.contiguous_format)
    _C.moe_slots(gate_idx.contiguous(), slot, num_experts, capacity, num_blocks)
    _count()
    return slot


def _moe_scatter(src, slot, w, num_experts, capacity, num_blocks):
    from . import moe_ops

    if not (_moe_ok(src, slot, w) and src.dtype in (torch.bfloat16, torch.float32) and src.dim() == 2 and src.shape[0] % num_blocks == 0
            and src.shape[0] > 0):
        _fallback("moe_index", f"moe_scatter {tuple(src.shape)} {src.dtype}")
        return moe_ops._moe_scatter(src, slot, w, num_experts, capacity, num_blocks)
    buf = torch.zeros((num_experts, num_blocks, capacity, src.shape[1]), dtype=src.dtype, device=src.device)
    # the gate weight is applied in the operand's precision (as the reference formula does), then widened for the kernel
    _C.moe_scatter(src.contiguous(), slot.contiguous(), w.to(src.dtype).float().contiguous(), buf, num_experts, capacity, num_blocks)
    _count()
    return buf


def _moe_gather(buf, slot, w):
    from . import moe_ops

    if not (_moe_ok(buf, slot, w) and buf.dtype in (torch.bfloat16, torch.float32) and buf.dim() == 4 and slot.shape[0] % buf.shape[1] == 0
            and slot.shape[0] > 0):
        _fallback("moe_index", f"moe_gather {tuple(buf.shape)} {buf.dtype}")
        return moe_ops._moe_gather(buf, slot, w)
    out = torch.empty((slot.shape[0], buf.shape[3]), dtype=buf.dtype, device=buf.device)
    _C.moe_gather(buf.contiguous(), slot.contiguous(), w.to(buf.dtype).float().contiguous(), out)
    _count()
    return out


def _moe_gate_grad(buf, slot, g):
    from . import moe_ops

    if not (_moe_ok(buf, slot, g) and buf.dtype in (torch.bfloat16, torch.float32) and buf.dim() == 4 and g.dtype == buf.dtype
            and slot.shape[0] % buf.shape[1] == 0 and slot.shape[0] > 0):
        _fallback("moe_index", f"moe_gate_grad {tuple(buf.shape)} {buf.dtype}")
        return moe_ops._moe_gate_grad(buf, slot, g)
    dw = torch.empty(slot.shape, dtype=torch.float32, device=buf.device)
    _C.moe_gate_grad(buf.contiguous(), slot.contiguous(), g.contiguous(), dw)
    _count()
    return dw


# ----------------------------------------------------------------------------------- pointwise etc.
def _dtype_cast(x, dtype):
    if x.dtype == dtype:
        return x
    from . import shadow

    hit = shadow.lookup(x, dtype)  # the optimizer already wrote this parameter in ``dtype``
    if hit is not None:
        return hit
    pair = {x.dtype, dtype}
    if pair == {torch.float32, torch.bfloat16} and x.is_contiguous() and x.data_ptr() % 16 == 0:
        out = torch.empty_like(x, dtype=dtype)
        _C.cast(x, out)
        _count()
        return out
    _fallback("cast", f"{x.dtype} -> {dtype}, contiguous={x.is_contiguous()}")
    return x.to(dtype)


def _rms_norm(x, w, eps):
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _C.rms_norm_fwd(x, w.to(x.dtype).contiguous(), y, rstd, eps)
    _count()
    return y, rstd


def _rms_norm_bwd(dy, x, w, rstd):
    dy, x = dy.contiguous(), x.contiguous()
    dx = torch.empty_like(x)
    dw = torch.empty_like(w, dtype=x.dtype)
    _C.rms_norm_bwd(dy, x, w.to(x.dtype).contiguous(), rstd.contiguous(), dx, dw, _scratch_f32(x.device, x.shape[-1]))
    _count(3)
    return dx, dw.to(w.dtype)


def _rope(x, cos, sin, conj):
    x = x.contiguous()
    y = torch.empty_like(x)
    _C.rope(x, cos.float().contiguous(), sin.float().contiguous(), y, conj)
    _count()
    return y


def _swiglu(a, b):
    a, b = a.contiguous(), b.contiguous()
    y = torch.empty_like(a)
    _C.swiglu_fwd(a, b, y)
    _count()
    return y


def _swiglu_bwd(dy, a, b):
    dy, a, b = dy.contiguous(), a.contiguous(), b.contiguous()
    da, db = torch.empty_like(a), torch.empty_like(b)
    _C.swiglu_bwd(dy, a, b, da, db)
    _count()
    return da, db


def _cross_entropy(logits, labels):
    logits = logits.contiguous()
    shape = logits.shape[:-1]
    loss = torch.empty(shape, dtype=torch.float32, device=logits.device)
    lse = torch.empty(shape, dtype=torch.float32, device=logits.device)
    _C.xent_fwd(logits, labels.contiguous(), loss, lse)
    _count()
    return loss, lse


def _cross_entropy_bwd(dloss, logits, labels, lse):
    logits = logits.contiguous()
    out = torch.empty_like(logits)
    _C.xent_bwd(dloss.float().contiguous(), logits, labels.contiguous(), lse.contiguous(), out)
    _count()
    return out


def _embedding(weight, ids):
    if weight.dtype not in (torch.bfloat16, torch.float32) or (weight.shape[1] * weight.element_size()) % 16 or ids.dtype != torch.long:
        _fallback("embedding", f"table {weight.dtype} {tuple(weight.shape)}, ids {ids.dtype}")
        return torch.nn.functional.embedding(ids, weight)
    out = torch.empty((*ids.shape, weight.shape[1]), dtype=weight.dtype, device=weight.device)
    _C.embedding_fwd(weight.contiguous(), ids.contiguous(), out)
    _count()
    return out


def _embedding_bwd(dy, ids, num_rows):
    dy = dy.contiguous()
    out = torch.zeros(num_rows, dy.shape[-1], dtype=torch.float32, device=dy.device)
    _C.embedding_bwd(dy, ids.contiguous(), out)
    _count()
    return out.to(dy.dtype)


# ----------------------------------------------------------------------------------- attention (library)
ATTENTION_BACKEND = os.environ.get("APB200_ATTENTION", "cudnn")  # "cudnn" | "flash"
# forward kernel: "library" (the backend above) or "own" (ops/csrc/attention_fwd.cu where its shapes apply: bf16,
# head dim 128, query length a multiple of 256, key length a multiple of 128; other shapes use the library)
ATTENTION_FORWARD = os.environ.get("APB200_ATTENTION_FWD", "library")
_cudnn_lse_ndim = [0]  # rank of the log-sum-exp tensor the cuDNN calls exchange (0 = not seen yet)


def _expand_kv(t, rep):
    if rep == 1:
        return t
    b, s, h, d = t.shape
    return t.unsqueeze(3).expand(b, s, h, rep, d).reshape(b, s, h * rep, d)


def attention_forward_own(q, k, v, causal, scale):
    """(out [B,S,H,D] bf16, lse [B,H,S] fp32) from this package's tcgen05 kernel, or None if it does not cover the shape."""
    if q.dtype != torch.bfloat16 or q.shape[-1] != 128:
        return None
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
    if not _C.attention_fwd(q, k, v, out, lse, bool(causal), float(scale), status_buffer(q.device)):
        return None
    _count()
    return out, lse


def _attention(q, k, v, causal, scale):
    if ATTENTION_FORWARD == "own":
        res = attention_forward_own(q, k, v, causal, scale)
        if res is not None:
            return res
    _fallback("attention", f"forward on the {ATTENTION_BACKEND} library kernel")
    rep = q.shape[2] // k.shape[2]
    if ATTENTION_BACKEND == "cudnn":
        rep = 1  # cuDNN takes grouped-query heads natively
    qt = q.transpose(1, 2)
    kt = _expand_kv(k, rep).transpose(1, 2)
    vt = _expand_kv(v, rep).transpose(1, 2)
    if ATTENTION_BACKEND == "cudnn":
        out, lse, *_ = torch.ops.aten._scaled_dot_product_cudnn_attention(qt, kt, vt, None, True, 0.0, causal, False, scale=scale)
        _cudnn_lse_ndim[0] = lse.ndim
        lse = lse.reshape(q.shape[0], q.shape[2], q.shape[1])
    else:
        out, lse, *_ = torch.ops.aten._scaled_dot_product_flash_attention(qt, kt, vt, 0.0, causal, False, scale=scale)
    return out.transpose(1, 2).contiguous(), lse


def _attention_bwd(dout, q, k, v, out, lse, causal, scale):
    _fallback("attention_bwd", f"backward on the {ATTENTION_BACKEND} library kernel")
    rep = q.shape[2] // k.shape[2]
    if ATTENTION_BACKEND == "cudnn":
        rep = 1
    b, s, h, d = q.shape
    sk = k.shape[1]
    qt = q.transpose(1, 2)
    kt = _expand_kv(k, rep).transpose(1, 2)
    vt = _expand_kv(v, rep).transpose(1, 2)
    seed = torch.zeros((), dtype=torch.long, device=q.device)
    if ATTENTION_BACKEND == "cudnn":
        if _cudnn_lse_ndim[0] == 0:  # forward ran elsewhere: ask a tiny cuDNN forward which rank it uses
            tq = torch.zeros(1, 1, 128, d, dtype=q.dtype, device=q.device)
            _cudnn_lse_ndim[0] = torch.ops.aten._scaled_dot_product_cudnn_attention(tq, tq, tq, None, True, 0.0, causal, False, scale=scale)[1].ndim
        lse_c = lse.unsqueeze(-1) if _cudnn_lse_ndim[0] == 4 else lse
        dq, dk, dv = torch.ops.aten._scaled_dot_product_cudnn_attention_backward(
            dout.transpose(1, 2), qt, kt, vt, out.transpose(1, 2), lse_c, seed, seed, None, None, None, s, sk, 0.0, causal,
            scale=scale,
        )
    else:
        dq, dk, dv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            dout.transpose(1, 2), qt, kt, vt, out.transpose(1, 2), lse, None, None, s, sk, 0.0, causal, seed, seed, scale=scale
        )
    dq = dq.transpose(1, 2).contiguous()
    dk = dk.transpose(1, 2)
    dv = dv.transpose(1, 2)
    if rep > 1:
        dk = dk.reshape(b, sk, k.shape[2], rep, d).sum(3)
        dv = dv.reshape(b, sk, k.shape[2], rep, d).sum(3)
    return dq, dk.contiguous(), dv.contiguous()


def _register() -> None:
    R = L.register_cuda_impl
    R("gemm", _gemm)
    R("mm_nd", _mm_nd)
    R("scaled_mm", _scaled_mm)
    R("mm_wgrad", _mm_wgrad)
    R("grouped_mm", _grouped_mm)
    R("moe_slots", _moe_slots)
    R("moe_scatter", _moe_scatter)
    R("moe_gather", _moe_gather)
    R("moe_gate_grad", _moe_gate_grad)
    R("grouped_mm_wgrad", _grouped_mm_wgrad)
    R("dtype_cast", _dtype_cast)
    R("rms_norm", _rms_norm)
    R("rms_norm_bwd", _rms_norm_bwd)
    R("rope", _rope)
    R("swiglu", _swiglu)
    R("swiglu_bwd", _swiglu_bwd)
    R("cross_entropy", _cross_entropy)
    R("cross_entropy_bwd", _cross_entropy_bwd)
    R("embedding", _embedding)
    R("embedding_bwd", _embedding_bwd)
    R("attention", _attention)
    R("attention_bwd", _attention_bwd)
