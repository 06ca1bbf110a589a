"""Mixture-of-experts operators that the planner can see and shard.

With these ops a routed-expert block is ordinary graph nodes – slot assignment, scatter into
per-expert buffers, grouped expert GEMMs, weighted gather back – instead of one opaque
``local_map`` region, so the ILP itself decides between expert parallelism (the buffer moves from
token-sharded to expert-sharded with one all-to-all), gathering the expert weights, or splitting
the expert hidden dim.

Dispatch is capacity based and *block local*: the ``T`` tokens are cut into ``num_blocks``
contiguous blocks and every (block, expert) pair owns ``capacity`` rows of the buffer
``[E, num_blocks, capacity, d]``.  The result therefore does not depend on how the token dim is
sharded (any shard count that divides ``num_blocks`` computes the same thing), every shape is
static, and a sharded expert partition is a plain ``Shard`` of the expert dim.  The reference's
experimental operator set (examples/native_ds3/moe_ops.py:27-683, moe_placements.py:14-811)
keeps variable-size expert partitions and needs a new ``PartitionedShard`` placement plus aligned /
unaligned all-to-all conversions for them; fixed per-block capacity makes that placement
unnecessary here.

    moe_slots(gate_idx [T,k], E, C, nb)            -> slot [T,k]   (row of the block's [E*C] buffer, E*C = dropped)
    moe_scatter(src [T,d], slot, w [T,k], E, C, nb) -> buf [E,nb,C,d]   buf[slot[t,j]] = w[t,j] * src[t]
    moe_gather(buf [E,nb,C,d], slot, w [T,k])       -> out [T,d]        out[t] = sum_j w[t,j] * buf[slot[t,j]]
    moe_gate_grad(buf, slot, g [T,d])               -> [T,k]            <buf[slot[t,j]], g[t]>
    grouped_mm(a [E,M,K], b [E,K,N] | [E,N,K], trans_b, dtype) -> [E,M,N]   one tcgen05 launch on CUDA
    grouped_mm_wgrad(a [E,M,Ka], b [E,M,Nb], dtype)             -> [E,Ka,Nb]
"""
from __future__ import annotations

import torch

from .library import _ag, _make_cuda_entry, lib, ops, reference_impls

lib.define("moe_slots(Tensor gate_idx, int num_experts, int capacity, int num_blocks) -> Tensor")
lib.define("moe_scatter(Tensor src, Tensor slot, Tensor w, int num_experts, int capacity, int num_blocks) -> Tensor")
lib.define("moe_gather(Tensor buf, Tensor slot, Tensor w) -> Tensor")
lib.define("moe_gate_grad(Tensor buf, Tensor slot, Tensor g) -> Tensor")
lib.define("grouped_mm(Tensor a, Tensor b, bool trans_b, ScalarType out_dtype) -> Tensor")
lib.define("grouped_mm_wgrad(Tensor a, Tensor b, ScalarType out_dtype) -> Tensor")


# ------------------------------------------------------------------------------------ references
def _moe_slots(gate_idx, num_experts, capacity, num_blocks):
    T, k = gate_idx.shape
    tb = T // num_blocks
    e = gate_idx.reshape(num_blocks, tb * k)                                  # assignments of each block, token-major
    order = torch.argsort(e, dim=1, stable=True)
    sorted_e = torch.gather(e, 1, order)
    counts = torch.zeros(num_blocks, num_experts, dtype=torch.long, device=e.device).scatter_add(1, e, torch.ones_like(e))
    starts = torch.cumsum(counts, 1) - counts
    pos_sorted = torch.arange(tb * k, device=e.device).unsqueeze(0) - torch.gather(starts, 1, sorted_e)
    pos = torch.empty_like(pos_sorted).scatter(1, order, pos_sorted)          # arrival rank inside the expert
    slot = torch.where(pos < capacity, e * capacity + pos, torch.full_like(pos, num_experts * capacity))
    return slot.reshape(T, k)


def _rows(slot, num_blocks, rows_per_block):
    """Row of the flattened [nb * (E*C + 1)] buffer (one spare row per block swallows dropped slots)."""
    T, k = slot.shape
    blk = (torch.arange(T, device=slot.device) // (T // num_blocks)).unsqueeze(1)
    return (blk * (rows_per_block + 1) + slot).reshape(-1)


def _moe_scatter(src, slot, w, num_experts, capacity, num_blocks):
    T, d = src.shape
    k = slot.shape[1]
    ec = num_experts * capacity
    rows = _rows(slot, num_blocks, ec)
    vals = (src.unsqueeze(1) * w.unsqueeze(2).to(src.dtype)).reshape(T * k, d)
    flat = src.new_zeros(num_blocks * (ec + 1), d).index_copy(0, rows, vals)
    buf = flat.view(num_blocks, ec + 1, d)[:, :ec]                             # [nb, E*C, d]
    return buf.reshape(num_blocks, num_experts, capacity, d).permute(1, 0, 2, 3).contiguous()


def _buf_rows(buf):
    E, nb, C, d = buf.shape
    flat = buf.permute(1, 0, 2, 3).reshape(nb, E * C, d)
    return torch.cat([flat, flat.new_zeros(nb, 1, d)], 1).reshape(nb * (E * C + 1), d), E * C


def _moe_gather(buf, slot, w):
    T, k = slot.shape
    flat, ec = _buf_rows(buf)
    picked = flat[_rows(slot, buf.shape[1], ec)].view(T, k, -1)
    return (picked * w.unsqueeze(2).to(buf.dtype)).sum(1)


def _moe_gate_grad(buf, slot, g):
    T, k = slot.shape
    flat, ec = _buf_rows(buf)
    picked = flat[_rows(slot, buf.shape[1], ec)].view(T, k, -1)
    return (picked.float() * g.unsqueeze(1).float()).sum(-1)


def _grouped_mm(a, b, trans_b, out_dtype):
    bb = b.transpose(1, 2) if trans_b else b
    if out_dtype == torch.float32 and a.dtype != torch.float32:
        return torch.bmm(a.float(), bb.float())
    return torch.bmm(a, bb).to(out_dtype)


def _grouped_mm_wgrad(a, b, out_dtype):
    if out_dtype == torch.float32 and a.dtype != torch.float32:
        return torch.bmm(a.float().transpose(1, 2), b.float())
    return torch.bmm(a.transpose(1, 2), b).to(out_dtype)


_REFS = {
    "moe_slots": _moe_slots,
    "moe_scatter": _moe_scatter,
    "moe_gather": _moe_gather,
    "moe_gate_grad": _moe_gate_grad,
    "grouped_mm": _grouped_mm,
    "grouped_mm_wgrad": _grouped_mm_wgrad,
}
_META = {
    "moe_slots": lambda gi, E, C, nb: gi.new_empty(gi.shape),
    "moe_scatter": lambda src, slot, w, E, C, nb: src.new_empty((E, nb, C, src.shape[1])),
    "moe_gather": lambda buf, slot, w: buf.new_empty((slot.shape[0], buf.shape[3])),
    "moe_gate_grad": lambda buf, slot, g: buf.new_empty(slot.shape, dtype=torch.float32),
    "grouped_mm": lambda a, b, tb, dt: a.new_empty((a.shape[0], a.shape[1], b.shape[1] if tb else b.shape[2]), dtype=dt),
    "grouped_mm_wgrad": lambda a, b, dt: a.new_empty((a.shape[0], a.shape[2], b.shape[2]), dtype=dt),
}
for _name, _fn in _REFS.items():
    lib.impl(_name, _fn, "CPU")
    lib.impl(_name, _META[_name], "Meta")
    lib.impl(_name, _make_cuda_entry(_name), "CUDA")
    reference_impls[_name] = _fn
# On a GPU every operator above resolves to a kernel wrapper of ``ops/cuda_impl.py`` (``csrc/moe_kernels.cu`` for the four index
# operators, the grouped tcgen05 GEMM for the products); the formulas in this file are their CPU semantics and the GPU tests' oracle.


# ------------------------------------------------------------------------------------ autograd
def _scatter_setup(ctx, inputs, output):
    src, slot, w, *_ = inputs
    ctx.save_for_backward(src, slot, w)


def _scatter_bwd(ctx, dbuf):
    src, slot, w = ctx.saved_tensors
    dsrc = ops.moe_gather(dbuf, slot, w)
    dw = ops.moe_gate_grad(dbuf, slot, src).to(w.dtype)
    return dsrc, None, dw, None, None, None


def _gather_setup(ctx, inputs, output):
    buf, slot, w = inputs
    ctx.save_for_backward(buf, slot, w)
    ctx.dims = (buf.shape[0], buf.shape[2], buf.shape[1])


def _gather_bwd(ctx, dout):
    buf, slot, w = ctx.saved_tensors
    E, C, nb = ctx.dims
    dbuf = ops.moe_scatter(dout, slot, w, E, C, nb)
    dw = ops.moe_gate_grad(buf, slot, dout).to(w.dtype)
    return dbuf, None, dw


def _gmm_setup(ctx, inputs, output):
    a, b, tb, _ = inputs
    ctx.save_for_backward(a, b)
    ctx.tb = tb


def _gmm_bwd(ctx, dc):
    a, b = ctx.saved_tensors
    da = ops.grouped_mm(dc, b, not ctx.tb, a.dtype)
    db = ops.grouped_mm_wgrad(dc, a, b.dtype) if ctx.tb else ops.grouped_mm_wgrad(a, dc, b.dtype)
    return da, db, None, None


_ag("moe_scatter", _scatter_bwd, _scatter_setup)
_ag("moe_gather", _gather_bwd, _gather_setup)
_ag("grouped_mm", _gmm_bwd, _gmm_setup)


# ------------------------------------------------------------------------------------ Python API
def moe_slots(gate_idx, num_experts: int, capacity: int, num_blocks: int):
    return ops.moe_slots(gate_idx, num_experts, capacity, num_blocks)


def moe_dispatch(x, slot, num_experts: int, capacity: int, num_blocks: int):
    """Tokens into per-(expert, block) buffers: ``[T, d] -> [E, num_blocks, capacity, d]``."""
    return ops.moe_scatter(x, slot, x.new_ones(slot.shape), num_experts, capacity, num_blocks)


def moe_combine(y, slot, gate_w):
    """Weighted sum of each token's expert outputs: ``[E, num_blocks, capacity, d] -> [T, d]``."""
    return ops.moe_gather(y, slot, gate_w)


def grouped_mm(a, b, trans_b: bool = False, out_dtype=None):
    return ops.grouped_mm(a, b, trans_b, out_dtype or a.dtype)
