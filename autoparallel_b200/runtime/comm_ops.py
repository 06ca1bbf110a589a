"""Collective operators that the lowered (per-rank) graph contains.

The planner's lowering emits these – one node per collective, synchronous in graph semantics –
instead of c10d functional collectives, so the scheduler and the fusion passes have a single
vocabulary to pattern-match (all-gather → GEMM, GEMM → reduce-scatter, ...), and so the same
graph runs on three back-ends:

* ``nccl`` / ``gloo`` / ``fake`` process groups through c10d functional collectives (the
  NCCL-only baseline plan, CPU tests, planning on fake ranks),
* this framework's symmetric-memory kernels (``runtime/symm.py``) when a group has been enabled
  for them – P2P loads over NVLink inside the kernel, no NCCL on the path.

Every op takes the tensor dim it acts on, so gathers / scatters on inner dims need no
``chunk + cat`` round trip through HBM in the graph.  ``group`` is a c10d group name
(``mesh.get_group(i).group_name``).  Reference: the reference lowers through DTensor's
``redistribute_local_tensor`` to ``_c10d_functional`` ops (autoparallel/shardings/
ordered_sharding.py:70-102) and wraps them for users in autoparallel/collectives.py:89-229.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.distributed._functional_collectives as funcol

NS = "apb200_comm"
lib = torch.library.Library(NS, "DEF")  # noqa: TOR901

lib.define("all_gather(Tensor x, int dim, str group, int group_size) -> Tensor")
lib.define("reduce_scatter(Tensor x, int dim, str group, int group_size) -> Tensor")
lib.define("all_reduce(Tensor x, str group, int group_size) -> Tensor")
lib.define("all_to_all(Tensor x, int split_dim, int concat_dim, str group, int group_size) -> Tensor")
lib.define("local_chunk(Tensor x, int dim, str group, int group_size) -> Tensor")

#: group name -> symmetric-memory communicator (set by runtime.symm.enable_for_group)
_symm_backends: dict[str, object] = {}
#: group name -> copy-engine communicator (set by runtime.dma.enable_for_mesh): gathers of tensors that live in the
#: peer arena and fp32 reduce-scatters on the leading dim move with the copy engines and take no SM
_dma_backends: dict[str, object] = {}
#: False = stand-alone collectives stay on NCCL even where a communicator exists (fused nodes still use it)
_symm_standalone = True


#: group name -> name of a second process group over the same ranks that carries the reductions, so a
#: latency-critical parameter gather never queues behind a bulk gradient reduce-scatter on one NCCL stream
_reduction_group: dict[str, str] = {}


def use_separate_reduction_groups(mesh, pg_options=None) -> None:
    """Create (collectively, on every rank) a second process group per mesh dim for reduce-scatter /
    all-reduce.  Both groups issue in the same program order on every rank; the GEMM kernels never
    wait on a peer, so the two NCCL streams cannot starve each other."""
    for i in range(mesh.ndim):
        if mesh.shape[i] <= 1:
            continue
        # every rank creates every subgroup of this mesh dim (new_group is collective over the world)
        pg_ranks = mesh.mesh.movedim(i, -1).reshape(-1, mesh.shape[i]).tolist()
        mine = mesh.get_group(i)
        my_ranks = dist.get_process_group_ranks(mine)
        for ranks in pg_ranks:
            g = dist.new_group(ranks, pg_options=pg_options)
            if sorted(ranks) == sorted(my_ranks):
                _reduction_group[mine.group_name] = g.group_name


def _red_group(group: str) -> str:
    return _reduction_group.get(group, group)


def _standalone_backend(group):
    return _symm_backends.get(group) if _symm_standalone else None


def _wait(t):
    return funcol.wait_tensor(t) if hasattr(funcol, "wait_tensor") else t


def _rank_in_group(group: str) -> int:
    pg = dist.distributed_c10d._resolve_process_group(group)
    return dist.get_rank(pg)


def _all_gather(x, dim, group, n):
    if x.dtype.is_floating_point and x.dtype.itemsize == 1:
        # float8: data movement only, and not every transport knows the dtype
        return _all_gather(x.view(torch.uint8), dim, group, n).view(x.dtype)
    dma = _dma_backends.get(group)
    if dma is not None and dma.can_gather(x, dim):
        return dma.all_gather(x, dim)
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.all_gather(x, dim)
    x = x.contiguous()
    out = torch.ops._c10d_functional.all_gather_into_tensor(x, n, group)
    out = torch.ops._c10d_functional.wait_tensor(out)
    if dim == 0:
        return out
    # [n*d0, ...] -> [n, d0, ...] -> move n next to ``dim`` -> merge
    out = out.view(n, *x.shape).movedim(0, dim)
    shape = list(x.shape)
    shape[dim] *= n
    return out.reshape(shape)


def _reduce_scatter(x, dim, group, n):
    dma = _dma_backends.get(group)
    if dma is not None and dma.can_reduce(x, dim):
        return dma.reduce_scatter(x, dim)
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.reduce_scatter(x, dim)
    shape = list(x.shape)
    shape[dim] //= n
    if dim != 0:
        x = x.view(*x.shape[:dim], n, shape[dim], *x.shape[dim + 1 :]).movedim(dim, 0)
    flat = x.reshape(-1) if x.is_contiguous() else x.contiguous().view(-1)
    out = torch.ops._c10d_functional.reduce_scatter_tensor(flat, "sum", n, _red_group(group))
    return torch.ops._c10d_functional.wait_tensor(out).view(shape)


def _all_reduce(x, group, n):
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.all_reduce(x)
    out = torch.ops._c10d_functional.all_reduce(x.contiguous(), "sum", _red_group(group))
    return torch.ops._c10d_functional.wait_tensor(out)


def _all_to_all(x, split_dim, concat_dim, group, n):
    """Each rank splits ``x`` into n chunks along ``split_dim``, sends chunk r to rank r, and
    concatenates what it receives along ``concat_dim`` (Shard(concat_dim) -> Shard(split_dim))."""
    if x.dtype.is_floating_point and x.dtype.itemsize == 1:
        return _all_to_all(x.view(torch.uint8), split_dim, concat_dim, group, n).view(x.dtype)
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.all_to_all(x, split_dim, concat_dim)
    chunks = x.chunk(n, dim=split_dim)
    send = torch.stack([c.contiguous() for c in chunks], 0)  # [n, ...chunk]
    flat = send.reshape(n * send.shape[1], *send.shape[2:]) if send.ndim > 1 else send
    rows = flat.shape[0] // n
    out = torch.ops._c10d_functional.all_to_all_single(flat, [rows] * n, [rows] * n, group)
    out = torch.ops._c10d_functional.wait_tensor(out)
    recv = out.view(n, *chunks[0].shape)
    return torch.cat(list(recv.unbind(0)), dim=concat_dim)


def _local_chunk(x, dim, group, n):
    r = _rank_in_group(group)
    size = x.shape[dim] // n
    return x.narrow(dim, r * size, size).contiguous()


for _name, _fn in (
    ("all_gather", _all_gather),
    ("reduce_scatter", _reduce_scatter),
    ("all_reduce", _all_reduce),
    ("all_to_all", _all_to_all),
    ("local_chunk", _local_chunk),
):
    lib.impl(_name, _fn, "CPU")
    lib.impl(_name, _fn, "CUDA")


def _shape_mul(x, dim, n):
    s = list(x.shape)
    s[dim] *= n
    return x.new_empty(s)


def _shape_div(x, dim, n):
    s = list(x.shape)
    s[dim] //= n
    return x.new_empty(s)


lib.impl("all_gather", lambda x, dim, group, n: _shape_mul(x, dim, n), "Meta")
lib.impl("reduce_scatter", lambda x, dim, group, n: _shape_div(x, dim, n), "Meta")
lib.impl("all_reduce", lambda x, group, n: torch.empty_like(x), "Meta")
lib.impl("local_chunk", lambda x, dim, group, n: _shape_div(x, dim, n), "Meta")


def _a2a_meta(x, split_dim, concat_dim, group, n):
    s = list(x.shape)
    s[split_dim] //= n
    s[concat_dim] *= n
    return x.new_empty(s)


lib.impl("all_to_all", _a2a_meta, "Meta")

ops = getattr(torch.ops, NS)


# ---------------------------------------------------------------------------- autograd pairs
def _setup(ctx, inputs, output):
    ctx.args = inputs[1:]


torch.library.register_autograd(
    f"{NS}::all_gather", lambda ctx, g: (ops.reduce_scatter(g, *ctx.args), None, None, None), setup_context=_setup, lib=lib
)
torch.library.register_autograd(
    f"{NS}::reduce_scatter", lambda ctx, g: (ops.all_gather(g, *ctx.args), None, None, None), setup_context=_setup, lib=lib
)
torch.library.register_autograd(
    f"{NS}::all_reduce", lambda ctx, g: (ops.all_reduce(g, *ctx.args), None, None), setup_context=_setup, lib=lib
)
torch.library.register_autograd(
    f"{NS}::all_to_all",
    lambda ctx, g: (ops.all_to_all(g, ctx.args[1], ctx.args[0], ctx.args[2], ctx.args[3]), None, None, None, None),
    setup_context=_setup,
    lib=lib,
)
torch.library.register_autograd(
    f"{NS}::local_chunk", lambda ctx, g: (ops.all_gather(g, *ctx.args), None, None, None), setup_context=_setup, lib=lib
)

COLLECTIVE_OPS = {
    ops.all_gather.default,
    ops.reduce_scatter.default,
    ops.all_reduce.default,
    ops.all_to_all.default,
}


# --------------------------------------------------------------------------------------------------
# Split-phase forms used by the overlap scheduler: ``*_start`` issues the collective on the
# communication stream and returns the (not yet valid) result; ``comm_wait`` makes the compute stream
# wait for it.  Between the two nodes the scheduler places independent compute.
# --------------------------------------------------------------------------------------------------
lib.define("all_gather_start(Tensor x, int dim, str group, int group_size) -> Tensor")
lib.define("reduce_scatter_start(Tensor x, int dim, str group, int group_size) -> Tensor")
lib.define("all_reduce_start(Tensor x, str group, int group_size) -> Tensor")
lib.define("comm_wait(Tensor x) -> Tensor")


#: SM pairs that the GEMM kernels are asked to give up whenever an NCCL collective is issued split-phase
#: (0 = never).  A persistent GEMM holds every SM, so a collective launched beside it would otherwise
#: start only when the compute stream runs dry; needs the GEMM's dynamic tile scheduling.
_yield_pairs = 0


def set_sm_yield(pairs: int) -> None:
    global _yield_pairs
    _yield_pairs = max(0, int(pairs))


def _request_sms(x) -> None:
    if _yield_pairs and x.is_cuda:
        from ..ops import cuda_impl

        cuda_impl.ensure_loaded()
        cuda_impl.extension().gemm_yield_request(_yield_pairs)


#: Host tensors (gloo ranks: the CPU test paths) complete their split-phase collectives at issue.  The schedule - which
#: node is issued where, which wait is deferred - is the same; only the library call is no longer in flight while the
#: graph runs on.  With several gloo collectives in flight next to the graph's own operators, about one run in twenty-five
#: of small multi-model numerics jobs ended in a corrupted heap ("malloc(): unaligned tcache chunk detected"), with
#: identical schedules on all ranks; the same collectives issued and waited from a plain loop never did, and the cause
#: was not found.  Device tensors are stream ordered and unaffected.  ``APB200_HOST_ASYNC=1`` restores in-flight issue.
_HOST_ASYNC = os.environ.get("APB200_HOST_ASYNC", "0") == "1"


def _issued(out):
    if not out.is_cuda and not _HOST_ASYNC:
        return torch.ops._c10d_functional.wait_tensor(out)
    return out


def _ag_start(x, dim, group, n):
    if x.dtype.is_floating_point and x.dtype.itemsize == 1:
        return _all_gather(x, dim, group, n)  # float8 moves as bytes (synchronous form)
    dma = _dma_backends.get(group)
    if dma is not None and dma.can_gather(x, dim):
        return dma.all_gather_start(x, dim)
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.all_gather_start(x, dim)
    if dim != 0:
        return _all_gather(x, dim, group, n)  # inner-dim gathers need a post-permute: keep synchronous
    _request_sms(x)
    return _issued(torch.ops._c10d_functional.all_gather_into_tensor(x.contiguous(), n, group))


def _rs_start(x, dim, group, n):
    dma = _dma_backends.get(group)
    if dma is not None and dma.can_reduce(x, dim):
        return dma.reduce_scatter_start(x, dim)
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.reduce_scatter_start(x, dim)
    if dim != 0:
        return _reduce_scatter(x, dim, group, n)
    shape = list(x.shape)
    shape[0] //= n
    _request_sms(x)
    out = _issued(torch.ops._c10d_functional.reduce_scatter_tensor(x.contiguous().view(-1), "sum", n, _red_group(group)))
    return out.view(shape)


def _ar_start(x, group, n):
    be = _standalone_backend(group)
    if be is not None and x.is_cuda:
        return be.all_reduce_start(x)
    return _issued(torch.ops._c10d_functional.all_reduce(x.contiguous(), "sum", _red_group(group)))


def _comm_wait(x):
    be = _symm_pending.pop(x.data_ptr(), None) if _symm_pending else None
    if be is not None:
        be.wait(x)
        return x
    return torch.ops._c10d_functional.wait_tensor(x)


#: data_ptr -> backend for results of symmetric-memory ``*_start`` calls still in flight
_symm_pending: dict[int, object] = {}

for _name, _fn in (("all_gather_start", _ag_start), ("reduce_scatter_start", _rs_start), ("all_reduce_start", _ar_start),
                   ("comm_wait", _comm_wait)):
    lib.impl(_name, _fn, "CPU")
    lib.impl(_name, _fn, "CUDA")
lib.impl("all_gather_start", lambda x, dim, group, n: _shape_mul(x, dim, n), "Meta")
lib.impl("reduce_scatter_start", lambda x, dim, group, n: _shape_div(x, dim, n), "Meta")
lib.impl("all_reduce_start", lambda x, group, n: torch.empty_like(x), "Meta")
lib.impl("comm_wait", lambda x: torch.empty_like(x), "Meta")

# A pending maximum / minimum (``Partial("max")``: the result of ``amax`` over a sharded dim, say) is completed by an
# all-reduce with that operator.  Kept apart from ``all_reduce`` (sums: gradients, partial products), which has kernels of
# its own and split-phase forms; this one always runs on the process group's library collective.
lib.define("all_reduce_op(Tensor x, str op, str group, int group_size) -> Tensor")


def _all_reduce_op(x, op, group, n):
    out = torch.ops._c10d_functional.all_reduce(x.contiguous(), op, group)
    return torch.ops._c10d_functional.wait_tensor(out)


lib.impl("all_reduce_op", _all_reduce_op, "CPU")
lib.impl("all_reduce_op", _all_reduce_op, "CUDA")
lib.impl("all_reduce_op", lambda x, op, group, n: torch.empty_like(x), "Meta")
COLLECTIVE_OPS.add(ops.all_reduce_op.default)

START_OF = {
    ops.all_gather.default: ops.all_gather_start.default,
    ops.reduce_scatter.default: ops.reduce_scatter_start.default,
    ops.all_reduce.default: ops.all_reduce_start.default,
}
START_OPS = set(START_OF.values())


# --------------------------------------------------------------------------------------------------
# GEMM fused with the neighbouring collective.  One graph node = one kernel per rank when the group
# has a symmetric-memory communicator (runtime/symm.py: communication CTAs + tcgen05 GEMM CTAs in
# the same launch); otherwise the unfused composition below, which is also the CPU semantics.
#   ag_mm  mode 0: y = x @ all_gather(w, 0)^T          (FSDP forward; w [N/n, K])
#          mode 1: y = x @ all_gather(w, 0)            (FSDP backward dgrad; gathered rows = contraction)
#          mode 2: y = all_gather(x, rows) @ w^T       (sequence-parallel activations -> column-parallel weight)
#          mode 3: y = all_gather(x, rows) @ w
#          returns (y, gathered operand); ``dim`` is the gather dim of x (modes 2/3; 0 for modes 0/1)
#   mm_rs  mode 0: reduce_scatter(a @ b^T, rows)   mode 1: reduce_scatter(a @ b, rows)
#          mode 2: reduce_scatter(a^T @ b, rows)       (weight gradient + gradient reduce-scatter)
#          ``dim`` is the scatter dim of the result; every dim before it has extent 1
# --------------------------------------------------------------------------------------------------
lib.define("ag_mm(Tensor x, Tensor w, int mode, int dim, ScalarType out_dtype, str group, int group_size) -> (Tensor, Tensor)")
lib.define("mm_rs(Tensor a, Tensor b, int mode, int dim, ScalarType out_dtype, float scale, str group, int group_size) -> Tensor")

_apb = torch.ops.apb200


def _ag_mm(x, w, mode, dim, out_dtype, group, n):
    be = _symm_backends.get(group)
    if be is not None and x.is_cuda:
        if mode in (0, 1) and be.can_fuse_gather(w) and x.dtype == torch.bfloat16:
            return be.ag_gemm_b(x, w, out_dtype) if mode == 0 else be.ag_gemm_bk(x, w, out_dtype)
        if mode in (2, 3) and x.dtype == torch.bfloat16 and be.can_fuse_gather(x.reshape(-1, x.shape[-1])):
            lead = list(x.shape[:-1])
            y, xf = be.ag_gemm_a(x, w, trans_b=(mode == 2), out_dtype=out_dtype)
            lead[dim] *= n
            return y.view(*lead, y.shape[-1]), xf.view(*lead, x.shape[-1])
    if mode in (0, 1):
        wf = _all_gather(w, 0, group, n)
        return _apb.mm_nd(x, wf, mode == 0, out_dtype), wf
    xf = _all_gather(x, dim, group, n)
    return _apb.mm_nd(xf, w, mode == 2, out_dtype), xf


def _mm_rs(a, b, mode, dim, out_dtype, scale, group, n):
    be = _symm_backends.get(group)
    if be is not None and a.is_cuda and a.dtype == torch.bfloat16 and out_dtype in (torch.float32, torch.bfloat16):
        if mode == 2:
            a2, b2 = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
            if be.can_fuse_rs(a2.shape[1], b2.shape[1]) and a2.shape[1] % 8 == 0 and b2.shape[1] % 8 == 0:
                return be.gemm_rs(a2, b2, True, True, out_dtype, scale)
        else:
            a2 = a.reshape(-1, a.shape[-1])
            N = b.shape[0] if mode == 0 else b.shape[1]
            if be.can_fuse_rs(a2.shape[0], N) and b.shape[1] % 8 == 0 and a2.shape[1] % 8 == 0:
                out = be.gemm_rs(a2, b, False, mode == 1, out_dtype, scale)
                lead = list(a.shape[:-1])
                lead[dim] //= n
                return out.view(*lead, N)
    if mode == 2:
        full = _apb.mm_wgrad(a, b, out_dtype)
    else:
        full = _apb.mm_nd(a, b, mode == 0, out_dtype)
    out = _reduce_scatter(full, dim, group, n)
    return out * scale if scale != 1.0 else out


def _ag_mm_meta(x, w, mode, dim, out_dtype, group, n):
    if mode in (0, 1):
        wf = w.new_empty((w.shape[0] * n, w.shape[1]))
        nn_ = wf.shape[0] if mode == 0 else wf.shape[1]
        return x.new_empty((*x.shape[:-1], nn_), dtype=out_dtype), wf
    lead = list(x.shape[:-1])
    lead[dim] *= n
    nn_ = w.shape[0] if mode == 2 else w.shape[1]
    return x.new_empty((*lead, nn_), dtype=out_dtype), x.new_empty((*lead, x.shape[-1]))


def _mm_rs_meta(a, b, mode, dim, out_dtype, scale, group, n):
    if mode == 2:
        return a.new_empty((a.shape[-1] // n, b.shape[-1]), dtype=out_dtype)
    lead = list(a.shape[:-1])
    lead[dim] //= n
    return a.new_empty((*lead, b.shape[0] if mode == 0 else b.shape[1]), dtype=out_dtype)


# fp8 forms.  The float8 operand and, when it is row-wise, its scale travel together; the product runs on
# ``apb200::scaled_mm``.  Modes as above restricted to the cases float8 training produces:
#   ag_scaled_mm  mode 0: y = x @ all_gather(w, 0)^T (w [N/n, K]; a row-wise scale_w [N/n, 1] is gathered with it)
#                 mode 2: y = all_gather(x, rows) @ w^T     mode 3: y = all_gather(x, rows) @ w
#                         (a row-wise scale_x [..., 1] is gathered with x)
#   scaled_mm_rs  mode 0 / 1: reduce_scatter((a * sa) @ (b * sb)^T | (a * sa) @ (b * sb), rows)
# Reference: autoparallel/graph_passes/async_tp/asynctp_ops.py:948-1026 (gather), :1189-1424 (reduce-scatter).
lib.define("ag_scaled_mm(Tensor x, Tensor w, Tensor scale_x, Tensor scale_w, int mode, int dim, ScalarType out_dtype, "
           "str group, int group_size) -> (Tensor, Tensor)")
lib.define("scaled_mm_rs(Tensor a, Tensor b, Tensor scale_a, Tensor scale_b, int mode, int dim, ScalarType out_dtype, "
           "str group, int group_size) -> Tensor")


def _ag_scaled_mm(x, w, sx, sw, mode, dim, out_dtype, group, n):
    if mode == 0:
        wf = _all_gather(w, 0, group, n)
        swf = _all_gather(sw.contiguous(), 0, group, n) if sw.numel() > 1 else sw
        return _apb.scaled_mm(x, wf, sx, swf, True, out_dtype), wf
    xf = _all_gather(x, dim, group, n)
    sxf = _all_gather(sx.contiguous(), dim, group, n) if sx.numel() > 1 else sx
    return _apb.scaled_mm(xf, w, sxf, sw, mode == 2, out_dtype), xf


def _scaled_mm_rs(a, b, sa, sb, mode, dim, out_dtype, group, n):
    # partial products are summed in fp32 (the reference stacks and sums the partials in the output dtype's accumulator)
    full = _apb.scaled_mm(a, b, sa, sb, mode == 0, torch.float32)
    return _reduce_scatter(full, dim, group, n).to(out_dtype)


def _ag_scaled_mm_meta(x, w, sx, sw, mode, dim, out_dtype, group, n):
    if mode == 0:
        wf = w.new_empty((w.shape[0] * n, w.shape[1]))
        return x.new_empty((*x.shape[:-1], wf.shape[0]), dtype=out_dtype), wf
    lead = list(x.shape[:-1])
    lead[dim] *= n
    return x.new_empty((*lead, w.shape[0] if mode == 2 else w.shape[1]), dtype=out_dtype), x.new_empty((*lead, x.shape[-1]))


def _scaled_mm_rs_meta(a, b, sa, sb, mode, dim, out_dtype, group, n):
    lead = list(a.shape[:-1])
    lead[dim] //= n
    return a.new_empty((*lead, b.shape[0] if mode == 0 else b.shape[1]), dtype=out_dtype)


for _name, _fn in (("ag_scaled_mm", _ag_scaled_mm), ("scaled_mm_rs", _scaled_mm_rs)):
    lib.impl(_name, _fn, "CPU")
    lib.impl(_name, _fn, "CUDA")
lib.impl("ag_scaled_mm", _ag_scaled_mm_meta, "Meta")
lib.impl("scaled_mm_rs", _scaled_mm_rs_meta, "Meta")

for _name, _fn in (("ag_mm", _ag_mm), ("mm_rs", _mm_rs)):
    lib.impl(_name, _fn, "CPU")
    lib.impl(_name, _fn, "CUDA")
lib.impl("ag_mm", _ag_mm_meta, "Meta")
lib.impl("mm_rs", _mm_rs_meta, "Meta")
FUSED_OPS = {ops.ag_mm.default, ops.mm_rs.default}
#: fp8 forms: compositions of a collective and the library's fp8 GEMM (no single-kernel implementation)
SCALED_FUSED_OPS = {ops.ag_scaled_mm.default, ops.scaled_mm_rs.default}
