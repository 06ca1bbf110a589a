"""Symmetric-memory communicator: this framework's own collectives over NVLink peer memory.

``SymmGroup`` owns one workspace per rank – allocated and exchanged through
``torch.distributed._symmetric_memory`` (CUDA VMM handles; the only thing taken from torch here is
the allocation + rendezvous) – and drives the kernels in ``ops/csrc/symm_comm.cu``: every
collective is ONE kernel per rank that signals, pulls over NVLink with plain peer loads and
reduces in fp32; no NCCL on the path.  ``enable_for_mesh`` installs a communicator for every mesh
dim, after which the ``apb200_comm`` graph ops route CUDA tensors here.

Split-phase calls (``*_start`` / ``wait``) run the kernel on a dedicated communication stream so
the overlap scheduler's issue/wait pairs translate to stream events.

Reference counterpart: the symmetric-memory "async-TP" ops
(autoparallel/graph_passes/async_tp/asynctp_ops.py:35-178, 1534-1703), which pipeline P2P copies
from the host; here signalling and data movement both happen inside the kernel.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from . import comm_ops

MODE_AG, MODE_RS, MODE_A2A = 0, 1, 2


class SymmGroup:
    def __init__(self, group, workspace_bytes: int = 1 << 30, num_ctas: int = 32):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import cuda_impl

        cuda_impl.ensure_loaded()
        self._C = cuda_impl.extension()
        self.pg = group if not isinstance(group, str) else dist.distributed_c10d._resolve_process_group(group)
        self.group_name = self.pg.group_name
        self.rank = dist.get_rank(self.pg)
        self.n = dist.get_world_size(self.pg)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.header = int(self._C.symm_header_bytes())
        self.capacity = int(workspace_bytes)
        self.ws = symm_mem.empty(self.header + self.capacity, dtype=torch.uint8, device=self.device)
        self.ws[: self.header].zero_()
        self.hdl = symm_mem.rendezvous(self.ws, self.group_name)
        self.peer_ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        # NVLS (opt-in, APB200_SYMM_NVLS=1): reduce-scatter sums through the workspace's multicast address with
        # ``multimem.ld_reduce`` (added inside NVSwitch) instead of n peer loads.  Off by default: not yet timed on
        # hardware, and a rank that dies while its memory is bound to a multicast object can fault its peers.
        import os

        self.multicast_ptr = int(getattr(self.hdl, "multicast_ptr", 0) or 0) if os.environ.get("APB200_SYMM_NVLS") == "1" else 0
        torch.cuda.synchronize()
        dist.barrier(self.pg)
        self.epoch = 0
        self.arrivals = [0] * 8  # running totals of the header's arrival counters
        self.num_ctas = num_ctas
        self.stream = torch.cuda.Stream(device=self.device)
        self.status = cuda_impl.status_buffer(self.device)
        self._pending: dict[int, torch.cuda.Event] = {}
        self.async_twin: Optional[SymmGroup] = None
        self.bytes_moved = 0

    # ------------------------------------------------------------------ synchronous forms
    def _launch(self, mode, src, dst, outer, inner_bytes, elem_kind=0, scale=1.0):
        from ..ops import cuda_impl

        self.epoch += 1
        self.arrivals[0] += self.num_ctas
        self.arrivals[1] += self.num_ctas
        self._C.symm_collective(mode, self.peer_ptrs, self.rank, self.epoch, src, dst, outer, inner_bytes, elem_kind, scale,
                                self.capacity, self.status, self.num_ctas, self.arrivals[0] & 0xFFFFFFFF,
                                self.arrivals[1] & 0xFFFFFFFF, self.multicast_ptr if mode == MODE_RS else 0)
        cuda_impl._count()

    def _split(self, shape, dim, itemsize):
        outer = math.prod(shape[:dim]) if dim > 0 else 1
        inner = math.prod(shape[dim:]) * itemsize
        return outer, inner

    def all_gather(self, x: torch.Tensor, dim: int = 0) -> torch.Tensor:
        x = x.contiguous()
        shape = list(x.shape)
        outer, inner = self._split(shape, dim, x.element_size())
        shape[dim] *= self.n
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
        if x.numel() * x.element_size() > self.capacity or inner % 16:
            return self._fallback("all_gather", x, dim)
        self._launch(MODE_AG, x, out, outer, inner)
        return out

    def reduce_scatter(self, x: torch.Tensor, dim: int = 0, scale: float = 1.0) -> torch.Tensor:
        x = x.contiguous()
        shape = list(x.shape)
        shape[dim] //= self.n
        outer, inner = self._split(shape, dim, x.element_size())
        if x.dtype not in (torch.float32, torch.bfloat16) or x.numel() * x.element_size() > self.capacity or inner % 16:
            return self._fallback("reduce_scatter", x, dim)
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
        self._launch(MODE_RS, x, out, outer, inner, 0 if x.dtype == torch.float32 else 1, scale)
        return out

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        flat = x.contiguous().view(-1)
        pad = (-flat.numel()) % (self.n * 16)
        if pad:
            flat = torch.nn.functional.pad(flat, (0, pad))
        part = self.reduce_scatter(flat, 0)
        full = self.all_gather(part, 0)
        return full[: x.numel()].view(x.shape)

    def all_to_all(self, x: torch.Tensor, split_dim: int, concat_dim: int) -> torch.Tensor:
        """Shard(concat_dim) -> Shard(split_dim): send chunk r of ``split_dim`` to rank r, concatenate
        what arrives along ``concat_dim``."""
        n = self.n
        # bring to [outer, n, inner] with the split dim leading its block
        xs = x.movedim(split_dim, 0).contiguous()  # [split, ...rest]
        rest = list(xs.shape[1:])
        chunk = xs.shape[0] // n
        inner = chunk * math.prod(rest) * x.element_size()
        if inner % 16 or xs.numel() * x.element_size() > self.capacity:
            return self._fallback("all_to_all", x, split_dim, concat_dim)
        out = torch.empty_like(xs)  # [n(peer), chunk, ...rest]
        self._launch(MODE_A2A, xs, out, 1, inner)
        recv = out.view(n, chunk, *rest).movedim(1, split_dim + 1)  # peer, then original dim order with chunked split dim
        # recv: [peer, d0, ..., chunk@split_dim, ...]; concatenate peers along concat_dim
        pieces = recv.unbind(0)
        return torch.cat(pieces, dim=concat_dim)

    # ------------------------------------------------------------------ GEMM fused with a collective
    FUSE_GATHER_A, FUSE_GATHER_B, FUSE_REDUCE_SCATTER = 1, 2, 3

    def _landed(self):
        if not hasattr(self, "_landed_buf"):
            self._landed_buf = torch.zeros(16, dtype=torch.int32, device=self.device)
            self._landed_total = 0
        return self._landed_buf

    def _fused(self, fuse, a, b, c, a_mn, b_mn, rows_per_shard, shard_src, rows_per_rank, scale):
        from ..ops import cuda_impl

        landed = self._landed()
        self.epoch += 1
        ctas = self.fused_comm_ctas
        # the kernel reports how many GEMM CTAs (or CTA pairs) a launch of this shape runs
        M_full = c.shape[0] * self.n if fuse == self.FUSE_REDUCE_SCATTER else c.shape[0]
        gemm_ctas = int(self._C.gemm_fused_ctas(fuse, M_full, c.shape[1], ctas))
        if fuse == self.FUSE_REDUCE_SCATTER:
            self.arrivals[2] += ctas
            self.arrivals[4] += gemm_ctas
        else:
            # every GEMM CTA carries a gather warp that arrives once per phase and once per shard
            self.arrivals[2] += gemm_ctas
            self.arrivals[3] += gemm_ctas
            self._landed_total += gemm_ctas
        targets = [self.arrivals[2] & 0xFFFFFFFF, self.arrivals[3] & 0xFFFFFFFF, self.arrivals[4] & 0xFFFFFFFF]
        self._C.gemm_fused(fuse, a, b, c, a_mn, b_mn, self.peer_ptrs, self.rank, self.epoch, rows_per_shard, shard_src, landed,
                           self._landed_total & 0xFFFFFFFF, rows_per_rank, scale, self.capacity, targets, ctas, self.status)
        cuda_impl._count()

    @property
    def _num_sms(self):
        return torch.cuda.get_device_properties(self.device).multi_processor_count

    fused_comm_ctas = 2  # GEMM -> reduce-scatter only: CTAs that wait for the peers' "done" and publish "slots free"

    def can_fuse_gather(self, shard: torch.Tensor) -> bool:
        nbytes = shard.numel() * shard.element_size()
        return (shard.dtype == torch.bfloat16 and shard.dim() == 2 and nbytes % 16 == 0 and nbytes <= self.capacity
                and shard.shape[1] % 8 == 0 and shard.data_ptr() % 16 == 0)

    def ag_gemm_b(self, x: torch.Tensor, w_shard: torch.Tensor, out_dtype=torch.bfloat16):
        """y = x @ all_gather(w_shard, 0)^T with x [M, K], w_shard [R, K]; returns (y [M, n*R], w_full)."""
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        w_shard = w_shard.contiguous()
        R, K = w_shard.shape
        w_full = torch.empty(self.n * R, K, dtype=w_shard.dtype, device=x.device)
        y = torch.empty(x2.shape[0], self.n * R, dtype=out_dtype, device=x.device)
        self._fused(self.FUSE_GATHER_B, x2, w_full, y, False, False, R, w_shard, 0, 1.0)
        return y.view(*x.shape[:-1], self.n * R), w_full

    def ag_gemm_bk(self, dy: torch.Tensor, w_shard: torch.Tensor, out_dtype=torch.bfloat16):
        """dx = dy @ all_gather(w_shard, 0) with dy [M, n*R], w_shard [R, K]; the gathered rows are the
        contraction dim.  Returns (dx [M, K], w_full)."""
        d2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        w_shard = w_shard.contiguous()
        R, K = w_shard.shape
        w_full = torch.empty(self.n * R, K, dtype=w_shard.dtype, device=dy.device)
        dx = torch.empty(d2.shape[0], K, dtype=out_dtype, device=dy.device)
        self._fused(self.FUSE_GATHER_B, d2, w_full, dx, False, True, R, w_shard, 0, 1.0)
        return dx.view(*dy.shape[:-1], K), w_full

    def ag_gemm_a(self, x_shard: torch.Tensor, w: torch.Tensor, trans_b: bool = True, out_dtype=torch.bfloat16):
        """y = all_gather(x_shard, 0) @ (w^T if trans_b else w); returns (y [n*R, N], x_full)."""
        xs = x_shard.reshape(-1, x_shard.shape[-1]).contiguous()
        w = w.contiguous()
        R, K = xs.shape
        x_full = torch.empty(self.n * R, K, dtype=xs.dtype, device=xs.device)
        N = w.shape[0] if trans_b else w.shape[1]
        y = torch.empty(self.n * R, N, dtype=out_dtype, device=xs.device)
        self._fused(self.FUSE_GATHER_A, x_full, w, y, False, not trans_b, R, xs, 0, 1.0)
        return y, x_full

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool, out_dtype=torch.float32, scale: float = 1.0):
        """reduce_scatter(opA @ opB, dim 0) in one kernel; returns this rank's [M/n, N] rows."""
        a, b = a.contiguous(), b.contiguous()
        M = a.shape[1] if a_mn else a.shape[0]
        N = b.shape[1] if b_mn else b.shape[0]
        out = torch.empty(M // self.n, N, dtype=out_dtype, device=a.device)
        self._fused(self.FUSE_REDUCE_SCATTER, a, b, out, a_mn, b_mn, 0, out, M // self.n, scale)
        return out

    def can_fuse_rs(self, M: int, N: int) -> bool:
        return M % (self.n * 128) == 0 and N % 8 == 0 and M * N * 4 <= self.capacity  # n fp32 slots of [M/n, N]

    def _fallback(self, kind, x, *dims):
        n, g = self.n, self.group_name
        be = comm_ops._symm_backends.pop(g, None)
        try:
            if kind == "all_gather":
                return comm_ops._all_gather(x, dims[0], g, n)
            if kind == "reduce_scatter":
                return comm_ops._reduce_scatter(x, dims[0], g, n)
            return comm_ops._all_to_all(x, dims[0], dims[1], g, n)
        finally:
            if be is not None:
                comm_ops._symm_backends[g] = be

    # ------------------------------------------------------------------ split-phase forms
    def _async(self, fn, x, *args):
        if self.async_twin is not None:
            # split-phase collectives run on the communication stream with their own workspace and
            # epoch sequence, so they never interleave with main-stream (fused / synchronous) ops
            return getattr(self.async_twin, "_async")(getattr(self.async_twin, fn.__name__), x, *args)
        cur = torch.cuda.current_stream()
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            out = fn(x, *args)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        x.record_stream(self.stream)
        out.record_stream(cur)
        self._pending[out.data_ptr()] = ev
        comm_ops._symm_pending[out.data_ptr()] = self
        return out

    def all_gather_start(self, x, dim):
        return self._async(self.all_gather, x, dim)

    def reduce_scatter_start(self, x, dim):
        return self._async(self.reduce_scatter, x, dim)

    def all_reduce_start(self, x):
        return self._async(self.all_reduce, x)

    def wait(self, out: torch.Tensor) -> None:
        ev = self._pending.pop(out.data_ptr(), None)
        if ev is None and self.async_twin is not None:
            ev = self.async_twin._pending.pop(out.data_ptr(), None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)


_groups: dict[str, SymmGroup] = {}


def enable_for_group(group, workspace_bytes: int = 1 << 30, num_ctas: int = 32) -> SymmGroup:
    pg = group if not isinstance(group, str) else dist.distributed_c10d._resolve_process_group(group)
    name = pg.group_name
    if name not in _groups:
        _groups[name] = SymmGroup(pg, workspace_bytes, num_ctas)
        _groups[name].async_twin = SymmGroup(pg, workspace_bytes, num_ctas)
        comm_ops._symm_backends[name] = _groups[name]
    return _groups[name]


def enable_for_mesh(mesh, workspace_bytes: int = 1 << 30, num_ctas: int = 32) -> list[SymmGroup]:
    return [enable_for_group(mesh.get_group(i), workspace_bytes, num_ctas) for i in range(mesh.ndim) if mesh.shape[i] > 1]


def enabled_for_mesh(mesh) -> bool:
    """True if every mesh dim of extent > 1 has a communicator."""
    try:
        names = [mesh.get_group(i).group_name for i in range(mesh.ndim) if mesh.shape[i] > 1]
    except Exception:
        return False
    return bool(names) and all(n in _groups for n in names)


def route_standalone_collectives(on: bool) -> None:
    """``False``: only the fused GEMM+collective nodes use the symmetric-memory kernels; stand-alone
    collectives (and their split-phase forms) go to NCCL.  ``True`` (default) routes everything here."""
    comm_ops._symm_standalone = bool(on)


def disable_all() -> None:
    for name in list(_groups):
        comm_ops._symm_backends.pop(name, None)
        _groups.pop(name, None)
    comm_ops._symm_standalone = True
