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
        torch.cuda.synchronize()
        dist.barrier(self.pg)
        self.epoch = 0
        self.num_ctas = num_ctas
        self.stream = torch.cuda.Stream(device=self.device)
        self.status = cuda_impl.status_buffer(self.device)
        self._pending: dict[int, torch.cuda.Event] = {}
        self.bytes_moved = 0

    # ------------------------------------------------------------------ synchronous forms
    def _launch(self, mode, src, dst, outer, inner_bytes, elem_kind=0, scale=1.0):
        from ..ops import cuda_impl

        self.epoch += 1
        self._C.symm_collective(mode, self.peer_ptrs, self.rank, self.epoch, src, dst, outer, inner_bytes, elem_kind, scale,
                                self.capacity, self.status, self.num_ctas)
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
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)


_groups: dict[str, SymmGroup] = {}


def enable_for_group(group, workspace_bytes: int = 1 << 30, num_ctas: int = 32) -> SymmGroup:
    pg = group if not isinstance(group, str) else dist.distributed_c10d._resolve_process_group(group)
    name = pg.group_name
    if name not in _groups:
        _groups[name] = SymmGroup(pg, workspace_bytes, num_ctas)
        comm_ops._symm_backends[name] = _groups[name]
    return _groups[name]


def enable_for_mesh(mesh, workspace_bytes: int = 1 << 30, num_ctas: int = 32) -> list[SymmGroup]:
    return [enable_for_group(mesh.get_group(i), workspace_bytes, num_ctas) for i in range(mesh.ndim) if mesh.shape[i] > 1]


def disable_all() -> None:
    for name in list(_groups):
        comm_ops._symm_backends.pop(name, None)
        _groups.pop(name, None)
