"""Copy-engine collectives: parameter all-gathers and gradient reduce-scatters that take no SM.

During a training step every SM runs a persistent tensor-core kernel, so a collective that is
itself a kernel (NCCL's, or a peer-load kernel of this framework) only becomes resident at kernel
boundaries and then competes with the GEMMs.  The collectives here move their bytes with the GPU's
copy engines instead: plain asynchronous device-to-device copies between this rank's memory and a
peer's mapping of a *symmetric arena* (``torch.distributed._symmetric_memory`` allocation, one
rendezvous for the whole world).

* ``PeerArena`` - the allocation, a bump allocator that gives every rank the same offsets (all
  ranks allocate the same sizes in the same order: even shardings), and an arena-wide barrier
  kernel with bounded waits.
* all-gather - the optimizer (``optim.AdamW(emit_bf16=True, shadow_arena=arena)``) writes the bf16
  copy of every parameter shard into the arena; gathering such a tensor is ``n`` copies that read
  the peers' arenas at the same offset.  No handshake per collective: the shards only change
  inside ``optimizer.step()``, which the optimizer brackets with two arena barriers.
* reduce-scatter - each rank's copy engines push chunk ``r`` of its fp32 partial into slot
  ``rank`` of owner ``r``'s staging ring; tiny kernels raise / await sequence numbers; the owner adds
  the slots with a light kernel (no shared memory, so it runs beside a persistent GEMM CTA).

Tensors that do not live in the arena, dims that are not leading, and dtypes other than fp32 for
reductions fall through to the next back-end (this framework's peer-load kernels or NCCL).

Reference counterpart: the reference relies on NCCL for these collectives and on Inductor's
overlap scheduler to hide them (autoparallel/compile.py:19-24); it has no SM-free path.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from . import comm_ops

_ALIGN = 256


class PeerArena:
    """One symmetric allocation per rank, addressable by every rank of the world."""

    def __init__(self, capacity_bytes: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import cuda_impl

        cuda_impl.ensure_loaded()
        self._C = cuda_impl.extension()
        self.pg = group or dist.group.WORLD
        self.rank = dist.get_rank(self.pg)
        self.n = dist.get_world_size(self.pg)
        self.world_ranks = dist.get_process_group_ranks(self.pg)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.capacity = int(capacity_bytes)
        self.buf = symm_mem.empty(self.capacity, dtype=torch.uint8, device=self.device)
        self.hdl = symm_mem.rendezvous(self.buf, self.pg.group_name)
        self.bases = [int(p) for p in self.hdl.buffer_ptrs]  # indexed by rank in ``group``
        self.base = self.bases[self.rank]
        self.status = cuda_impl.status_buffer(self.device)
        self._top = 0
        self.flag_bytes = int(self._C.dma_flag_bytes())
        self._flags_off = self._reserve(self.flag_bytes)
        self.buf[self._flags_off : self._flags_off + self.flag_bytes].zero_()
        self._epoch = 0
        torch.cuda.synchronize()
        dist.barrier(self.pg)

    # ------------------------------------------------------------------ allocation
    def _reserve(self, nbytes: int) -> int:
        off = (self._top + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + nbytes > self.capacity:
            raise MemoryError(f"peer arena exhausted: {off + nbytes} > {self.capacity} bytes")
        self._top = off + nbytes
        return off

    def alloc(self, shape, dtype) -> torch.Tensor:
        """A tensor inside the arena.  Every rank must make the same calls in the same order."""
        numel = math.prod(shape)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = self._reserve(max(nbytes, 1))
        return self.buf[off : off + nbytes].view(dtype).view(*shape)

    def offset_of(self, x: torch.Tensor) -> Optional[int]:
        off = x.data_ptr() - self.base
        if 0 <= off and off + x.numel() * x.element_size() <= self.capacity and x.device == self.device:
            return off
        return None

    @property
    def bytes_free(self) -> int:
        return self.capacity - self._top

    # ------------------------------------------------------------------ synchronisation
    def barrier(self) -> None:
        """Stream-ordered barrier over the arena's group (one tiny kernel, bounded waits)."""
        from ..ops import cuda_impl

        self._epoch += 1
        flags = [b + self._flags_off for b in self.bases]
        self._C.dma_barrier(flags, self.rank, self._epoch & 0xFFFFFFFF, self.status)
        cuda_impl._count()


class DmaGroup:
    """Copy-engine all-gather / reduce-scatter for one process group whose members share ``arena``."""

    def __init__(self, group, arena: PeerArena, ring: int = 4, slot_bytes: int = 64 << 20, sum_ctas: int = 48):
        self.pg = group if not isinstance(group, str) else dist.distributed_c10d._resolve_process_group(group)
        self.group_name = self.pg.group_name
        self.arena = arena
        self._C = arena._C
        self.rank = dist.get_rank(self.pg)
        self.n = dist.get_world_size(self.pg)
        arena_index = {wr: i for i, wr in enumerate(arena.world_ranks)}
        members = dist.get_process_group_ranks(self.pg)
        self.bases = [arena.bases[arena_index[wr]] for wr in members]
        self.ring = max(1, min(int(ring), int(self._C.dma_ring_max())))
        self.slot_bytes = int(slot_bytes)
        self.sum_ctas = int(sum_ctas)
        # identical reservations on every rank of the world keep the arena's offsets symmetric
        flags_off = arena._reserve(arena.flag_bytes)
        arena.buf[flags_off : flags_off + arena.flag_bytes].zero_()
        self.flags = [b + flags_off for b in self.bases]
        self.stage_off = arena._reserve(self.ring * self.n * self.slot_bytes) if self.n > 1 else 0
        # three streams: pulls never wait for a peer; pushes wait for "slot consumed"; sums wait for "pushed"
        self.gather_stream = torch.cuda.Stream(device=arena.device)
        self.push_stream = torch.cuda.Stream(device=arena.device)
        self.sum_stream = torch.cuda.Stream(device=arena.device)
        self.reductions = self.n > 1 and self.slot_bytes > 0
        self.seq = 0
        self._pending: dict[int, torch.cuda.Event] = {}
        self.stats = {"all_gather": 0, "reduce_scatter": 0, "bytes_pulled": 0, "bytes_pushed": 0}
        torch.cuda.synchronize()
        dist.barrier(self.pg)

    # ------------------------------------------------------------------ eligibility
    def can_gather(self, x: torch.Tensor, dim: int) -> bool:
        if not (x.is_cuda and x.is_contiguous() and x.numel() > 0):
            return False
        return self.arena.offset_of(x) is not None

    def can_reduce(self, x: torch.Tensor, dim: int) -> bool:
        if not (self.reductions and x.is_cuda and x.dtype == torch.float32 and dim == 0 and x.numel() > 0
                and x.shape[0] % self.n == 0):
            return False
        chunk = x.numel() * 4 // self.n
        return chunk % 16 == 0 and chunk <= self.slot_bytes and x.data_ptr() % 16 == 0

    # ------------------------------------------------------------------ collectives (split phase)
    def all_gather_start(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        shape = list(x.shape)
        outer = math.prod(shape[:dim]) if dim > 0 else 1
        inner = math.prod(shape[dim:]) * x.element_size()
        shape[dim] *= self.n
        cur = torch.cuda.current_stream()
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
        # the output block may have been freed by a kernel that is still queued on the compute stream
        self.gather_stream.wait_stream(cur)
        with torch.cuda.stream(self.gather_stream):
            self._C.dma_all_gather(out, self.bases, self.arena.offset_of(x), outer, inner, self.rank)
            ev = torch.cuda.Event()
            ev.record(self.gather_stream)
        out.record_stream(self.gather_stream)
        self._pending[out.data_ptr()] = ev
        comm_ops._symm_pending[out.data_ptr()] = self
        self.stats["all_gather"] += 1
        self.stats["bytes_pulled"] += (self.n - 1) * outer * inner
        return out

    def all_gather(self, x: torch.Tensor, dim: int) -> torch.Tensor:
        out = self.all_gather_start(x, dim)
        self.wait(out)
        comm_ops._symm_pending.pop(out.data_ptr(), None)
        return out

    def reduce_scatter_start(self, x: torch.Tensor, dim: int, scale: float = 1.0) -> torch.Tensor:
        from ..ops import cuda_impl

        x = x.contiguous()
        shape = list(x.shape)
        shape[0] //= self.n
        cur = torch.cuda.current_stream()
        out = torch.empty(shape, dtype=torch.float32, device=x.device)
        self.seq += 1
        seq = self.seq
        entry = seq % self.ring
        self.push_stream.wait_stream(cur)
        self.sum_stream.wait_stream(cur)
        with torch.cuda.stream(self.push_stream):
            self._C.dma_rs_push(x, self.bases, self.flags, self.stage_off, self.slot_bytes, entry, self.ring, seq & 0xFFFFFFFF,
                                self.rank, self.arena.status)
        with torch.cuda.stream(self.sum_stream):
            self._C.dma_rs_sum(x, out, self.bases, self.flags, self.stage_off, self.slot_bytes, entry, seq & 0xFFFFFFFF,
                               float(scale), self.rank, self.sum_ctas, self.arena.status)
            ev = torch.cuda.Event()
            ev.record(self.sum_stream)
        x.record_stream(self.push_stream)
        x.record_stream(self.sum_stream)
        out.record_stream(self.sum_stream)
        self._pending[out.data_ptr()] = ev
        comm_ops._symm_pending[out.data_ptr()] = self
        self.stats["reduce_scatter"] += 1
        self.stats["bytes_pushed"] += (self.n - 1) * out.numel() * 4
        cuda_impl._count(5)  # consumed-wait, pushed-signal, pushed-wait, sum, consumed-signal
        return out

    def reduce_scatter(self, x: torch.Tensor, dim: int, scale: float = 1.0) -> torch.Tensor:
        out = self.reduce_scatter_start(x, dim, scale)
        self.wait(out)
        comm_ops._symm_pending.pop(out.data_ptr(), None)
        return out

    def wait(self, out: torch.Tensor) -> None:
        ev = self._pending.pop(out.data_ptr(), None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)


_arena: Optional[PeerArena] = None
_groups: dict[str, DmaGroup] = {}


def arena() -> Optional[PeerArena]:
    return _arena


def enable_for_mesh(mesh, arena_bytes: int, ring: int = 4, slot_bytes: int = 64 << 20, sum_ctas: int = 48,
                    reductions: bool = True) -> PeerArena:
    """Create the world arena and one communicator per mesh dim of extent > 1 (collective over the world)."""
    global _arena
    if _arena is None:
        _arena = PeerArena(arena_bytes)
    for i in range(mesh.ndim):
        if mesh.shape[i] <= 1:
            continue
        pg = mesh.get_group(i)
        if pg.group_name not in _groups:
            g = DmaGroup(pg, _arena, ring=ring, slot_bytes=slot_bytes if reductions else 0, sum_ctas=sum_ctas)
            _groups[pg.group_name] = g
            comm_ops._dma_backends[pg.group_name] = g
    return _arena


def disable_all() -> None:
    global _arena
    for name in list(_groups):
        comm_ops._dma_backends.pop(name, None)
        _groups.pop(name, None)
    _arena = None


def stats() -> dict:
    out = {"all_gather": 0, "reduce_scatter": 0, "bytes_pulled": 0, "bytes_pushed": 0}
    for g in _groups.values():
        for k in out:
            out[k] += g.stats[k]
    return out
