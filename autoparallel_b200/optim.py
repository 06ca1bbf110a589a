"""AdamW on local shards with one multi-tensor sm_100a kernel launch per step.

State layout follows ``torch.optim.AdamW`` (``step``, ``exp_avg``, ``exp_avg_sq`` per parameter;
for DTensor parameters the state tensors are DTensors with the parameter's placement), so
``torch.distributed.checkpoint`` state-dict helpers treat it like the stock optimizer – the
reference simply uses ``torch.optim`` on DTensor parameters (tests/test_dcp_roundtrip.py:142).
On CUDA the update for *all* parameters is one kernel launch driven by a device-resident table of
pointers that is built once; on CPU the same math runs in PyTorch.
"""
from __future__ import annotations

import struct
from typing import Iterable

import torch
from torch.distributed.tensor import DTensor


def _local(t):
    return t._local_tensor if isinstance(t, DTensor) else t


def lp_dev_capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


class AdamW(torch.optim.Optimizer):
    CHUNK = 65536

    def __init__(self, params: Iterable, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_scale: float = 1.0,
                 emit_bf16: bool = False, shadow_arena=None):
        """``emit_bf16``: also write every updated fp32 parameter as bf16 into a shadow buffer that
        ``apb200::dtype_cast`` hands out in place of a cast (ops/shadow.py); costs 2 bytes per parameter.
        ``shadow_arena`` (``runtime.dma.PeerArena``): the shadows are allocated inside the peer-addressable arena, so
        that parameter all-gathers can be served by the copy engines; ``step()`` then brackets the update with two
        arena barriers (no peer may still be reading the old shards, none may read the new ones too early)."""
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.grad_scale = grad_scale
        self.emit_bf16 = emit_bf16
        self.shadow_arena = shadow_arena if emit_bf16 else None
        self._shadows: dict = {}
        self._tables: dict = {}
        #: per parameter group: {"host": pinned fp32[3], "dev": fp32[3]} = (lr, bias correction 1, bias correction 2), read
        #: by the kernel at run time when a step has been captured in a CUDA graph (``runtime.graph_step``)
        self._hyper: dict = {}
        self._graph_keepalive: list = []

    @staticmethod
    def _even_shards(p) -> bool:
        """True when every rank holds a shard of the same shape.  Only then do all ranks make the same arena allocations
        in the same order, which is what keeps the arena's offsets equal on every rank (a peer's shard is read at this
        rank's own offset)."""
        spec = getattr(p, "_spec", None)
        if spec is None:
            return True
        shape = list(p.shape)
        for i, pl in enumerate(spec.placements):
            if pl.is_shard():
                n = spec.mesh.size(i)
                if shape[pl.dim] % n:
                    return False
                shape[pl.dim] //= n
        return True

    def _shadow_of(self, p):
        lp = _local(p)
        sh = self._shadows.get(id(p))
        if sh is None or sh.shape != lp.shape or sh.device != lp.device:
            sh = None
            if self.shadow_arena is not None and lp.is_cuda and self._even_shards(p):
                try:
                    sh = self.shadow_arena.alloc(tuple(lp.shape), torch.bfloat16)
                except MemoryError:
                    sh = None  # arena full: this shard's gathers fall back to the ordinary collectives
            if sh is None:
                sh = torch.empty_like(lp, dtype=torch.bfloat16)
            self._shadows[id(p)] = sh
        return sh

    def _init_state(self, p):
        st = self.state[p]
        if len(st) == 0:
            st["step"] = torch.zeros((), dtype=torch.float32)
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    def _table(self, gi: int, plist):
        """Device table of (p, g, m, v, p_lp, n) records + chunk list; rebuilt if a pointer moved."""
        key = tuple((_local(p).data_ptr(), _local(p.grad).data_ptr()) for p in plist)
        cached = self._tables.get(gi)
        if cached is not None and cached[0] == key:
            return cached[1], cached[2], cached[3]
        recs, chunks = bytearray(), []
        for ti, p in enumerate(plist):
            st = self.state[p]
            lp, lg = _local(p), _local(p.grad)
            n = lp.numel()
            lp_ptr = self._shadow_of(p).data_ptr() if self.emit_bf16 and lp.dtype == torch.float32 else 0
            recs += struct.pack("<QQQQQq", lp.data_ptr(), lg.data_ptr(), _local(st["exp_avg"]).data_ptr(),
                                _local(st["exp_avg_sq"]).data_ptr(), lp_ptr, n)
            chunks += [(ti, c) for c in range((n + self.CHUNK - 1) // self.CHUNK)]
        dev = _local(plist[0]).device
        # Gradients are fresh tensors every step, so the record table changes every step: stage it in
        # pinned memory and copy asynchronously (a pageable copy would stall the host until the GPU has
        # drained the whole backward pass).  The chunk list only depends on the sizes and is kept.
        nbytes = len(recs)
        capturing = lp_dev_capturing()
        stage = cached[4] if cached is not None and cached[4].numel() == nbytes else None
        if stage is None:
            stage = {"host": torch.empty(nbytes, dtype=torch.uint8, pin_memory=True),
                     "dev": torch.empty(nbytes, dtype=torch.uint8, device=dev), "ev": None}
            ch = torch.tensor(chunks, dtype=torch.int32).reshape(-1, 2).to(dev)
        else:
            stage, ch = cached[5], cached[2]
        if stage["ev"] is not None and not capturing:
            stage["ev"].synchronize()  # the previous copy out of the pinned buffer has completed
        stage["host"].copy_(torch.frombuffer(recs, dtype=torch.uint8))
        stage["dev"].copy_(stage["host"], non_blocking=True)
        if not capturing:  # (a captured copy re-reads the pinned table on every replay: it must stay as written here)
            stage["ev"] = torch.cuda.Event()
            stage["ev"].record()
        table = stage["dev"]
        if capturing:
            # the captured copy re-reads this pinned table on every replay: keep it (and the chunk list) alive and out
            # of reach of later eager steps, which build their own
            self._graph_keepalive.append((stage, ch))
            self._tables.pop(gi, None)
        else:
            self._tables[gi] = (key, table, ch, len(chunks), stage["host"], stage)
        return table, ch, len(chunks)

    def _hyper_buffers(self, gi: int, device):
        h = self._hyper.get(gi)
        if h is None:
            h = {"host": torch.zeros(3, dtype=torch.float32, pin_memory=True), "dev": torch.zeros(3, dtype=torch.float32, device=device)}
            self._hyper[gi] = h
        return h

    def prepare_capture(self) -> None:
        """Allocate, ahead of a stream capture, what ``step()`` would otherwise allocate inside it (pinned memory
        cannot be obtained while a stream is capturing).  Needs one eager ``step()`` to have run."""
        for gi, group in enumerate(self.param_groups):
            plist = [p for p in group["params"]]
            if plist:
                self._hyper_buffers(gi, _local(plist[0]).device)
            if gi not in self._tables:
                raise RuntimeError("run one eager optimizer step before capturing (the pointer table is sized by it)")

    @torch.no_grad()
    def advance_for_replay(self) -> None:
        """Before replaying a captured step: count the step and hand the kernel this step's learning rate and bias
        corrections (12 bytes per parameter group, copied on the current stream ahead of the graph launch)."""
        for gi, group in enumerate(self.param_groups):
            plist = [p for p in group["params"] if p in self.state and len(self.state[p])]
            if not plist:
                continue
            b1, b2 = group["betas"]
            for p in plist:
                self.state[p]["step"] += 1
            step = float(self.state[plist[0]]["step"])
            h = self._hyper_buffers(gi, _local(plist[0]).device)
            if h.get("ev") is not None:
                h["ev"].synchronize()  # the previous step's copy has read the pinned values (host runs at most one step ahead)
            h["host"][0] = group["lr"]
            h["host"][1] = 1 - b1**step
            h["host"][2] = 1 - b2**step
            h["dev"].copy_(h["host"], non_blocking=True)
            h["ev"] = torch.cuda.Event()
            h["ev"].record()

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for gi, group in enumerate(self.param_groups):
            plist = [p for p in group["params"] if p.grad is not None]
            if not plist:
                continue
            for p in plist:
                self._init_state(p)
            b1, b2 = group["betas"]
            capturing = lp_dev_capturing()
            step = None
            for p in plist:
                st = self.state[p]
                if not capturing:  # a captured step is counted when it is replayed (``advance_for_replay``)
                    st["step"] += 1
                step = float(st["step"]) if step is None else step
            step = max(step, 1.0)
            bc1, bc2 = 1 - b1**step, 1 - b2**step
            lp0 = _local(plist[0])
            fast = lp0.is_cuda and all(
                _local(p).dtype == torch.float32 and _local(p.grad).dtype == torch.float32 and _local(p).is_contiguous()
                and _local(p.grad).is_contiguous()
                for p in plist
            )
            if fast:
                from .ops import cuda_impl

                cuda_impl.ensure_loaded()
                table, ch, n = self._table(gi, plist)
                if self.shadow_arena is not None:
                    self.shadow_arena.barrier()  # every rank has finished reading the old shards
                hyper = self._hyper_buffers(gi, lp0.device)["dev"] if capturing else None
                cuda_impl.extension().adamw(table, ch, n, group["lr"], b1, b2, group["eps"], group["weight_decay"], bc1, bc2,
                                            self.grad_scale, hyper)
                cuda_impl._count()
                if self.shadow_arena is not None:
                    self.shadow_arena.barrier()  # the new shards are complete on every rank before anyone pulls
                if self.emit_bf16:
                    from .ops import shadow

                    for p in plist:
                        shadow.publish(_local(p), self._shadow_of(p))
            else:
                for p in plist:
                    st = self.state[p]
                    lp, g = _local(p), _local(p.grad).to(torch.float32) * self.grad_scale
                    m, v = _local(st["exp_avg"]), _local(st["exp_avg_sq"])
                    m.mul_(b1).add_(g, alpha=1 - b1)
                    v.mul_(b2).addcmul_(g, g, value=1 - b2)
                    upd = (m / bc1) / ((v / bc2).sqrt() + group["eps"])
                    lp.mul_(1 - group["lr"] * group["weight_decay"]).add_(upd.to(lp.dtype), alpha=-group["lr"])
                    if self.emit_bf16 and lp.dtype == torch.float32:
                        from .ops import shadow

                        sh = self._shadow_of(p)
                        sh.copy_(lp)
                        shadow.publish(lp, sh)
        return loss
