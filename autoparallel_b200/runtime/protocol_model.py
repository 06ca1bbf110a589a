"""Host model of the flag protocol that the symmetric-memory kernels follow, for checking it without a GPU.

Every rank owns a workspace ``[ flags | staging ]`` that all ranks can address.  Flags carry the epoch of
the collective that wrote them and only grow:

* ``ready[r]`` on rank p – rank r's staging content for this epoch is complete (p may pull from it),
* ``done[r]``  on rank p – rank r will not touch p's staging for this epoch any more,
* ``contrib[r]`` on rank p – rank r has stored all its partial results into p's staging (GEMM → reduce-scatter).

The device code is in ``ops/csrc/symm_proto.cuh`` (waits, flag layout), ``symm_comm.cu`` (stand-alone
collectives), ``gemm_core.cuh`` / ``gemm_fused.cu`` (fused kernels).  This module restates the same steps with
one Python thread per rank and the same ordering rules, so that the protocol – not the CUDA – can be
exercised under arbitrary interleavings, with ranks that are late, and with a rank that never raises a flag.
A wait that runs out does what the kernels do: it records ``(rank, flag, peer, expected, observed)`` and the
collective returns an error instead of blocking.
"""
from __future__ import annotations

import dataclasses
import random
import threading
import time
from typing import Callable, Optional

import numpy as np


@dataclasses.dataclass
class WaitTimeout:
    rank: int
    flag: str
    peer: int
    expected: int
    observed: int


class Workspace:
    """One rank's symmetric buffer: three flag arrays and a staging area."""

    def __init__(self, n: int, stage_elems: int):
        self.ready = [0] * n
        self.done = [0] * n
        self.contrib = [0] * n
        self.stage = np.zeros(stage_elems, dtype=np.float32)


class Fabric:
    """All workspaces plus the condition variable that stands in for memory becoming visible."""

    def __init__(self, n: int, stage_elems: int, wait_limit_s: float = 0.5, jitter: float = 0.0, seed: int = 0):
        self.n = n
        self.ws = [Workspace(n, stage_elems) for _ in range(n)]
        self.cv = threading.Condition()
        self.wait_limit_s = wait_limit_s
        self.jitter = jitter
        self.rng = random.Random(seed)
        self.errors: list[WaitTimeout] = []

    # -- the two primitives of symm_proto.cuh
    def raise_flag(self, owner: int, kind: str, idx: int, epoch: int) -> None:
        """``st.release`` of ``epoch`` into ``kind[idx]`` of rank ``owner``'s workspace."""
        self._pause()
        with self.cv:
            flags = getattr(self.ws[owner], kind)
            flags[idx] = max(flags[idx], epoch)
            self.cv.notify_all()

    def wait_ge(self, rank: int, kind: str, idx: int, epoch: int) -> bool:
        """Bounded ``ld.acquire`` spin on ``kind[idx] >= epoch`` of ``rank``'s own workspace."""
        deadline = time.monotonic() + self.wait_limit_s
        with self.cv:
            flags = getattr(self.ws[rank], kind)
            while flags[idx] < epoch:
                left = deadline - time.monotonic()
                if left <= 0:
                    self.errors.append(WaitTimeout(rank, kind, idx, epoch, flags[idx]))
                    return False
                self.cv.wait(left)
        return True

    def _pause(self) -> None:
        if self.jitter:
            time.sleep(self.rng.random() * self.jitter)


# ------------------------------------------------------------------------------------- collectives
def all_gather(f: Fabric, rank: int, epoch: int, shard: np.ndarray, skip_ready: bool = False) -> Optional[np.ndarray]:
    """Pull-based all-gather (symm_comm.cu; the gather warp of the fused kernel follows the same steps)."""
    n, me = f.n, f.ws[rank]
    m = shard.size
    for peer in range(n):  # phase 0: my staging is free once every peer has finished the previous collective
        if peer != rank and not f.wait_ge(rank, "done", peer, epoch - 1):
            return None
    me.stage[:m] = shard
    if not skip_ready:  # (failure injection: a rank that never publishes)
        for peer in range(n):
            if peer != rank:
                f.raise_flag(peer, "ready", rank, epoch)
    out = np.empty(n * m, dtype=np.float32)
    out[rank * m:(rank + 1) * m] = shard
    for k in range(1, n):  # phase 1: pull every peer's shard, nearest rank first
        peer = (rank + k) % n
        if not f.wait_ge(rank, "ready", peer, epoch):
            return None
        f._pause()
        out[peer * m:(peer + 1) * m] = f.ws[peer].stage[:m]
    for peer in range(n):  # phase 2: I will not read anybody's staging again in this epoch
        if peer != rank:
            f.raise_flag(peer, "done", rank, epoch)
    return out


def gemm_reduce_scatter(f: Fabric, rank: int, epoch: int, partial: np.ndarray) -> Optional[np.ndarray]:
    """Push-based reduce-scatter of the fused GEMM: ``partial`` is this rank's full-size product; block r
    of it belongs to rank r and is stored into slot ``rank`` of r's staging area."""
    n, me = f.n, f.ws[rank]
    m = partial.size // n
    for peer in range(n):  # communication CTAs: slots are free once every peer has left the previous collective
        if peer != rank and not f.wait_ge(rank, "done", peer, epoch - 1):
            return None
    for peer in range(n):
        f.raise_flag(peer, "ready", rank, epoch)  # ... including myself: my own epilogue waits on it too
    for k in range(1, n + 1):  # epilogues: other ranks' blocks first, own block last
        owner = (rank + k) % n
        if not f.wait_ge(rank, "ready", owner, epoch):
            return None
        f._pause()
        f.ws[owner].stage[rank * m:(rank + 1) * m] = partial[owner * m:(owner + 1) * m]
    for peer in range(n):  # last GEMM CTA: all my stores are out
        f.raise_flag(peer, "contrib", rank, epoch)
        if peer != rank:
            f.raise_flag(peer, "done", rank, epoch)
    for peer in range(n):  # final sum once every rank's contribution has landed
        if not f.wait_ge(rank, "contrib", peer, epoch):
            return None
    return me.stage[: n * m].reshape(n, m).sum(0)


def run_ranks(n: int, body: Callable[[Fabric, int], object], stage_elems: int, **fabric_kw):
    """Run ``body(fabric, rank)`` on one thread per rank; returns (fabric, results by rank)."""
    f = Fabric(n, stage_elems, **fabric_kw)
    results: list = [None] * n

    def work(r):
        results[r] = body(f, r)

    threads = [threading.Thread(target=work, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    return f, results


# ------------------------------------------------------------------------------------- dynamic GEMM tiles
class TileCounters:
    """The four device integers of the dynamic tile scheduler (gemm_core.cuh, ``DYN``): next tile, pairs that
    have left, SM-pair requests of collectives, pairs that gave up their SMs in this launch."""

    def __init__(self):
        self.lock = threading.Lock()
        self.next_tile = 0
        self.left = 0
        self.requests = 0
        self.yielded = 0

    def request(self, pairs: int, cap: int = 32) -> None:
        with self.lock:
            self.requests += max(0, min(pairs, cap - self.requests))


def run_dynamic_gemm(counters: TileCounters, num_tiles: int, num_pairs: int, readers: int = 10, ring: int = 4,
                     jitter: float = 0.0, seed: int = 0) -> dict:
    """One launch: per CTA pair a fetching thread (the even CTA's producer) publishes tile indices through a
    ``ring``-entry ring that ``readers`` consumer threads (odd CTA's producer, MMA thread, eight epilogue
    warps) read and release.  Returns, per pair, the tiles each reader saw; the caller checks that every
    tile was handled exactly once and by all readers of one pair alike."""
    rng = random.Random(seed)
    seen = {p: [[] for _ in range(readers)] for p in range(num_pairs)}

    def pair_body(p):
        cv = threading.Condition()
        slots = [None] * ring
        ready = [0] * ring   # phase counters: entry published (it // ring + 1)
        freed = [0] * ring   # readers that released the entry, cumulative

        def fetch():
            it = 0
            while True:
                s = it % ring
                with cv:
                    cv.wait_for(lambda: freed[s] >= readers * (it // ring))  # everybody has read the previous use
                t, leave = -1, False
                with counters.lock:  # the atomics of the kernel, in the same order
                    if counters.requests > 0:
                        counters.requests -= 1
                        if counters.yielded < num_pairs // 2:
                            counters.yielded += 1
                            leave = True
                        else:
                            counters.requests += 1
                    if not leave:
                        t = counters.next_tile
                        counters.next_tile += 1
                        if t >= num_tiles:
                            t = -1
                if jitter:
                    time.sleep(rng.random() * jitter)
                with cv:
                    slots[s] = t
                    ready[s] = it // ring + 1
                    cv.notify_all()
                it += 1
                if t < 0:
                    with counters.lock:
                        counters.left += 1
                        if counters.left == num_pairs:  # last pair out zeroes the per-launch counters
                            counters.next_tile = counters.left = counters.yielded = 0
                    return

        def read(r):
            it = 0
            while True:
                s = it % ring
                with cv:
                    cv.wait_for(lambda: ready[s] >= it // ring + 1)
                    t = slots[s]
                    freed[s] += 1
                    cv.notify_all()
                it += 1
                if t < 0:
                    return
                seen[p][r].append(t)
                if jitter:
                    time.sleep(rng.random() * jitter)

        ths = [threading.Thread(target=fetch)] + [threading.Thread(target=read, args=(r,)) for r in range(readers)]
        for t in ths:
            t.start()
        for t in ths:
            t.join()

    pairs = [threading.Thread(target=pair_body, args=(p,)) for p in range(num_pairs)]
    for t in pairs:
        t.start()
    for t in pairs:
        t.join()
    return seen


# ------------------------------------------------------------------------------------- attention pipeline
class PhaseBarrier:
    """An mbarrier: ``count`` arrivals complete the current phase; ``wait(parity)`` returns once the phase of
    that parity has completed, i.e. as soon as the barrier's current phase has the other parity."""

    def __init__(self, count: int, cv: threading.Condition, limit_s: float):
        self.count, self.pending, self.phase, self.cv, self.limit_s = count, count, 0, cv, limit_s

    def arrive(self, n: int = 1) -> None:
        with self.cv:
            self.pending -= n
            assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
            if self.pending == 0:
                self.pending = self.count
                self.phase += 1
                self.cv.notify_all()

    def wait(self, parity: int) -> bool:
        with self.cv:
            return self.cv.wait_for(lambda: (self.phase & 1) != parity, self.limit_s)


def run_attention_pipeline(q: np.ndarray, k: np.ndarray, v: np.ndarray, causal: bool, scale: float,
                           jitter: float = 0.0, seed: int = 0, ring: int = 3, tile: int = 128):
    """Host model of one CTA of the attention forward kernel (ops/csrc/attention_fwd.cu): a loader, the MMA
    issuer and one softmax thread per query tile exchange the same barriers, ring slots and accumulators in
    the same order, with tensor-core work completing asynchronously.  ``q`` is [2 * tile, d] (the CTA's two
    query tiles, assumed to be the LAST rows of the sequence when ``causal``), ``k`` / ``v`` are [Sk, d].
    Returns (out, lse, errors)."""
    rng = random.Random(seed)
    cv = threading.Condition()
    lim = 5.0
    nq = 2
    sk = k.shape[0]
    first_row = sk - nq * tile if causal else 0  # absolute position of the CTA's first query row
    qi = first_row // (nq * tile)
    n_it = [(nq * qi + 1 + t) if causal else sk // tile for t in range(nq)]
    n_max = n_it[-1]
    kv_full = [PhaseBarrier(1, cv, lim) for _ in range(ring)]
    kv_empty = [PhaseBarrier(1, cv, lim) for _ in range(ring)]
    s_full = [PhaseBarrier(1, cv, lim) for _ in range(nq)]
    p_full = [PhaseBarrier(1, cv, lim) for _ in range(nq)]  # (128 thread arrivals in the kernel; one thread here)
    pv_full = [PhaseBarrier(1, cv, lim) for _ in range(nq)]
    slots: list = [None] * ring
    S: list = [None] * nq
    P: list = [None] * nq
    PV: list = [None] * nq
    errors: list[str] = []
    out = np.zeros((nq * tile, q.shape[1]), dtype=np.float64)
    lse = np.zeros(nq * tile, dtype=np.float64)
    async_work: list[threading.Thread] = []

    def pause():
        if jitter:
            time.sleep(rng.random() * jitter)

    def tensor_core(fn, *bars):
        """MMAs complete some time after they are issued; the commit barriers fire afterwards."""
        def work():
            pause()
            fn()
            for b in bars:
                b.arrive()
        th = threading.Thread(target=work)
        async_work.append(th)
        th.start()
        return th

    def loader():
        for i in range(2 * n_max):
            s = i % ring
            if not kv_empty[s].wait(((i // ring) & 1) ^ 1):
                errors.append(f"loader: slot {s} never freed (item {i})")
                return
            pause()
            j = i >> 1
            src = v if (i & 1) else k
            slots[s] = ("V" if (i & 1) else "K", j, src[j * tile:(j + 1) * tile].copy())
            kv_full[s].arrive()

    def mma():
        pending: list[threading.Thread] = []

        def wait_kv(i):
            if not kv_full[i % ring].wait((i // ring) & 1):
                errors.append(f"mma: item {i} never arrived")
                return False
            return True

        def issue(fn, *bars):
            # MMAs of one thread complete in order: each waits for the one before it
            prev = pending[-1] if pending else None

            def chained():
                if prev is not None:
                    prev.join()
                fn()
            pending.append(tensor_core(chained, *bars))

        def qk(t, slot, j):
            def fn():
                kind, jj, data = slots[slot]
                if (kind, jj) != ("K", j):
                    errors.append(f"QK tile {t} iteration {j} read {kind}{jj}")
                S[t] = q[t * tile:(t + 1) * tile] @ data.T
            issue(fn, s_full[t])

        def pv(t, slot, j):
            def fn():
                kind, jj, data = slots[slot]
                if (kind, jj) != ("V", j):
                    errors.append(f"PV tile {t} iteration {j} read {kind}{jj}")
                PV[t] = P[t] @ data
            issue(fn, pv_full[t])

        if not wait_kv(0):
            return
        for t in range(nq):
            qk(t, 0, 0)
        issue(lambda: None, kv_empty[0])
        for j in range(n_max):
            iv, ik = 2 * j + 1, 2 * j + 2
            more = j + 1 < n_max
            if not wait_kv(iv) or (more and not wait_kv(ik)):
                return
            for t in range(nq):
                if j >= n_it[t]:
                    continue
                if not p_full[t].wait(j & 1):
                    errors.append(f"mma: P of tile {t} iteration {j} never arrived")
                    return
                pv(t, iv % ring, j)
                if j + 1 < n_it[t]:
                    qk(t, ik % ring, j + 1)
            issue(lambda: None, kv_empty[iv % ring])
            if more:
                issue(lambda: None, kv_empty[ik % ring])

    def softmax(t):
        o = np.zeros((tile, q.shape[1]))
        m_run = np.full(tile, -np.inf)
        l_run = np.zeros(tile)
        sl2 = scale * 1.4426950408889634
        rows = np.arange(tile)[:, None]
        cols = np.arange(tile)[None, :]
        for j in range(n_it[t]):
            if not s_full[t].wait(j & 1):
                errors.append(f"softmax {t}: S of iteration {j} never arrived")
                return
            pause()
            s = S[t].copy()
            mask = (cols <= rows) if (causal and j == n_it[t] - 1) else np.ones((tile, tile), bool)
            mx = np.where(mask, s, -np.inf).max(1)
            m_new = np.maximum(m_run, mx * sl2)
            alpha = np.exp2(m_run - m_new)
            if j > 0:
                if not pv_full[t].wait((j - 1) & 1):
                    errors.append(f"softmax {t}: PV of iteration {j - 1} never arrived")
                    return
                o = (o + PV[t]) * alpha[:, None]
            l_run = l_run * alpha
            m_run = m_new
            e = np.where(mask, np.exp2(s * sl2 - m_new[:, None]), 0.0)
            l_run = l_run + e.sum(1)
            pause()
            P[t] = e
            p_full[t].arrive()
        if not pv_full[t].wait((n_it[t] - 1) & 1):
            errors.append(f"softmax {t}: last PV never arrived")
            return
        out[t * tile:(t + 1) * tile] = (o + PV[t]) / l_run[:, None]
        lse[t * tile:(t + 1) * tile] = (m_run + np.log2(l_run)) * 0.6931471805599453

    ths = [threading.Thread(target=loader), threading.Thread(target=mma)] + [threading.Thread(target=softmax, args=(t,)) for t in range(nq)]
    for th in ths:
        th.start()
    for th in ths:
        th.join()
    for th in async_work:
        th.join()
    return out, lse, errors


def swizzle128_offset(row: int, chunk16: int) -> int:
    """Byte offset of 16-byte unit ``chunk16`` (0..7) of ``row`` inside a 128-byte-swizzled [rows x 128 B] tile:
    the unit index is XORed with the row index modulo 8 (what TMA writes and the MMA descriptors expect)."""
    return row * 128 + ((chunk16 ^ (row & 7)) << 4)
