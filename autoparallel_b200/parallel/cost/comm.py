"""Communication cost of changing a tensor's placement (microseconds).

``redistribute_cost(src, dst)`` walks the mesh dims and prices each per-dim transition with the
collective it lowers to – ``Shard→Replicate`` all-gather, ``Partial→Replicate`` all-reduce,
``Partial→Shard`` reduce-scatter, ``Shard(a)→Shard(b)`` all-to-all, ``Replicate→Shard`` a local
slice – forbidding transitions that would *create* a partial sum (reference semantics:
autoparallel/cost_models/collective_runtime_estimation.py:115-229).

Collectives are priced by a ``Topology``: an α–β model per mesh dim whose constants come from
measurements on NVLink 5 / NVSwitch (peer copy 770 GB/s per direction per GPU, 8-rank all-reduce
bus bandwidth 725 GB/s at 1 GiB) or from a calibration table produced by timing this
framework's own collective kernels (``cost/calibrate.py``).  The reference instead falls back to
an 87.7 GB/s ring model on an 8-GPU B200 host because its NCCL model maps "B200" to 72 GPUs per
node (autoparallel/cost_models/nccl_cost_model.py:1341-1400).
"""
from __future__ import annotations

import bisect
import dataclasses
import json
import math
from typing import Optional, Sequence

from ..strategies.dtensor_adapter import DTensorSpec, Shard

INF = float("inf")


@dataclasses.dataclass
class LinkModel:
    """α–β constants for one mesh dim."""

    bw_gbs: float = 770.0  # per-GPU unidirectional bandwidth available to the collective
    allreduce_busbw_gbs: float = 725.0
    a2a_bw_gbs: float = 700.0
    latency_us: dict = dataclasses.field(default_factory=lambda: {2: 6.0, 4: 8.0, 8: 12.0})

    def alpha(self, n: int) -> float:
        if n in self.latency_us:
            return self.latency_us[n]
        ks = sorted(self.latency_us)
        return self.latency_us[ks[-1]] * max(1.0, math.log2(max(n, 2)) / math.log2(ks[-1]))


NVLINK5 = LinkModel()
INFINIBAND = LinkModel(bw_gbs=45.0, allreduce_busbw_gbs=40.0, a2a_bw_gbs=35.0, latency_us={2: 25.0, 4: 35.0, 8: 50.0})
CPU_LOOPBACK = LinkModel(bw_gbs=10.0, allreduce_busbw_gbs=8.0, a2a_bw_gbs=8.0, latency_us={2: 20.0, 4: 30.0, 8: 40.0})


class Topology:
    """Per-mesh-dim link models plus optional measured tables.

    ``tables[(kind, n)] = sorted [(bytes, microseconds)]`` overrides the α–β formula by
    log-linear interpolation; ``kind`` ∈ {all_gather, reduce_scatter, all_reduce, all_to_all}
    and ``bytes`` is the full (gathered / pre-scatter) message size per rank.
    """

    def __init__(self, links: Sequence[LinkModel], tables: Optional[dict] = None):
        self.links = list(links)
        self.tables = tables or {}

    @classmethod
    def for_mesh(cls, mesh, gpus_per_node: int = 8) -> "Topology":
        if mesh.device_type != "cuda":
            return cls([CPU_LOOPBACK] * mesh.ndim)
        links = []
        stride = 1
        # mesh dims are laid out row-major over ranks: the last dim has stride 1
        strides = []
        for n in reversed(mesh.shape):
            strides.append(stride)
            stride *= n
        strides.reverse()
        for n, st in zip(mesh.shape, strides):
            spans_nodes = st * n > gpus_per_node
            links.append(INFINIBAND if spans_nodes else NVLINK5)
        return cls(links)

    @staticmethod
    def measured_table_path(device: str = "B200", backend: str = "nccl") -> Optional[str]:
        """Path of the collective table measured on ``device`` that ships with the package, if there is one."""
        import os

        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tables", f"{device.lower()}_nvswitch_{backend}.json")
        return path if os.path.exists(path) else None

    def load_table(self, path: str) -> None:
        with open(path) as f:
            raw = json.load(f)
        for kind, per_n in raw.get("collectives", {}).items():
            for n, pts in per_n.items():
                self.tables[(kind, int(n))] = sorted((float(b), float(us)) for b, us in pts)

    # -- primitives: ``nbytes`` = size of the FULL tensor on this mesh dim (gathered size)
    def _table(self, kind: str, n: int, nbytes: float) -> Optional[float]:
        pts = self.tables.get((kind, n))
        if not pts:
            return None
        xs = [p[0] for p in pts]
        i = bisect.bisect_left(xs, nbytes)
        if i == 0:
            return pts[0][1]
        if i >= len(pts):
            b0, t0 = pts[-1]
            return t0 * nbytes / b0
        (b0, t0), (b1, t1) = pts[i - 1], pts[i]
        w = (math.log(nbytes) - math.log(b0)) / (math.log(b1) - math.log(b0))
        return t0 + w * (t1 - t0)

    def all_gather(self, dim: int, n: int, nbytes: float) -> float:
        t = self._table("all_gather", n, nbytes)
        if t is not None:
            return t
        l = self.links[dim]
        return l.alpha(n) + nbytes * (n - 1) / n / (l.bw_gbs * 1e3)

    def reduce_scatter(self, dim: int, n: int, nbytes: float) -> float:
        t = self._table("reduce_scatter", n, nbytes)
        if t is not None:
            return t
        l = self.links[dim]
        return l.alpha(n) + nbytes * (n - 1) / n / (l.bw_gbs * 1e3)

    def all_reduce(self, dim: int, n: int, nbytes: float) -> float:
        t = self._table("all_reduce", n, nbytes)
        if t is not None:
            return t
        l = self.links[dim]
        return l.alpha(n) * 1.5 + nbytes * 2 * (n - 1) / n / (l.allreduce_busbw_gbs * 1e3)

    def all_to_all(self, dim: int, n: int, nbytes_local: float) -> float:
        t = self._table("all_to_all", n, nbytes_local)
        if t is not None:
            return t
        l = self.links[dim]
        return l.alpha(n) + nbytes_local * (n - 1) / n / (l.a2a_bw_gbs * 1e3)


class NcclTopology(Topology):
    """Prices every collective with the NCCL model (``cost/nccl_model.py``, ``cost/nccl_tuning.py``): measured tables
    inside one NVSwitch node, the per-algorithm / per-protocol tuning model across nodes.  Tables loaded with
    ``load_table`` still take precedence.  Selected by ``AutoParallel(..., cost_model="nccl")``."""

    def __init__(self, config, mesh_shape: Sequence[int], tables: Optional[dict] = None):
        from . import nccl_model, nccl_tuning

        super().__init__(nccl_model.topology_link_models(config, mesh_shape), tables)
        self.config = config
        self._m = nccl_model
        self.dims = [nccl_tuning.derive_mesh_dim_topo(config, tuple(mesh_shape), i) for i in range(len(mesh_shape))]

    def _price(self, kind: str, coll, dim: int, n: int, nbytes: float) -> float:
        t = self._table(kind, n, nbytes)
        if t is not None:
            return t
        return self._m.dim_collective_time_us(coll, nbytes, self.dims[dim], self.config)

    def all_gather(self, dim: int, n: int, nbytes: float) -> float:
        return self._price("all_gather", self._m.Coll.ALL_GATHER, dim, n, nbytes)

    def reduce_scatter(self, dim: int, n: int, nbytes: float) -> float:
        return self._price("reduce_scatter", self._m.Coll.REDUCE_SCATTER, dim, n, nbytes)

    def all_reduce(self, dim: int, n: int, nbytes: float) -> float:
        return self._price("all_reduce", self._m.Coll.ALL_REDUCE, dim, n, nbytes)

    def all_to_all(self, dim: int, n: int, nbytes_local: float) -> float:
        return self._price("all_to_all", self._m.Coll.ALL_TO_ALL, dim, n, nbytes_local)


_topology: Optional[Topology] = None
_cache: dict = {}


def set_topology(t: Optional[Topology]) -> None:
    global _topology
    _topology = t
    _cache.clear()


def get_topology(mesh=None) -> Topology:
    global _topology
    if _topology is None:
        assert mesh is not None
        return Topology.for_mesh(mesh)
    return _topology


def reset_cache() -> None:
    _cache.clear()


def _spec_key(s: DTensorSpec):
    return (tuple(s.placements), tuple(s.tensor_meta.shape), s.tensor_meta.dtype)


def redistribute_cost(src: DTensorSpec, dst: DTensorSpec, hbm_bytes_per_us: float = 6.5e6) -> float:
    """Microseconds to take a tensor from ``src`` placement to ``dst`` placement."""
    if src.placements == dst.placements:
        return 0.0
    key = (_spec_key(src), tuple(dst.placements), id(_topology))
    hit = _cache.get(key)
    if hit is not None:
        return hit
    from ..lower.redistribute import RedistributeError, plan_redistribution

    mesh = src.mesh
    topo = get_topology(mesh)
    itemsize = src.tensor_meta.dtype.itemsize
    local = list(src.tensor_meta.shape)
    for n, p in zip(mesh.shape, src.placements):
        if isinstance(p, Shard):
            local[p.dim] = -(-local[p.dim] // n)
    try:
        steps = plan_redistribution(src.placements, dst.placements, mesh.shape)
    except RedistributeError:
        steps = None
    cost = 0.0 if steps is not None else INF
    for st in steps or ():
        n = mesh.shape[st.mesh_dim]
        nbytes_local = (math.prod(local) if local else 1) * itemsize
        if st.kind == "all_gather":
            cost += topo.all_gather(st.mesh_dim, n, nbytes_local * n)
            if st.dim != 0:
                cost += 0.25 * nbytes_local * n / hbm_bytes_per_us  # strided landing of the gathered chunks
            local[st.dim] *= n
        elif st.kind == "all_reduce":
            cost += topo.all_reduce(st.mesh_dim, n, nbytes_local)
        elif st.kind == "reduce_scatter":
            cost += topo.reduce_scatter(st.mesh_dim, n, nbytes_local)
            if st.dim != 0:
                cost += 0.25 * nbytes_local / hbm_bytes_per_us
            local[st.dim] = -(-local[st.dim] // n)
        elif st.kind == "all_to_all":
            cost += topo.all_to_all(st.mesh_dim, n, nbytes_local)
            cost += 2.0 * nbytes_local / hbm_bytes_per_us  # pack + unpack
            local[st.dim2] *= n
            local[st.dim] = -(-local[st.dim] // n)
        elif st.kind == "local_chunk":
            cost += nbytes_local / n / hbm_bytes_per_us + 1.0
            local[st.dim] = -(-local[st.dim] // n)
    _cache[key] = cost
    return cost
