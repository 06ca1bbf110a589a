"""Analytic model of NCCL collective time (ring / tree / NVLS × LL / LL128 / Simple).

This is the fallback pricing for mesh dims whose collectives still run through NCCL (the
NCCL-only baseline plan, inter-node dims) and the reference point the measured NVLink-5 table is
compared against.  Two layers: groups inside one NVSwitch node are priced from measured bandwidth / latency
tables (a ring through a switch never pays per-hop link latency, so the per-step model overestimates it);
everything else goes through ``nccl_tuning`` – per-algorithm bandwidth capped per channel, per-protocol
efficiency, base + per-step latencies, Tree / Ring corrections.  Numbers for H100 come from
nccl-tests fits; B200 numbers are measured on an 8-GPU NVSwitch node (peer copy 770 GB/s per
direction, 8-rank all-reduce bus bandwidth 725 GB/s at 1 GiB).  Reference:
autoparallel/cost_models/nccl_cost_model.py:40-1473 (whose "B200 ⇒ 72 GPUs per node" rule disables
itself on an 8-GPU host, :1341-1400 – here detection is by ranks per host, never by device name).
"""
from __future__ import annotations

import dataclasses
import enum
import math
from typing import Optional, Sequence


class Arch(enum.Enum):
    AMPERE = "ampere"
    HOPPER = "hopper"
    BLACKWELL = "blackwell"


class Algo(enum.Enum):
    RING = "ring"
    TREE = "tree"
    NVLS = "nvls"
    NVLS_TREE = "nvls_tree"
    COLLNET_DIRECT = "collnet_direct"
    COLLNET_CHAIN = "collnet_chain"


class Proto(enum.Enum):
    LL = "ll"
    LL128 = "ll128"
    SIMPLE = "simple"


class Coll(enum.Enum):
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"
    ALL_REDUCE = "all_reduce"
    ALL_TO_ALL = "all_to_all"
    BROADCAST = "broadcast"


@dataclasses.dataclass(frozen=True)
class TopoConfig:
    arch: Arch
    gpus_per_node: int
    n_nodes: int = 1
    intra_bw_gbs: float = 640.0  # per-GPU NVLink bandwidth available to a collective
    inter_bw_gbs: float = 50.0  # per-GPU NIC bandwidth
    nvswitch: bool = True
    nvls: bool = True
    max_channels: int = 32
    n_channels: int = 0  # channels a collective uses (0: the architecture's default)
    collnet: bool = False  # in-network reduction offered by the fabric (SHARP)


_NVLS_EFF = {Arch.AMPERE: 0.0, Arch.HOPPER: 0.85, Arch.BLACKWELL: 0.74}

#: measured intra-node algorithm bandwidth at 1 GiB (GB/s) and small-message latency (us) on NVSwitch
_MEASURED_INTRA = {
    Arch.HOPPER: {
        "ag_rs_bw": {2: 537.0, 4: 434.0, 8: 394.0},
        "ar_bw": {2: 324.0, 4: 236.0, 8: 267.0},
        "ag_rs_lat": {2: 8.0, 4: 17.0, 8: 30.0},
        "ar_lat": {2: 10.0, 4: 15.0, 8: 31.0},
        "a2a_bw": 380.0,
        "a2a_lat": 50.0,
    },
    Arch.BLACKWELL: {
        "ag_rs_bw": {2: 690.0, 4: 700.0, 8: 710.0},
        "ar_bw": {2: 520.0, 4: 400.0, 8: 414.0},  # busbw 725 at n=8: algbw = busbw * n / (2 (n-1))
        "ag_rs_lat": {2: 8.0, 4: 10.0, 8: 14.0},
        "ar_lat": {2: 9.0, 4: 11.0, 8: 16.0},
        "a2a_bw": 640.0,
        "a2a_lat": 25.0,
    },
    Arch.AMPERE: {
        "ag_rs_bw": {2: 180.0, 4: 160.0, 8: 150.0},
        "ar_bw": {2: 110.0, 4: 90.0, 8: 95.0},
        "ag_rs_lat": {2: 10.0, 4: 20.0, 8: 35.0},
        "ar_lat": {2: 12.0, 4: 20.0, 8: 38.0},
        "a2a_bw": 120.0,
        "a2a_lat": 60.0,
    },
}


def _interp(table: dict, n: int) -> float:
    ks = sorted(table)
    if n <= ks[0]:
        return table[ks[0]]
    if n >= ks[-1]:
        return table[ks[-1]]
    for a, b in zip(ks, ks[1:]):
        if a <= n <= b:
            w = (math.log2(n) - math.log2(a)) / (math.log2(b) - math.log2(a))
            return table[a] + w * (table[b] - table[a])
    return table[ks[-1]]


def eligible(algo: Algo, coll: Coll, topo: TopoConfig, n_ranks: int) -> bool:
    if algo is Algo.RING:
        return True
    if coll is not Coll.ALL_REDUCE and algo in (Algo.TREE, Algo.NVLS_TREE):
        return False
    if algo is Algo.TREE:
        return True
    if algo is Algo.NVLS:
        return topo.nvls and _NVLS_EFF[topo.arch] > 0 and topo.n_nodes == 1 and n_ranks > 2
    if algo is Algo.NVLS_TREE:
        return topo.nvls and _NVLS_EFF[topo.arch] > 0 and topo.n_nodes > 1
    if algo in (Algo.COLLNET_DIRECT, Algo.COLLNET_CHAIN):
        return topo.collnet and topo.n_nodes > 1 and coll is Coll.ALL_REDUCE
    return False


def collective_time_us(coll: Coll, nbytes: float, n_ranks: int, topo: TopoConfig) -> float:
    """Best (algorithm, protocol) time, with the measured NVSwitch layer for single-node groups."""
    if n_ranks <= 1 or nbytes <= 0:
        return 0.0
    if coll is Coll.ALL_TO_ALL:
        return all_to_all_time_us(nbytes, n_ranks, topo)
    if topo.nvswitch and n_ranks <= topo.gpus_per_node:
        m = _MEASURED_INTRA[topo.arch]
        if coll is Coll.ALL_REDUCE:
            return _interp(m["ar_lat"], n_ranks) + nbytes / (_interp(m["ar_bw"], n_ranks) * 1e3)
        return _interp(m["ag_rs_lat"], n_ranks) + nbytes / (_interp(m["ag_rs_bw"], n_ranks) * 1e3)
    # everything else (several nodes, or no NVSwitch): the per-algorithm, per-protocol tuning model
    from . import nccl_tuning as T

    ppn = max(1, min(topo.gpus_per_node, n_ranks))
    ch = topo.n_channels or T.DEFAULT_CHANNELS[topo.arch]
    d = T.DimTopo(n_ranks, ppn, max(1, n_ranks // ppn), ch, topo.intra_bw_gbs / ch, topo.inter_bw_gbs / ch)
    return T.best_time_us(coll, nbytes, d, topo)[0]


def dim_collective_time_us(coll: Coll, nbytes: float, d, topo: TopoConfig) -> float:
    """Like ``collective_time_us`` for the group of one mesh dim (``d``: ``nccl_tuning.DimTopo``), whose members
    may be spread over nodes with fewer than ``gpus_per_node`` of them in each."""
    from . import nccl_tuning as T

    if d.n_ranks <= 1 or nbytes <= 0:
        return 0.0
    if coll is Coll.ALL_TO_ALL:
        return T.all_to_all_us(nbytes, d, topo)
    if topo.nvswitch and d.n_nodes == 1:
        return collective_time_us(coll, nbytes, d.n_ranks, topo)
    return T.best_time_us(coll, nbytes, d, topo)[0]


def all_to_all_time_us(nbytes_local: float, n_ranks: int, topo: TopoConfig) -> float:
    from . import nccl_tuning as T

    ppn = max(1, min(topo.gpus_per_node, n_ranks))
    ch = topo.n_channels or T.DEFAULT_CHANNELS[topo.arch]
    d = T.DimTopo(n_ranks, ppn, max(1, n_ranks // ppn), ch, topo.intra_bw_gbs / ch, topo.inter_bw_gbs / ch)
    return T.all_to_all_us(nbytes_local, d, topo)


def a100_topo(n_nodes: int = 1) -> TopoConfig:
    return TopoConfig(Arch.AMPERE, 8, n_nodes, intra_bw_gbs=87.7 * 2, inter_bw_gbs=25.0, nvls=False)


def h100_topo(n_nodes: int = 1) -> TopoConfig:
    return TopoConfig(Arch.HOPPER, 8, n_nodes, intra_bw_gbs=320.0, inter_bw_gbs=50.0)


def b200_topo(n_nodes: int = 1) -> TopoConfig:
    return TopoConfig(Arch.BLACKWELL, 8, n_nodes, intra_bw_gbs=770.0, inter_bw_gbs=50.0)


def gb200_nvl72_topo(n_racks: int = 1) -> TopoConfig:
    return TopoConfig(Arch.BLACKWELL, 72, n_racks, intra_bw_gbs=770.0, inter_bw_gbs=50.0)


def detect_topology(world_size: int, ranks_per_host: Optional[int] = None, device_name: str = "") -> TopoConfig:
    """Topology from what is observable: ranks per host (default: all on one host up to 8) and, only
    for the architecture generation, the device name."""
    from .nccl_tuning import arch_from_device_name

    arch = arch_from_device_name(device_name) or Arch.BLACKWELL  # this package targets B200: unknown names plan as such
    rph = ranks_per_host or min(world_size, 8)
    n_nodes = max(1, world_size // rph)
    base = {Arch.BLACKWELL: b200_topo, Arch.HOPPER: h100_topo, Arch.AMPERE: a100_topo}[arch](n_nodes)
    return dataclasses.replace(base, gpus_per_node=rph)


def topology_link_models(topo: TopoConfig, mesh_shape: Sequence[int]):
    """Per-mesh-dim ``LinkModel`` for ``cost.comm.Topology`` built from this model (innermost mesh
    dim is the fastest-varying rank index)."""
    from .comm import LinkModel

    links = []
    stride = 1
    per_dim = []
    for n in reversed(mesh_shape):
        per_dim.append((n, stride))
        stride *= n
    per_dim.reverse()
    for n, st in per_dim:
        spans = st * n > topo.gpus_per_node
        m = _MEASURED_INTRA[topo.arch]
        if spans:
            links.append(LinkModel(bw_gbs=topo.inter_bw_gbs, allreduce_busbw_gbs=topo.inter_bw_gbs * 0.9, a2a_bw_gbs=topo.inter_bw_gbs * 0.8,
                                   latency_us={2: 25.0, 4: 35.0, 8: 50.0}))
        else:
            links.append(LinkModel(bw_gbs=_interp(m["ag_rs_bw"], n), allreduce_busbw_gbs=_interp(m["ar_bw"], n) * 2 * (n - 1) / max(n, 1),
                                   a2a_bw_gbs=m["a2a_bw"], latency_us=dict(m["ag_rs_lat"])))
    return links
