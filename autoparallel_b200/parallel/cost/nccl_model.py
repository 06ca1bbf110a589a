"""Analytic model of NCCL collective time (ring / tree / NVLS × LL / LL128 / Simple).

This is the fallback pricing for mesh dims whose collectives still run through NCCL (the
NCCL-only baseline plan, inter-node dims) and the reference point the measured NVLink-5 table is
compared against.  It follows the structure of NCCL's tuning model – per-algorithm bus bandwidth
capped per channel, per-protocol efficiency, base + per-hop latencies – with an empirical layer for
NVSwitch nodes where a ring never pays per-hop link latency.  Numbers for H100 come from
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


#: protocol efficiency (fraction of the link a protocol's framing leaves) and per-step latency, us
_PROTO_EFF = {Proto.LL: 0.5, Proto.LL128: 0.92, Proto.SIMPLE: 1.0}
_PROTO_LAT = {Proto.LL: 0.6, Proto.LL128: 1.0, Proto.SIMPLE: 2.4}
_BASE_LAT = {Algo.RING: 6.6, Algo.TREE: 8.4, Algo.NVLS: 5.0, Algo.NVLS_TREE: 7.0}
_NET_LAT = {Proto.LL: 5.0, Proto.LL128: 8.5, Proto.SIMPLE: 14.0}
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
    return False


def algo_time_us(coll: Coll, algo: Algo, proto: Proto, nbytes: float, n_ranks: int, topo: TopoConfig) -> float:
    """Time of one collective under a fixed (algorithm, protocol).  ``nbytes``: all-gather – gathered
    size; reduce-scatter – input size; all-reduce – tensor size."""
    if n_ranks <= 1 or nbytes <= 0:
        return 0.0
    spans_nodes = n_ranks > topo.gpus_per_node
    link = topo.inter_bw_gbs if spans_nodes else topo.intra_bw_gbs
    bw = link * _PROTO_EFF[proto]
    steps_lat = _PROTO_LAT[proto] + (_NET_LAT[proto] if spans_nodes else 0.0)
    n = n_ranks
    if algo is Algo.RING:
        if coll is Coll.ALL_REDUCE:
            traffic, steps = 2.0 * (n - 1) / n * nbytes, 2 * (n - 1)
        else:
            traffic, steps = (n - 1) / n * nbytes, n - 1
        if topo.nvswitch and not spans_nodes:
            steps = 1 + math.log2(n)  # through a switch a "ring" step costs no extra link hop
        return _BASE_LAT[algo] + steps * steps_lat + traffic / (bw * 1e3)
    if algo is Algo.TREE:
        depth = 2 * math.ceil(math.log2(n))
        return _BASE_LAT[algo] + depth * steps_lat + 2.0 * nbytes / (bw * 1e3)
    if algo is Algo.NVLS:
        # the switch reduces / multicasts: every GPU pushes its data once and receives the result once
        eff = _NVLS_EFF[topo.arch]
        traffic = nbytes if coll is Coll.ALL_REDUCE else (n - 1) / n * nbytes
        return _BASE_LAT[algo] + 2 * steps_lat + traffic / (link * eff * 1e3)
    if algo is Algo.NVLS_TREE:
        eff = _NVLS_EFF[topo.arch]
        nodes = max(1, n // topo.gpus_per_node)
        intra = nbytes / (topo.intra_bw_gbs * eff * 1e3)
        inter = 2.0 * nbytes / (topo.inter_bw_gbs * 1e3) * (nodes - 1) / nodes
        return _BASE_LAT[algo] + 2 * math.ceil(math.log2(max(nodes, 2))) * (steps_lat + _NET_LAT[proto]) + intra + inter
    raise ValueError(algo)


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
    best = math.inf
    for algo in Algo:
        if not eligible(algo, coll, topo, n_ranks):
            continue
        for proto in Proto:
            if proto is Proto.LL128 and algo in (Algo.NVLS, Algo.NVLS_TREE):
                continue
            best = min(best, algo_time_us(coll, algo, proto, nbytes, n_ranks, topo))
    return best


def all_to_all_time_us(nbytes_local: float, n_ranks: int, topo: TopoConfig) -> float:
    m = _MEASURED_INTRA[topo.arch]
    if n_ranks <= topo.gpus_per_node:
        return m["a2a_lat"] + nbytes_local * (n_ranks - 1) / n_ranks / (m["a2a_bw"] * 1e3)
    nodes = n_ranks // topo.gpus_per_node
    off_node = nbytes_local * (n_ranks - topo.gpus_per_node) / n_ranks
    on_node = nbytes_local * (topo.gpus_per_node - 1) / n_ranks
    lat = {2: 37.0, 4: 42.0, 8: 60.0, 16: 98.0, 32: 290.0}
    return _interp(lat, nodes) + max(off_node / (topo.inter_bw_gbs * 1e3), on_node / (m["a2a_bw"] * 1e3))


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
    name = device_name.upper()
    arch = Arch.BLACKWELL if ("B200" in name or "B100" in name or "GB200" in name) else Arch.HOPPER if ("H100" in name or "H200" in name) else Arch.AMPERE if "A100" in name else Arch.BLACKWELL
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
