"""Per-algorithm, per-protocol model of NCCL collectives, after the structure of NCCL's own tuning model.

For every (collective, algorithm, protocol) NCCL predicts ``latency + bytes / bandwidth`` and runs the cheapest
eligible combination.  This module restates that prediction for a *mesh dim* of a device mesh:

* ``derive_mesh_dim_topo`` – which ranks a collective over one mesh dim spans: ranks per node, nodes, channels and
  the per-channel bandwidths (innermost mesh dim = consecutive ranks);
* ``algo_bus_bw_gbs`` – bus bandwidth: channels x per-channel link bandwidth, capped per architecture
  (LL by the LL ceiling, LL128 and Tree by per-channel ceilings), scaled by protocol efficiency
  (LL 1/2 ... 1/4, LL128 0.92), Tree at half rate, NVLS / CollNet by their own efficiency factors;
* ``algo_latency_us`` – base latency of the (algorithm, protocol) plus per-step link latencies: a Ring pays
  ``n - 1`` (all-gather, reduce-scatter) or ``2 (n - 1)`` steps, intra-node steps at NVLink latency and one
  network step per node boundary; a Tree pays ``2 log2`` levels; NVLS pays a constant;
* ``algo_time_us`` – the two combined, with NCCL's small-message Tree correction and an empirical layer:
  multi-node Ring correction that grows with ring depth, a plateau where a multi-node Simple ring stops
  getting faster, and a per-node synchronisation overhead;
* ``best_time_us`` – minimum over eligible algorithms (Ring always; Tree and NVLS-Tree for all-reduce only; NVLS
  needs NVSwitch + Hopper or newer; NVLS-Tree needs several nodes; CollNet needs the fabric flag) and protocols
  (NVLS and CollNet: Simple only);
* ``all_to_all_us`` – copy-engine path inside a node, NIC-bound path across nodes with a start-up ramp.

Constants are NCCL's published tuning constants (latencies in microseconds, bandwidths in GB/s) plus fits to
nccl-tests logs; Blackwell doubles Hopper's per-channel ceilings (NVLink 5 = 2 x NVLink 4).
Reference: autoparallel/cost_models/nccl_cost_model.py:40-1473 and tests/test_nccl_cost_model.py.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Sequence

from .nccl_model import Algo, Arch, Coll, Proto, TopoConfig

_P = (Proto.LL, Proto.LL128, Proto.SIMPLE)

#: base latency per (algorithm, protocol), us
BASE_LAT = {
    Algo.TREE: {Proto.LL: 6.8, Proto.LL128: 14.0, Proto.SIMPLE: 8.4},
    Algo.RING: {Proto.LL: 6.6, Proto.LL128: 14.0, Proto.SIMPLE: 8.4},
    Algo.COLLNET_DIRECT: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 0.0},
    Algo.COLLNET_CHAIN: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 0.0},
    Algo.NVLS: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 0.0},
    Algo.NVLS_TREE: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 0.0},
}
#: per-step latency over NVLink and over the network, us
NVLINK_LAT = {
    Algo.TREE: {Proto.LL: 0.6, Proto.LL128: 1.25, Proto.SIMPLE: 4.0},
    Algo.RING: {Proto.LL: 0.6, Proto.LL128: 1.9, Proto.SIMPLE: 3.4},
    Algo.COLLNET_DIRECT: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 3.7},
    Algo.COLLNET_CHAIN: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 2.8},
    Algo.NVLS: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 25.0},
    Algo.NVLS_TREE: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 25.0},
}
NET_LAT = {
    Algo.TREE: {Proto.LL: 5.0, Proto.LL128: 8.5, Proto.SIMPLE: 14.0},
    Algo.RING: {Proto.LL: 2.7, Proto.LL128: 4.0, Proto.SIMPLE: 14.0},
    Algo.COLLNET_DIRECT: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 31.0},
    Algo.COLLNET_CHAIN: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 30.0},
    Algo.NVLS: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 18.0},
    Algo.NVLS_TREE: {Proto.LL: 0.0, Proto.LL128: 0.0, Proto.SIMPLE: 14.0},
}
#: ceilings by (architecture, node-count class: 1 node, 2 nodes, 4 or more), GB/s
LL_MAX_BW = {Arch.AMPERE: (87.7, 22.5, 19.0), Arch.HOPPER: (141.0, 45.0, 35.0), Arch.BLACKWELL: (282.0, 90.0, 70.0)}
PER_CH_MAX_TREE_BW = {Arch.AMPERE: (24.0, 23.6, 17.8), Arch.HOPPER: (38.7, 41.4, 36.0), Arch.BLACKWELL: (77.4, 82.8, 72.0)}
PER_CH_MAX_RING_LL128_BW = {Arch.AMPERE: (20.0, 20.0, 20.0), Arch.HOPPER: (36.7, 36.7, 36.7), Arch.BLACKWELL: (73.4, 73.4, 73.4)}
PER_CH_MAX_TREE_LL128_BW = {Arch.AMPERE: (20.0, 20.0, 20.0), Arch.HOPPER: (36.7, 36.7, 29.0), Arch.BLACKWELL: (73.4, 73.4, 58.0)}
NVLS_EFFICIENCY = {Arch.AMPERE: 0.0, Arch.HOPPER: 0.85, Arch.BLACKWELL: 0.74}
DEFAULT_CHANNELS = {Arch.AMPERE: 12, Arch.HOPPER: 16, Arch.BLACKWELL: 32}
#: small-message correction of the Tree prediction: factor by log2(bytes / 64), 0..22 (beyond: 1)
TREE_CORRECTION = {
    Proto.LL: (1.0, 1.0, 1.0, 1.0, 0.9, 0.8, 0.7, 0.7, 0.7, 0.7, 0.6, 0.5, 0.4, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0, 1.0, 1.0, 1.0),
    Proto.LL128: (1.0, 1.0, 1.0, 1.0, 1.0, 0.9, 0.8, 0.8, 0.8, 0.7, 0.6, 0.6, 0.6, 0.6, 0.6, 0.6, 0.8, 0.9, 0.9, 0.9, 0.9, 1.0, 1.0),
    Proto.SIMPLE: (0.9, 0.9, 0.9, 0.9, 0.9, 0.9, 0.9, 0.8, 0.7, 0.6, 0.6, 0.5, 0.5, 0.5, 0.5, 0.6, 0.7, 0.8, 0.7, 0.7, 0.8, 0.9, 0.9),
}


@dataclasses.dataclass(frozen=True)
class DimTopo:
    """What a collective over one mesh dim sees."""

    n_ranks: int
    ppn: int        # ranks of the group that share a node
    n_nodes: int    # nodes the group spans
    n_channels: int
    bw_intra: float  # per-channel NVLink bandwidth, GB/s
    bw_inter: float  # per-channel network bandwidth, GB/s


def derive_mesh_dim_topo(topo: TopoConfig, mesh_shape: Sequence[int], dim: int) -> DimTopo:
    """Ranks are laid out row-major over the mesh: the group of mesh dim ``dim`` strides over the product of
    the inner dims, so ``gpus_per_node // inner`` of its members (at most its size) sit in one node."""
    inner = 1
    for n in mesh_shape[dim + 1:]:
        inner *= n
    n_ranks = mesh_shape[dim]
    ppn = max(1, min(topo.gpus_per_node // inner, n_ranks))
    n_nodes = max(1, n_ranks // ppn)
    ch = topo.n_channels or DEFAULT_CHANNELS[topo.arch]
    return DimTopo(n_ranks, ppn, n_nodes, ch, topo.intra_bw_gbs / ch, topo.inter_bw_gbs / ch)


def _node_class(n_nodes: int) -> int:
    return 0 if n_nodes <= 1 else 1 if n_nodes == 2 else 2


def eligible_algos(coll: Coll, d: DimTopo, topo: TopoConfig) -> list[Algo]:
    out = [Algo.RING]
    if coll is Coll.ALL_REDUCE:
        out.append(Algo.TREE)
    nvls_ok = topo.nvls and topo.nvswitch and NVLS_EFFICIENCY[topo.arch] > 0 and d.ppn > 2
    if nvls_ok and d.n_nodes == 1:
        out.append(Algo.NVLS)
    if nvls_ok and d.n_nodes > 1 and coll is Coll.ALL_REDUCE:
        out.append(Algo.NVLS_TREE)
    if topo.collnet and d.n_nodes > 1 and coll is Coll.ALL_REDUCE:
        out += [Algo.COLLNET_DIRECT, Algo.COLLNET_CHAIN]
    return out


def eligible_protos(algo: Algo) -> list[Proto]:
    return list(_P) if algo in (Algo.RING, Algo.TREE) else [Proto.SIMPLE]


def algo_bus_bw_gbs(coll: Coll, algo: Algo, proto: Proto, d: DimTopo, topo: TopoConfig) -> float:
    """Bus bandwidth (GB/s) as NCCL's tuning model defines it; 0 when the combination does not exist."""
    if proto not in eligible_protos(algo):
        return 0.0
    nc = _node_class(d.n_nodes)
    # ``inter_bw_gbs`` is one GPU's NIC: the ``ppn`` ranks of a node drive ``ppn`` rails, one channel set each
    per_ch = d.bw_intra if d.n_nodes == 1 else min(d.bw_intra, d.bw_inter * d.ppn)
    bw = d.n_channels * per_ch
    n = d.n_ranks
    if algo is Algo.RING:
        if proto is Proto.LL:
            bw = min(LL_MAX_BW[topo.arch][nc], bw * (0.5 if d.n_nodes == 1 else 0.25))
        elif proto is Proto.LL128:
            bw = min(bw * 0.92, d.n_channels * PER_CH_MAX_RING_LL128_BW[topo.arch][nc])
        # bus bandwidth of a ring: every byte crosses (n - 1) / n of the links once (twice for all-reduce)
        return bw * n / (2.0 * (n - 1)) if coll is Coll.ALL_REDUCE else bw * n / (n - 1)
    if algo is Algo.TREE:
        if proto is Proto.LL:
            bw = min(bw / 3.8, LL_MAX_BW[topo.arch][nc])
        elif proto is Proto.LL128:
            bw = min(bw * 0.92 * (7.0 / 9.0 if d.n_nodes == 1 else 120.0 / 128.0), d.n_channels * PER_CH_MAX_TREE_LL128_BW[topo.arch][nc])
        else:
            bw = min(bw * 0.92, d.n_channels * PER_CH_MAX_TREE_BW[topo.arch][nc])
        return bw * 0.5  # data goes up and down the tree
    if algo is Algo.NVLS:
        eff = NVLS_EFFICIENCY[topo.arch]
        # the switch reduces / multicasts: a GPU sends its data once and receives the result once
        return d.n_channels * d.bw_intra * eff * (1.0 if coll is Coll.ALL_REDUCE else n / (n - 1.0))
    if algo is Algo.NVLS_TREE:
        eff = NVLS_EFFICIENCY[topo.arch]
        return min(d.n_channels * d.bw_intra * eff, d.n_channels * d.bw_inter * d.ppn * 0.5)
    if algo is Algo.COLLNET_DIRECT:
        return min(d.n_channels * d.bw_intra, d.n_channels * d.bw_inter * d.ppn) * 0.5
    if algo is Algo.COLLNET_CHAIN:
        return min(d.n_channels * d.bw_intra, d.n_channels * d.bw_inter * d.ppn) * 0.5
    return 0.0


def algo_latency_us(coll: Coll, algo: Algo, proto: Proto, d: DimTopo, topo: TopoConfig) -> float:
    base = BASE_LAT[algo][proto]
    intra, net = NVLINK_LAT[algo][proto], NET_LAT[algo][proto]
    n = d.n_ranks
    if algo is Algo.RING:
        steps = 2 * (n - 1) if coll is Coll.ALL_REDUCE else n - 1
        net_steps = 0
        if d.n_nodes > 1:
            net_steps = (2 * (d.n_nodes - 1) if coll is Coll.ALL_REDUCE else d.n_nodes - 1)
            if proto is Proto.SIMPLE and coll is Coll.ALL_REDUCE:
                net = net * 1.0  # (NCCL doubles this for plugins without GPUDirect; assumed present)
        return base + (steps - net_steps) * intra + net_steps * net
    if algo is Algo.TREE:
        return base + 2.0 * ((d.ppn - 1) * intra + _log2i(d.n_nodes) * net)
    if algo is Algo.NVLS:
        return base + intra
    if algo is Algo.NVLS_TREE:
        return base + intra + 2.0 * _log2i(d.n_nodes) * net
    if algo is Algo.COLLNET_DIRECT:
        return base + 2.0 * (min(1, d.ppn - 1) * intra + (d.ppn - 1) * 0.4) + net
    if algo is Algo.COLLNET_CHAIN:
        return base + 2.0 * (d.ppn - 1) * intra + net
    return math.inf


def _log2i(n: int) -> int:
    return max(0, int(n).bit_length() - 1)


# ------------------------------------------------------------------------------------- empirical layer
#: measured / predicted ratio of multi-node rings by message size (bytes -> factor); small messages are
#: slower than the per-step model says because every step also synchronises through the proxy thread
RING_CORRECTION = ((1 << 12, 1.9), (1 << 16, 1.7), (1 << 20, 1.4), (1 << 24, 1.15), (1 << 28, 1.0))
RING_DEPTH_REFERENCE_NODES = 2      # node count the correction table was fitted at
RING_PLATEAU_BYTES = 1 << 22        # below this a multi-node Simple ring costs about the same
PER_NODE_SYNC_US = 1.5              # proxy / flush overhead per extra node
#: copy-engine all-to-all inside a node: bandwidth (GB/s) and start-up (us)
A2A_CE_BW = {Arch.AMPERE: 120.0, Arch.HOPPER: 380.0, Arch.BLACKWELL: 640.0}
A2A_CE_LAT = {Arch.AMPERE: 60.0, Arch.HOPPER: 50.0, Arch.BLACKWELL: 25.0}
#: multi-node all-to-all start-up by node count (us), NIC efficiency once ramped and bytes at half efficiency
A2A_MULTI_NODE_LAT = ((2, 37.0), (4, 42.0), (8, 60.0), (16, 98.0), (32, 290.0))
A2A_NIC_EFFICIENCY = 0.85
A2A_NIC_RAMP_BYTES = 1 << 20


def interp_log(points: Sequence[tuple], x: float) -> float:
    """Piecewise-linear in log2(x) through ``points`` ((x, y), ascending), clamped at both ends."""
    if x <= points[0][0]:
        return points[0][1]
    if x >= points[-1][0]:
        return points[-1][1]
    for (x0, y0), (x1, y1) in zip(points, points[1:]):
        if x0 <= x <= x1:
            w = (math.log2(x) - math.log2(x0)) / (math.log2(x1) - math.log2(x0))
            return y0 + w * (y1 - y0)
    return points[-1][1]


def ring_correction(nbytes: float, n_nodes: int) -> float:
    """Factor on a multi-node ring's predicted time: the fitted table, with the excess over 1 growing with
    the ring's depth (log2 of the node count relative to the fit)."""
    if n_nodes <= 1:
        return 1.0
    base = interp_log(RING_CORRECTION, max(nbytes, 1.0))
    depth = max(1.0, math.log2(n_nodes) / math.log2(RING_DEPTH_REFERENCE_NODES))
    return 1.0 + (base - 1.0) * depth


def tree_correction(proto: Proto, nbytes: float) -> float:
    idx = _log2i(max(int(nbytes), 64) >> 6)
    table = TREE_CORRECTION[proto]
    return table[idx] if idx < len(table) else 1.0


def algo_time_us(coll: Coll, algo: Algo, proto: Proto, nbytes: float, d: DimTopo, topo: TopoConfig) -> float:
    """``nbytes``: all-gather - gathered size; reduce-scatter - input size; all-reduce - tensor size."""
    if d.n_ranks <= 1 or nbytes <= 0:
        return 0.0
    bw = algo_bus_bw_gbs(coll, algo, proto, d, topo)
    if bw <= 0:
        return math.inf
    if algo is Algo.TREE and coll is Coll.ALL_REDUCE:
        bw *= tree_correction(proto, nbytes)
    lat = algo_latency_us(coll, algo, proto, d, topo)
    size = nbytes
    if algo is Algo.RING and d.n_nodes > 1:
        def corrected(b: float) -> float:
            sz = max(b, float(RING_PLATEAU_BYTES)) if proto is Proto.SIMPLE else b  # chunking: the pipeline never gets shorter
            return (lat + sz / (bw * 1e3)) * ring_correction(b, d.n_nodes)

        # the correction falls with size faster than the transfer term grows between some knots: a larger message
        # is never priced below a smaller one
        t = max([corrected(nbytes)] + [corrected(float(k)) for k, _ in RING_CORRECTION if k < nbytes])
    else:
        t = lat + size / (bw * 1e3)
    return t + PER_NODE_SYNC_US * (d.n_nodes - 1)


def best_time_us(coll: Coll, nbytes: float, d: DimTopo, topo: TopoConfig) -> tuple[float, Optional[Algo], Optional[Proto]]:
    best = (math.inf, None, None)
    for algo in eligible_algos(coll, d, topo):
        for proto in eligible_protos(algo):
            t = algo_time_us(coll, algo, proto, nbytes, d, topo)
            if t < best[0]:
                best = (t, algo, proto)
    return best


def all_to_all_us(nbytes_local: float, d: DimTopo, topo: TopoConfig) -> float:
    """``nbytes_local``: bytes one rank holds before the exchange."""
    n = d.n_ranks
    if n <= 1 or nbytes_local <= 0:
        return 0.0
    if d.n_nodes == 1:
        return A2A_CE_LAT[topo.arch] + nbytes_local * (n - 1) / n / (A2A_CE_BW[topo.arch] * 1e3)
    off_node = nbytes_local * (n - d.ppn) / n
    on_node = nbytes_local * (d.ppn - 1) / n
    nic = topo.inter_bw_gbs * A2A_NIC_EFFICIENCY * off_node / (off_node + A2A_NIC_RAMP_BYTES)  # ramps up with size
    lat = interp_log(A2A_MULTI_NODE_LAT, d.n_nodes)
    return lat + max(off_node / (max(nic, 1e-6) * 1e3), on_node / (A2A_CE_BW[topo.arch] * 1e3))


def arch_from_device_name(name: str) -> Optional[Arch]:
    """Architecture generation from ``torch.cuda.get_device_name`` (None for devices this model has no numbers for)."""
    n = name.upper()
    if any(k in n for k in ("GB200", "GB300", "B200", "B100", "B300")):
        return Arch.BLACKWELL
    if any(k in n for k in ("H100", "H200", "H800", "GH200")):
        return Arch.HOPPER
    if any(k in n for k in ("A100", "A800")):
        return Arch.AMPERE
    return None
