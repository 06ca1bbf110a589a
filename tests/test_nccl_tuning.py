"""The per-algorithm / per-protocol NCCL model: mesh-dim topology, bandwidth and latency formulas, eligibility,
corrections, all-to-all and device detection.  (Reference: tests/test_nccl_cost_model.py.)"""
import dataclasses
import math

import pytest

from autoparallel_b200.parallel.cost import nccl_model as M
from autoparallel_b200.parallel.cost import nccl_tuning as T

AR, AG, RS = M.Coll.ALL_REDUCE, M.Coll.ALL_GATHER, M.Coll.REDUCE_SCATTER
RING, TREE, NVLS, NVLS_TREE = M.Algo.RING, M.Algo.TREE, M.Algo.NVLS, M.Algo.NVLS_TREE
LL, LL128, SIMPLE = M.Proto.LL, M.Proto.LL128, M.Proto.SIMPLE


def dim(topo, shape=None, d=0):
    return T.derive_mesh_dim_topo(topo, shape or (topo.n_nodes * topo.gpus_per_node,), d)


# ---------------------------------------------------------------------------- mesh dim -> ranks, nodes, channels
def test_mesh_dims_map_to_ranks_per_node_and_nodes():
    one = dim(M.a100_topo())
    assert (one.n_ranks, one.ppn, one.n_nodes, one.n_channels) == (8, 8, 1, 12)
    two = M.a100_topo(2)
    inner, outer = dim(two, (2, 8), 1), dim(two, (2, 8), 0)
    assert (inner.n_ranks, inner.ppn, inner.n_nodes) == (8, 8, 1)
    assert (outer.n_ranks, outer.ppn, outer.n_nodes) == (2, 1, 2)
    h = dataclasses.replace(M.h100_topo(4), n_channels=16)
    d2, d1, d0 = (dim(h, (2, 4, 4), i) for i in (2, 1, 0))
    assert (d2.ppn, d2.n_nodes) == (4, 1) and (d1.ppn, d1.n_nodes) == (2, 2) and (d0.ppn, d0.n_nodes) == (1, 2)
    assert d2.bw_intra == pytest.approx(320.0 / 16) and d2.bw_inter == pytest.approx(50.0 / 16)
    assert dim(dataclasses.replace(M.a100_topo(), n_channels=8)).n_channels == 8


# ---------------------------------------------------------------------------- bandwidth and latency formulas
def test_ring_and_tree_bandwidth_formulas():
    topo = M.a100_topo()
    d = dim(topo)
    link = topo.intra_bw_gbs
    assert T.algo_bus_bw_gbs(AR, RING, SIMPLE, d, topo) == pytest.approx(link * 8 / (2 * 7))
    assert T.algo_bus_bw_gbs(AG, RING, SIMPLE, d, topo) == pytest.approx(link * 8 / 7)
    capped = min(link * 0.92, 12 * T.PER_CH_MAX_TREE_BW[M.Arch.AMPERE][0])
    assert T.algo_bus_bw_gbs(AR, TREE, SIMPLE, d, topo) == pytest.approx(capped * 0.5)
    # protocols: LL is capped by the architecture's LL ceiling, LL128 by the per-channel ceiling; both below Simple
    assert T.algo_bus_bw_gbs(AR, RING, LL, d, topo) <= T.LL_MAX_BW[M.Arch.AMPERE][0] * 8 / 14 + 1e-9
    assert T.algo_bus_bw_gbs(AR, RING, LL128, d, topo) <= 12 * T.PER_CH_MAX_RING_LL128_BW[M.Arch.AMPERE][0] * 8 / 14 + 1e-9
    assert T.algo_bus_bw_gbs(AR, TREE, LL, d, topo) < 0.5 * T.algo_bus_bw_gbs(AR, TREE, SIMPLE, d, topo)
    assert T.algo_bus_bw_gbs(AR, NVLS, LL, dim(M.h100_topo()), M.h100_topo()) == 0.0  # NVLS: Simple only


def test_nvls_bandwidth_by_architecture():
    h, a = M.h100_topo(), M.a100_topo()
    assert T.algo_bus_bw_gbs(AR, NVLS, SIMPLE, dim(h), h) == pytest.approx(320.0 * T.NVLS_EFFICIENCY[M.Arch.HOPPER])
    assert T.algo_bus_bw_gbs(AR, NVLS, SIMPLE, dim(a), a) == 0.0


def test_latency_formulas():
    topo = M.h100_topo()
    d = dim(topo)
    ring = T.BASE_LAT[RING][SIMPLE] + 14 * T.NVLINK_LAT[RING][SIMPLE]
    assert T.algo_latency_us(AR, RING, SIMPLE, d, topo) == pytest.approx(ring)
    assert T.algo_latency_us(AG, RING, SIMPLE, d, topo) == pytest.approx(T.BASE_LAT[RING][SIMPLE] + 7 * T.NVLINK_LAT[RING][SIMPLE])
    assert T.algo_latency_us(AR, TREE, SIMPLE, d, topo) == pytest.approx(T.BASE_LAT[TREE][SIMPLE] + 2 * 7 * T.NVLINK_LAT[TREE][SIMPLE])
    assert T.algo_latency_us(AR, RING, LL, d, topo) < T.algo_latency_us(AR, RING, SIMPLE, d, topo)
    four = M.h100_topo(4)
    d4 = dim(four)
    multi = T.algo_latency_us(AR, RING, SIMPLE, d4, four)
    assert multi == pytest.approx(T.BASE_LAT[RING][SIMPLE] + (62 - 6) * T.NVLINK_LAT[RING][SIMPLE] + 6 * T.NET_LAT[RING][SIMPLE])
    assert T.algo_latency_us(AR, TREE, SIMPLE, d4, four) == pytest.approx(
        T.BASE_LAT[TREE][SIMPLE] + 2 * (7 * T.NVLINK_LAT[TREE][SIMPLE] + 2 * T.NET_LAT[TREE][SIMPLE])
    )
    assert T.algo_latency_us(AR, RING, LL, d4, four) < multi  # LL's network step is cheaper too


# ---------------------------------------------------------------------------- eligibility
def test_algorithm_and_protocol_eligibility():
    h1, h4, a1 = M.h100_topo(), M.h100_topo(4), M.a100_topo()
    assert set(T.eligible_algos(AG, dim(h1), h1)) == {RING, NVLS}           # no trees for all-gather
    assert set(T.eligible_algos(RS, dim(h1), h1)) == {RING, NVLS}
    assert set(T.eligible_algos(AR, dim(h1), h1)) == {RING, TREE, NVLS}
    assert set(T.eligible_algos(AR, dim(h4), h4)) == {RING, TREE, NVLS_TREE}  # NVLS-Tree needs several nodes
    assert set(T.eligible_algos(AR, dim(a1), a1)) == {RING, TREE}           # Ampere has no NVLS
    no_switch = dataclasses.replace(h1, nvswitch=False)
    assert NVLS not in T.eligible_algos(AR, dim(no_switch), no_switch)
    sharp = dataclasses.replace(h4, collnet=True)
    assert {M.Algo.COLLNET_DIRECT, M.Algo.COLLNET_CHAIN} <= set(T.eligible_algos(AR, dim(sharp), sharp))
    assert M.Algo.COLLNET_DIRECT not in T.eligible_algos(AR, dim(h4), h4)
    assert M.Algo.COLLNET_DIRECT not in T.eligible_algos(AG, dim(sharp), sharp)
    assert T.eligible_protos(RING) == [LL, LL128, SIMPLE] and T.eligible_protos(TREE) == [LL, LL128, SIMPLE]
    for algo in (NVLS, NVLS_TREE, M.Algo.COLLNET_DIRECT, M.Algo.COLLNET_CHAIN):
        assert T.eligible_protos(algo) == [SIMPLE]


def test_which_algorithm_wins():
    h1, h4 = M.h100_topo(), M.h100_topo(4)
    assert T.best_time_us(AR, 1 << 28, dim(h1), h1)[1] is NVLS                  # large, one NVSwitch node
    assert T.best_time_us(AR, 1 << 10, dim(h1), h1)[2] is LL                    # tiny: a low-latency protocol
    t, algo, _ = T.best_time_us(AR, 1 << 26, dim(h4), h4)
    assert algo in (TREE, NVLS_TREE)                                            # log-depth beats a 32-rank ring
    assert t < T.algo_time_us(AR, RING, SIMPLE, 1 << 26, dim(h4), h4)


# ---------------------------------------------------------------------------- corrections
def test_tree_and_ring_corrections():
    assert T.tree_correction(SIMPLE, 64) == 0.9 and T.tree_correction(SIMPLE, 64 << 11) == 0.5
    assert T.tree_correction(LL, 1 << 40) == 1.0                                # beyond the table
    assert T.ring_correction(1 << 20, 1) == 1.0                                 # single node: untouched
    base = T.ring_correction(1 << 20, 2)
    assert base == pytest.approx(1.4) and T.ring_correction(1 << 30, 2) == 1.0  # large messages: no effect
    assert T.ring_correction(1 << 20, 8) == pytest.approx(1.0 + 0.4 * 3)        # deeper rings: excess x log2(nodes)
    assert T.interp_log(T.RING_CORRECTION, 1 << 14) == pytest.approx((1.9 + 1.7) / 2)
    h1, h4 = M.h100_topo(), M.h100_topo(4)
    # plateau: below the pipeline's chunk size a multi-node Simple ring costs the same; other protocols / one node do not
    sync = T.PER_NODE_SYNC_US * 3

    def uncorrected(nbytes):
        return (T.algo_time_us(AG, RING, SIMPLE, nbytes, dim(h4), h4) - sync) / T.ring_correction(nbytes, 4)

    assert uncorrected(1 << 10) == pytest.approx(uncorrected(1 << 12), rel=1e-9)
    assert T.algo_time_us(AG, RING, LL, 1 << 14, dim(h4), h4) < T.algo_time_us(AG, RING, LL, 1 << 22, dim(h4), h4)
    assert T.algo_time_us(AG, RING, SIMPLE, 1 << 14, dim(h1), h1) < T.algo_time_us(AG, RING, SIMPLE, 1 << 20, dim(h1), h1)


# ---------------------------------------------------------------------------- end-to-end properties
@pytest.mark.parametrize("make", [M.a100_topo, M.h100_topo, M.b200_topo])
@pytest.mark.parametrize("nodes", [1, 2, 8])
def test_costs_are_positive_finite_and_monotone(make, nodes):
    topo = make(nodes)
    d = dim(topo)
    for coll in (AR, AG, RS):
        times = [T.best_time_us(coll, 1 << s, d, topo)[0] for s in range(10, 31, 2)]
        assert all(0 < t < math.inf for t in times)
        assert all(a <= b * (1 + 1e-9) for a, b in zip(times, times[1:])), (coll, times)
    a2a = [T.all_to_all_us(1 << s, d, topo) for s in range(12, 31, 2)]
    assert all(0 < t < math.inf for t in a2a) and all(a < b for a, b in zip(a2a, a2a[1:]))
    if nodes == 1:  # (across many nodes a log-depth all-reduce can beat a 64-step ring reduce-scatter)
        assert T.best_time_us(AR, 1 << 26, d, topo)[0] > T.best_time_us(RS, 1 << 26, d, topo)[0]


def test_multi_node_scaling():
    lat = [T.all_to_all_us(1 << 10, dim(M.h100_topo(n)), M.h100_topo(n)) for n in (2, 4, 8, 16, 32)]
    assert all(a < b for a, b in zip(lat, lat[1:])) and lat[-1] < 16 * lat[0]       # grows, but sublinearly
    slow, fast = dataclasses.replace(M.h100_topo(4), inter_bw_gbs=10.0), dataclasses.replace(M.h100_topo(4), inter_bw_gbs=20.0)
    big = 1 << 30
    assert T.all_to_all_us(big, dim(fast), fast) < 0.6 * T.all_to_all_us(big, dim(slow), slow)  # NIC bound
    assert T.best_time_us(AG, big, dim(fast), fast)[0] < 0.6 * T.best_time_us(AG, big, dim(slow), slow)[0]
    # Blackwell's NVLink is twice Hopper's: intra-node ceilings double
    for table in (T.LL_MAX_BW, T.PER_CH_MAX_TREE_BW, T.PER_CH_MAX_RING_LL128_BW):
        assert all(b == pytest.approx(2 * h) for b, h in zip(table[M.Arch.BLACKWELL], table[M.Arch.HOPPER]))


def test_device_names():
    names = {"NVIDIA A100-SXM4-80GB": M.Arch.AMPERE, "NVIDIA H100 80GB HBM3": M.Arch.HOPPER, "NVIDIA H200": M.Arch.HOPPER,
             "NVIDIA B200": M.Arch.BLACKWELL, "NVIDIA GB200": M.Arch.BLACKWELL}
    for name, arch in names.items():
        assert T.arch_from_device_name(name) is arch
    assert T.arch_from_device_name("Tesla T4") is None
    # an 8-GPU B200 host is one NVSwitch node of 8, whatever the name suggests about racks
    d = M.detect_topology(8, device_name="NVIDIA B200")
    assert (d.gpus_per_node, d.n_nodes) == (8, 1)


def test_planning_with_the_nccl_cost_model_across_two_nodes():
    """cost_model="nccl" on a 2 x 8 mesh: the outer dim crosses nodes, so parameters are sharded over the inner
    (NVSwitch) dim first and nothing large is gathered over the network."""
    import torch
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor.placement_types import Replicate, Shard
    from torch.testing._internal.distributed.fake_pg import FakeStore

    from autoparallel_b200 import AutoParallel
    from autoparallel_b200.parallel.cost import comm

    if dist.is_initialized():
        dist.destroy_process_group()
    dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=16)
    try:
        mesh = init_device_mesh("cpu", (2, 8), mesh_dim_names=("dp", "tp"))
        with torch.device("meta"):
            model = torch.nn.Sequential(torch.nn.Linear(1024, 4096, bias=False), torch.nn.ReLU(), torch.nn.Linear(4096, 1024, bias=False))
        with AutoParallel(model, lambda: torch.rand(64, 1024), mesh, cost_model="nccl", plan_device="B200") as ap:
            topo = comm.get_topology(mesh)
            assert isinstance(topo, comm.NcclTopology)
            assert (topo.dims[0].n_nodes, topo.dims[0].ppn, topo.dims[1].n_nodes, topo.dims[1].ppn) == (2, 1, 1, 8)
            big = 1 << 26
            assert topo.all_gather(0, 2, big) > 2 * topo.all_gather(1, 8, big)  # the network dim is the slow one
            ap.add_parameter_memory_constraint()
            ap.add_input_constraints([(Shard(0), Replicate())])
            sol = ap.optimize_placement()
            for node in ap.joint.param_nodes.values():
                placements = sol[node].output_spec.placements
                assert isinstance(placements[1], Shard), placements
    finally:
        dist.destroy_process_group()
        dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=8)  # what the session fixture set up
