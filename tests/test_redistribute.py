"""Ordering of per-mesh-dim collectives for one placement change."""
import pytest
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200.parallel.lower.redistribute import RedistributeError, plan_redistribution

R, P = Replicate(), Partial()


def S(d):
    return Shard(d)


def kinds(steps):
    return [(s.kind, s.mesh_dim) for s in steps]


def test_identity_is_empty():
    assert plan_redistribution((S(0), R), (S(0), R), (2, 4)) == []


def test_single_dim_transitions():
    assert kinds(plan_redistribution((S(0),), (R,), (8,))) == [("all_gather", 0)]
    assert kinds(plan_redistribution((P,), (R,), (8,))) == [("all_reduce", 0)]
    assert kinds(plan_redistribution((P,), (S(1),), (8,))) == [("reduce_scatter", 0)]
    assert kinds(plan_redistribution((R,), (S(0),), (8,))) == [("local_chunk", 0)]
    st = plan_redistribution((S(0),), (S(1),), (8,))
    assert kinds(st) == [("all_to_all", 0)] and st[0].dim == 1 and st[0].dim2 == 0


def test_nested_shards_gather_inner_first_and_split_outer_first():
    assert kinds(plan_redistribution((S(0), S(0)), (R, R), (2, 4))) == [("all_gather", 1), ("all_gather", 0)]
    assert kinds(plan_redistribution((R, R), (S(0), S(0)), (2, 4))) == [("local_chunk", 0), ("local_chunk", 1)]
    assert kinds(plan_redistribution((P, P), (S(0), S(0)), (2, 4))) == [("reduce_scatter", 0), ("reduce_scatter", 1)]


def test_outer_change_under_inner_shard_regathers_inner():
    # (S0, S0) -> (R, S0): the inner shard must be undone first so chunks stay contiguous
    assert kinds(plan_redistribution((S(0), S(0)), (R, S(0)), (2, 4))) == [
        ("all_gather", 1), ("all_gather", 0), ("local_chunk", 1)]


def test_creating_partial_is_refused():
    with pytest.raises(RedistributeError):
        plan_redistribution((R,), (P,), (8,))
    with pytest.raises(RedistributeError):
        plan_redistribution((S(0),), (P,), (8,))


def test_size_one_mesh_dims_are_free():
    assert plan_redistribution((S(0), R), (R, R), (1, 4)) == []


def test_renested_shards_change_the_outer_mesh_dim_with_one_collective():
    # tp outer / dp inner: gathering over dp alone returns the contiguous tp chunk
    assert kinds(plan_redistribution((S(0), S(0)), (R, S(0)), (2, 4), order=(1, 0))) == [("all_gather", 0)]
    assert kinds(plan_redistribution((P, S(0)), (S(0), S(0)), (2, 4), order=(1, 0))) == [("reduce_scatter", 0)]
    # the default order is unchanged by passing it explicitly
    assert plan_redistribution((S(0), S(0)), (R, S(0)), (2, 4), order=(0, 1)) == plan_redistribution((S(0), S(0)), (R, S(0)), (2, 4))


def test_whole_mesh_runs_become_one_collective_on_the_flattened_mesh():
    from autoparallel_b200.parallel.lower.redistribute import FLAT, fuse_over_flat_mesh

    ag = fuse_over_flat_mesh(plan_redistribution((S(0), S(0)), (R, R), (2, 4)), 2)
    assert kinds(ag) == [("all_gather", FLAT)] and ag[0].dim == 0
    rs = fuse_over_flat_mesh(plan_redistribution((P, P), (S(1), S(1)), (2, 4)), 2)
    assert kinds(rs) == [("reduce_scatter", FLAT)] and rs[0].dim == 1
    # different tensor dims, partial coverage or a re-nested order are left alone
    for src, dst, order in (((S(0), S(1)), (R, R), None), ((S(0), S(0)), (R, S(0)), None), ((S(0), S(0)), (R, R), (1, 0))):
        steps = plan_redistribution(src, dst, (2, 4), order=order)
        assert fuse_over_flat_mesh(steps, 2, order) == steps


def test_local_shard_follows_the_nesting_order():
    import torch

    from autoparallel_b200.parallel.lower.ordered import local_shard

    full = torch.arange(8.0).view(8, 1)
    got = {(i, j): local_shard(full, (S(0), S(0)), (i, j), (2, 2), order).flatten().tolist()
           for order in (None,) for i in range(2) for j in range(2)}
    assert got == {(0, 0): [0.0, 1.0], (0, 1): [2.0, 3.0], (1, 0): [4.0, 5.0], (1, 1): [6.0, 7.0]}
    got = {(i, j): local_shard(full, (S(0), S(0)), (i, j), (2, 2), (1, 0)).flatten().tolist() for i in range(2) for j in range(2)}
    assert got == {(0, 0): [0.0, 1.0], (1, 0): [2.0, 3.0], (0, 1): [4.0, 5.0], (1, 1): [6.0, 7.0]}
