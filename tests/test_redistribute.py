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
