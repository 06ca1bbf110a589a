"""Strategy enumeration: framework rules, view mapping, filtering."""
import torch
from torch.distributed.tensor.placement_types import Partial, Replicate, Shard

from autoparallel_b200.parallel.strategies import rules
from autoparallel_b200.parallel.strategies.dtensor_adapter import all_options, local_shape


def _pl(strategy):
    return [tuple(s.output_spec.placements) for s in strategy.strategies]


def test_all_options_respects_divisibility(mesh_1d, mesh_2d):
    t = torch.empty(16, 4, 8)
    opts = _pl(all_options(mesh_1d, t))
    assert (Replicate(),) in opts and (Shard(0),) in opts and (Shard(2),) in opts
    assert (Shard(1),) not in opts  # 4 < 8 ranks
    opts2 = _pl(all_options(mesh_2d, t))
    assert (Shard(0), Shard(0)) in opts2 and (Shard(1), Shard(1)) not in opts2
    assert (Shard(1), Replicate()) in opts2  # 4 >= 2 on dp
    # uneven shards only when asked for
    assert (Shard(0),) not in _pl(all_options(mesh_1d, torch.empty(15, 3)))
    assert (Shard(0),) in _pl(all_options(mesh_1d, torch.empty(15, 3), even_only=False))       # 2, 2, 2, 2, 2, 2, 2, 1
    assert (Shard(0),) not in _pl(all_options(mesh_1d, torch.empty(12, 3), even_only=False))   # 2 x 6, then two empty ranks


def test_local_shape():
    assert local_shape([16, 8], (2, 4), (Shard(0), Shard(0))) == [2, 8]
    assert local_shape([16, 8], (2, 4), (Shard(0), Shard(1))) == [8, 2]
    assert local_shape([1, 8], (2, 4), (Shard(0), Replicate())) is None


def test_view_placement_map():
    vm = rules.view_placement_map
    # split of the sharded dim: shard follows the leading factor
    assert vm([8, 64, 256], [8, 64, 8, 32], (8,), (Shard(2),)) == (Shard(2),)
    # merge of leading dims keeps a shard of the outermost one
    assert vm([8, 64, 256], [512, 256], (8,), (Shard(0),)) == (Shard(0),)
    # the inner merged dim cannot stay sharded
    assert vm([8, 64, 256], [512, 256], (8,), (Shard(1),)) is None
    # untouched dims pass through, partial passes through
    assert vm([8, 64, 256], [512, 256], (8,), (Shard(2),)) == (Shard(1),)
    assert vm([8, 64, 256], [512, 256], (8,), (Partial(),)) == (Partial(),)
    # two mesh dims on the same tensor dim need both factors to divide
    assert vm([8, 64], [8, 8, 8], (2, 4), (Shard(1), Shard(1))) == (Shard(1), Shard(1))
    assert vm([8, 64], [8, 4, 16], (2, 4), (Shard(1), Shard(1))) is None


def _ctx(mesh, op, args, in_vals, out_val):
    in_strats = [all_options(mesh, v) for v in in_vals]
    return rules.RuleCtx(mesh, op, args, {}, in_vals, in_strats, out_val, True)


def test_mm_nd_rule_enumerates_row_col_and_contraction_sharding(mesh_1d):
    a, b = torch.empty(8, 64, 32), torch.empty(16, 32)
    out = torch.empty(8, 64, 16)
    st = rules.get_rule(torch.ops.apb200.mm_nd.default)(_ctx(mesh_1d, torch.ops.apb200.mm_nd.default, (None, None, True, torch.float32), [a, b], out))
    combos = {(tuple(s.output_specs.placements), tuple(s.input_specs[0].placements), tuple(s.input_specs[1].placements)) for s in st.strategies}
    assert ((Shard(0),), (Shard(0),), (Replicate(),)) in combos          # data parallel
    assert ((Shard(1),), (Shard(1),), (Replicate(),)) in combos          # sequence parallel
    assert ((Shard(2),), (Replicate(),), (Shard(0),)) in combos          # column parallel
    assert ((Partial(),), (Shard(2),), (Shard(1),)) in combos            # row parallel
    assert ((Replicate(),), (Replicate(),), (Replicate(),)) in combos


def test_mm_wgrad_rule(mesh_1d):
    a, b = torch.empty(8, 64, 16), torch.empty(8, 64, 32)
    out = torch.empty(16, 32)
    st = rules.get_rule(torch.ops.apb200.mm_wgrad.default)(_ctx(mesh_1d, torch.ops.apb200.mm_wgrad.default, (None, None, torch.float32), [a, b], out))
    combos = {(tuple(s.output_specs.placements), tuple(s.input_specs[0].placements)) for s in st.strategies}
    assert ((Partial(),), (Shard(0),)) in combos  # batch-sharded activations -> pending gradient sum
    assert ((Shard(0),), (Shard(2),)) in combos


def test_attention_rule_is_batch_or_head_parallel(mesh_1d):
    q, k = torch.empty(8, 64, 16, 32), torch.empty(8, 64, 8, 32)
    o, lse = torch.empty(8, 64, 16, 32), torch.empty(8, 16, 64)
    op = torch.ops.apb200.attention.default
    st = rules.get_rule(op)(_ctx(mesh_1d, op, (None, None, None, True, 0.1), [q, k, k], (o, lse)))
    outs = {tuple(s.output_specs[0].placements) for s in st.strategies}
    assert outs == {(Replicate(),), (Shard(0),), (Shard(2),)}
    for s in st.strategies:
        if s.output_specs[0].placements == (Shard(2),):
            assert s.output_specs[1].placements == (Shard(1),)  # lse is [B, H, S]


def test_rms_norm_never_shards_the_normalised_dim(mesh_1d):
    x, w = torch.empty(8, 64, 256), torch.empty(256)
    op = torch.ops.apb200.rms_norm.default
    st = rules.get_rule(op)(_ctx(mesh_1d, op, (None, None, 1e-5), [x, w], (x, torch.empty(8, 64))))
    for s in st.strategies:
        assert s.output_specs[0].placements != (Shard(2),)
        assert s.input_specs[1].placements == (Replicate(),)
