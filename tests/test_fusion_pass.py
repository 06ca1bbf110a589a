"""Collective-fusion pass: pattern coverage and exact shapes of the fused nodes (CPU, fake ranks)."""
import torch
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel, ForwardInputs
from autoparallel_b200.models import llama3
from autoparallel_b200.parallel.frontend.mp_cast import MPPolicy
from autoparallel_b200.runtime import comm_ops


def _lower(mesh, batch, fuse=True):
    cfg = llama3.llama3_debug(n_layers=2, dim=512, n_heads=8, n_kv_heads=4, ffn_hidden=2048, vocab_size=4096, max_seq_len=512)
    with torch.device("meta"):
        model = llama3.Transformer(cfg)

    def input_fn():
        return ForwardInputs((torch.randint(0, cfg.vocab_size, (batch, 512)),), {"labels": torch.randint(0, cfg.vocab_size, (batch, 512))})

    with AutoParallel(model, input_fn, mesh, MPPolicy(torch.bfloat16, torch.float32), plan_device="B200", fuse_collectives=fuse) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)] * 2)
        ap.optimize_placement()
        return ap, ap.lower()


def test_fused_nodes_replace_gather_and_scatter_next_to_gemms(mesh_1d):
    ap, low = _lower(mesh_1d, batch=8)
    assert ap.fusion_stats["ag_mm"] > 0
    targets = [n.target for n in low.gm.graph.nodes if n.op == "call_function"]
    assert comm_ops.ops.ag_mm.default in targets
    assert (comm_ops.ops.mm_rs.default in targets) == (ap.fusion_stats["mm_rs"] > 0)
    # weight-gradient GEMMs reduce-scatter in their epilogue, in the fp32 the policy asks for
    for n in low.gm.graph.nodes:
        if n.op == "call_function" and n.target is comm_ops.ops.mm_rs.default and n.args[2] == 2:
            assert n.args[4] == torch.float32


def test_fused_meta_shapes_match_unfused_graph(mesh_1d):
    """Local batch of one sequence: the gathered dim has extent 1 before the gather, which is the
    case where the gather dim must be carried explicitly."""
    ap, low = _lower(mesh_1d, batch=8)
    for n in low.gm.graph.nodes:
        if n.op != "call_function" or n.target not in comm_ops.FUSED_OPS:
            continue
        fake_args = [a.meta["val"] if isinstance(a, torch.fx.Node) else a for a in n.args]
        with torch.device("meta"):
            metas = [torch.empty(a.shape, dtype=a.dtype, device="meta") if isinstance(a, torch.Tensor) else a for a in fake_args]
        out = n.target(*metas)
        want = n.meta["val"]
        if isinstance(out, tuple):
            assert tuple(out[0].shape) == tuple(want[0].shape) and tuple(out[1].shape) == tuple(want[1].shape)
        else:
            assert tuple(out.shape) == tuple(want.shape)
