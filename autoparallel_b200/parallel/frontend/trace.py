"""Joint forward+backward graph capture on fake tensors.

``build_joint_graph`` turns a meta-device ``nn.Module`` plus an ``input_fn`` describing the
*global* inputs into one ATen-level FX graph that computes the forward outputs and the
gradients of every parameter, together with an index of which placeholder / output is
which (parameter, buffer, user input, tangent; forward output, gradient).  Reference call
stack: autoparallel/api.py:157-228 and autoparallel/tracing.py:14-137.

The capture itself uses the same upstream entry points as the reference (Dynamo functional
export + AOTAutograd joint export); everything downstream of the captured graph – partitioning,
execution, scheduling – is this framework's own, so the AOT ``ExitStack`` is closed as soon as
the graph is in hand.
"""
from __future__ import annotations

import contextlib
import copy
import dataclasses
import logging
import time
from typing import Any, Callable, Optional

import torch
import torch.fx as fx
import torch.nn as nn
from torch._subclasses import FakeTensorMode

from .mp_cast import cast_reads

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class ForwardInputs:
    """Positional and keyword inputs of ``model.forward`` (reference: input_validation.py:13-24)."""

    args: tuple = ()
    kwargs: dict = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class JointGraph:
    gm: fx.GraphModule
    #: fqn -> placeholder node
    param_nodes: dict[str, fx.Node]
    buffer_nodes: dict[str, fx.Node]
    #: user inputs in flat (tree_flatten((args, kwargs))) order; None where the leaf is not a graph input
    input_nodes: list[Optional[fx.Node]]
    tangent_nodes: list[fx.Node]
    #: forward outputs in flat order (fx.Node or constant)
    fwd_outputs: list[Any]
    #: fqn -> gradient node (None when the parameter gets no gradient)
    param_grads: dict[str, Optional[fx.Node]]
    input_grads: list[Optional[fx.Node]]
    out_spec: Any  # pytree spec of the user-visible forward output
    traced_inputs: ForwardInputs
    #: number of forward outputs at the head of the output tuple
    num_fwd_outputs: int = 0
    #: buffers the forward mutates in place (batch-norm statistics, counters): fqn -> node of the new value.  The new
    #: values ride at the END of ``fwd_outputs`` (after the ``num_user_outputs`` values the caller sees).
    buffer_updates: dict = dataclasses.field(default_factory=dict)
    num_user_outputs: int = 0

    def tangent_of(self, out_idx: int) -> Optional[fx.Node]:
        for n in self.tangent_nodes:
            if n.meta["apb200_tangent_of"] == out_idx:
                return n
        return None


def normalize_inputs(raw) -> ForwardInputs:
    if isinstance(raw, ForwardInputs):
        return ForwardInputs(tuple(raw.args), dict(raw.kwargs))
    if isinstance(raw, tuple):
        return ForwardInputs(raw)
    return ForwardInputs((raw,))


def move_to_fake(model: nn.Module, mode: FakeTensorMode, device) -> nn.Module:
    """Swap every meta parameter/buffer for a fake tensor on ``device``, preserving aliases.

    Tied weights (one tensor reachable under two names) map to one fake tensor, so the traced
    graph has a single placeholder for them (reference: tracing.py:39-85).
    """
    memo: dict[int, torch.Tensor] = {}
    for mod in model.modules():
        for store, is_param in ((mod._parameters, True), (mod._buffers, False)):
            for name, t in list(store.items()):
                if t is None:
                    continue
                if id(t) not in memo:
                    if t.device.type != "meta":
                        raise AssertionError(
                            f"{type(mod).__name__}.{name} must live on the meta device (found {t.device}); "
                            "build the model under `with torch.device('meta')`"
                        )
                    with mode:
                        f = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=device)
                    if is_param:
                        f = nn.Parameter(f, requires_grad=t.requires_grad)
                    memo[id(t)] = f
                    memo[id(f)] = f
                store[name] = memo[id(t)]
    return model


def decomposition_table():
    """Core ATen decompositions minus the ops the planner wants to see whole.

    Kept whole (they have sharding rules and fused kernels): layer norm fwd/bwd, softmax fwd/bwd,
    embedding backward, threshold_backward, full_like/empty_like, stack.  ``addmm`` becomes
    ``bias + a @ b`` so linear layers with bias still expose an ``mm`` to tensor parallelism
    (reference: tracing.py:14-36).
    """
    from torch._decomp import core_aten_decompositions

    aten = torch.ops.aten
    table = dict(core_aten_decompositions())
    for op in (
        aten.full_like.default,
        aten.empty_like.default,
        aten.threshold_backward.default,
        aten.native_layer_norm.default,
        aten.native_layer_norm_backward.default,
        aten.embedding_dense_backward.default,
        aten._softmax.default,
        aten._softmax_backward_data.default,
        aten.stack.default,
        aten.addmm.default,
        aten._scaled_dot_product_flash_attention_for_cpu.default,
    ):
        table.pop(op, None)

    def addmm(self, mat1, mat2, beta=1, alpha=1):
        out = mat1 @ mat2
        if alpha != 1:
            out = out * alpha
        return (self if beta == 1 else self * beta) + out

    table[aten.addmm.default] = addmm
    return table


@contextlib.contextmanager
def _local_map_capture():
    """Make Dynamo keep ``local_map`` regions as one higher-order node (if this torch can)."""
    try:
        from torch._dynamo.variables.higher_order_ops import LocalMapWrappedHigherOrderVariable as vt
        from torch._higher_order_ops import local_map as lm

        with vt.enable(), lm.defer_inlining():
            yield
    except ImportError:  # pragma: no cover - older torch
        yield


@contextlib.contextmanager
def _flex_attention_on_fake_cpu():
    """Planning runs on fake CPU tensors, and flex attention's Python front end refuses inputs on the CPU
    that require gradients (its eager CPU kernel has no backward).  Nothing is computed while tracing, and
    the captured higher-order operators are device independent, so the check is lifted for the capture."""
    try:
        import torch.nn.attention.flex_attention as fa
    except ImportError:  # pragma: no cover
        yield
        return
    saved = getattr(fa, "_validate_device", None)
    if saved is None:
        yield
        return
    fa._validate_device = lambda query, key, value: None
    try:
        yield
    finally:
        fa._validate_device = saved


def _add_unused_state(model: nn.Module, gm: fx.GraphModule) -> None:
    """Dynamo drops parameters ``forward`` never reads; re-attach them so they are sharded,
    initialised and checkpointed like the others (reference: tracing.py:99-137)."""
    from torch.fx.graph_module import _assign_attr

    have = set(dict(gm.named_parameters(remove_duplicate=False))) | set(dict(gm.named_buffers(remove_duplicate=False)))
    first = next((n for n in gm.graph.nodes if n.op not in ("placeholder", "get_attr")), None)
    added = False
    for fqn, t in list(model.named_parameters()) + list(model.named_buffers()):
        if fqn in have:
            continue
        _assign_attr(t, gm, fqn)
        with gm.graph.inserting_before(first):
            n = gm.graph.create_node("get_attr", target=fqn)
            n.meta["val"] = t
        added = True
    if added:
        gm.recompile()


def _unalias_outputs(captured: fx.GraphModule) -> int:
    """Outputs that share storage with an earlier output (``return y, y.t()``) get a copy of their own.

    AOTAutograd leaves such an output out of the differentiated graph - it has no tangent there - and expects a run-time
    wrapper to rebuild it as a view of the other output so that autograd reaches it that way.  The per-rank graphs of this
    framework run without that wrapper (and a view recorded with global sizes would be wrong on a shard anyway), so
    gradients arriving through the second output would be dropped without an error.  A copy is a node of the graph like
    any other: it gets its own tangent."""
    from torch.multiprocessing.reductions import StorageWeakRef
    from torch.utils import _pytree as pytree

    g = captured.graph
    out = next(n for n in g.nodes if n.op == "output")
    flat, spec = pytree.tree_flatten(out.args[0])
    seen: set = set()
    count = 0
    for i, v in enumerate(flat):
        ev = v.meta.get("example_value", v.meta.get("val")) if isinstance(v, fx.Node) else None
        if not isinstance(ev, torch.Tensor):
            continue
        try:
            key = StorageWeakRef(ev.untyped_storage())
        except Exception:
            continue
        if key in seen:
            with g.inserting_before(out):
                c = g.call_function(torch.clone, (v,))
            c.meta = dict(v.meta)
            flat[i] = c
            count += 1
        else:
            seen.add(key)
    if count:
        out.args = (pytree.tree_unflatten(flat, spec),)
        g.lint()
        captured.recompile()
    return count


def build_joint_graph(
    model: nn.Module, input_fn: Callable, fake_mode: FakeTensorMode, canonicalize: bool = True, pattern_ops: bool = True
) -> JointGraph:
    from torch._dynamo.functional_export import _dynamo_graph_capture_for_export
    from torch._functorch.aot_autograd import aot_export_joint_with_descriptors
    from torch.export._trace import _restore_state_dict

    t0 = time.perf_counter()
    with fake_mode:
        traced_inputs = normalize_inputs(input_fn())

    with contextlib.ExitStack() as stack:
        # allow_rnn: nn.RNN / nn.GRU / nn.LSTM are captured as their ATen operators instead of being refused; with the
        # oneDNN flag off their decomposition takes the generic per-step form rather than a fused CPU-only operator that
        # the planning host offers but the devices the graph will run on do not have
        with cast_reads(True), _local_map_capture(), _flex_attention_on_fake_cpu(), \
                torch._dynamo.config.patch(allow_rnn=True), torch.backends.mkldnn.flags(enabled=False), \
                torch._dynamo.utils._disable_saved_tensors_hooks_during_tracing():
            captured = _dynamo_graph_capture_for_export(model)(*traced_inputs.args, **traced_inputs.kwargs)
            _restore_state_dict(model, captured)
            _add_unused_state(model, captured)
            _unalias_outputs(captured)
            pattern_stats = {}
            if pattern_ops:
                # stock-PyTorch idioms (nn.RMSNorm, F.silu * x, complex RoPE, F.scaled_dot_product_attention) become this
                # framework's operators before differentiation, so their backward is the operators' own
                from ..passes.pattern_ops import rewrite_to_framework_ops

                pattern_stats = rewrite_to_framework_ops(captured)
            jd = aot_export_joint_with_descriptors(
                stack,
                captured,
                traced_inputs.args,
                traced_inputs.kwargs or None,
                decompositions=decomposition_table(),
            )
        gm = jd.graph_module
        out_spec = getattr(jd, "out_spec", None)
    if canonicalize:
        from .graph_canon import canonicalize as _canon

        _canon(gm)
    joint = index_joint_graph(gm, traced_inputs, out_spec)
    joint.pattern_stats = pattern_stats
    logger.info("joint graph captured in %.3fs (%d nodes); idioms rewritten to framework operators: %s",
                time.perf_counter() - t0, len(gm.graph.nodes), pattern_stats)
    return joint


def index_joint_graph(gm: fx.GraphModule, traced_inputs: ForwardInputs, out_spec=None) -> JointGraph:
    """Classify placeholders and outputs from the descriptors AOTAutograd attached to them."""
    from torch._functorch._aot_autograd import descriptors as D
    from torch.utils._pytree import tree_flatten

    params: dict[str, fx.Node] = {}
    buffers: dict[str, fx.Node] = {}
    n_flat = len(tree_flatten((traced_inputs.args, traced_inputs.kwargs))[0])
    inputs: list[Optional[fx.Node]] = [None] * n_flat
    tangents: list[fx.Node] = []
    for n in gm.graph.nodes:
        if n.op != "placeholder":
            continue
        d = n.meta.get("desc")
        if isinstance(d, D.ParamAOTInput):
            params[d.target] = n
            n.meta["apb200_kind"] = ("param", d.target)
        elif isinstance(d, D.BufferAOTInput):
            buffers[d.target] = n
            n.meta["apb200_kind"] = ("buffer", d.target)
        elif isinstance(d, D.PlainAOTInput):
            if d.idx >= len(inputs):
                inputs.extend([None] * (d.idx + 1 - len(inputs)))
            inputs[d.idx] = n
            n.meta["apb200_kind"] = ("input", d.idx)
        elif isinstance(d, D.TangentAOTInput):
            tangents.append(n)
            out_idx = d.output.idx if isinstance(d.output, D.PlainAOTOutput) else -1
            n.meta["apb200_tangent_of"] = out_idx
            n.meta["apb200_kind"] = ("tangent", out_idx)
        else:
            raise NotImplementedError(f"unsupported joint-graph input {n.name}: {d!r}")

    out_node = next(n for n in gm.graph.nodes if n.op == "output")
    out_vals = list(out_node.args[0])
    out_descs = out_node.meta.get("desc")
    fwd_outputs: list[Any] = []
    param_grads: dict[str, Optional[fx.Node]] = {k: None for k in params}
    input_grads: list[Optional[fx.Node]] = [None] * len(inputs)
    buffer_updates: dict[str, fx.Node] = {}
    for v, d in zip(out_vals, out_descs):
        if isinstance(d, D.PlainAOTOutput):
            fwd_outputs.append(v)
        elif isinstance(d, D.InputMutationAOTOutput) and isinstance(d.mutated_input, D.BufferAOTInput) and isinstance(v, fx.Node):
            buffer_updates[d.mutated_input.target] = v
        elif isinstance(d, D.GradAOTOutput):
            src = d.grad_of
            if isinstance(src, D.ParamAOTInput):
                param_grads[src.target] = v
            elif isinstance(src, D.PlainAOTInput):
                input_grads[src.idx] = v
        elif v is None:
            continue  # gradient slot of an input that does not require grad
        else:
            raise NotImplementedError(f"unsupported joint-graph output descriptor {d!r}")
    num_user = len(fwd_outputs)
    fwd_outputs = fwd_outputs + list(buffer_updates.values())
    return JointGraph(
        gm=gm,
        buffer_updates=buffer_updates,
        num_user_outputs=num_user,
        param_nodes=params,
        buffer_nodes=buffers,
        input_nodes=inputs,
        tangent_nodes=tangents,
        fwd_outputs=fwd_outputs,
        param_grads=param_grads,
        input_grads=input_grads,
        out_spec=out_spec,
        traced_inputs=traced_inputs,
        num_fwd_outputs=len(fwd_outputs),
    )


def clone_model_for_tracing(model: nn.Module) -> nn.Module:
    """Deep copy that keeps parameter aliasing (``copy.deepcopy`` memoises shared tensors)."""
    return copy.deepcopy(model)
