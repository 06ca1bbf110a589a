"""Harness-only compatibility layer: lets the unmodified reference package run on torch 2.11.

The reference targets a newer torch nightly than the one in this image and reads a few private
DTensor symbols that do not exist here yet.  This module adds them to *torch* (never to the
reference, whose source stays byte-identical) before ``autoparallel`` is imported.  Every symbol
touched is listed in ``SHIMMED`` so the benchmark line can name them.

Call ``install()`` once, before importing ``autoparallel``.
"""
from __future__ import annotations

import functools
import inspect

SHIMMED: list[str] = []


def _note(name: str) -> None:
    if name not in SHIMMED:
        SHIMMED.append(name)


def install() -> list[str]:
    import torch  # noqa: F401
    import torch.distributed.tensor._ops.utils as ops_utils
    import torch.distributed.tensor._sharding_prop as sharding_prop

    # 1. _SingleDimStrategyInfo.allow_uneven_sharding (newer torch: a dataclass field, default False).
    info = getattr(sharding_prop, "_SingleDimStrategyInfo", None)
    if info is not None and not hasattr(info, "allow_uneven_sharding"):
        info.allow_uneven_sharding = False  # class attribute = default for every instance
        _note("torch.distributed.tensor._sharding_prop._SingleDimStrategyInfo.allow_uneven_sharding=False")

    # 2. expand_to_full_mesh_op_strategy(..., allow_uneven_sharding=) : accept the keyword and drop it
    #    (False is this torch's behaviour: shardings that do not divide evenly are filtered).
    fn = ops_utils.expand_to_full_mesh_op_strategy
    if "allow_uneven_sharding" not in inspect.signature(fn).parameters and not getattr(fn, "_apb_compat", False):

        @functools.wraps(fn)
        def expand_to_full_mesh_op_strategy(*args, allow_uneven_sharding=False, **kwargs):
            return fn(*args, **kwargs)

        expand_to_full_mesh_op_strategy._apb_compat = True
        ops_utils.expand_to_full_mesh_op_strategy = expand_to_full_mesh_op_strategy
        _note("torch.distributed.tensor._ops.utils.expand_to_full_mesh_op_strategy(allow_uneven_sharding=) dropped")
    # 3. ShardingPropagator.decomp_strategy : newer torch keeps one DecompShardingStrategy instance
    #    on the propagator; this torch has the same logic as static methods that take the propagator.
    if not hasattr(sharding_prop.ShardingPropagator, "decomp_strategy"):
        from torch.distributed.tensor._decompositions import DecompShardingStrategy

        class _BoundDecompStrategy:
            def __init__(self, prop):
                self._prop = prop

            def ensure_schema_info(self, op):
                return DecompShardingStrategy.ensure_schema_info(op, self._prop)

            def propagate_strategy(self, op_schema):
                return DecompShardingStrategy.propagate_strategy(op_schema, self._prop)

        sharding_prop.ShardingPropagator.decomp_strategy = property(lambda self: _BoundDecompStrategy(self))
        _note("torch.distributed.tensor._sharding_prop.ShardingPropagator.decomp_strategy (bound view of the static DecompShardingStrategy)")
    # 4. torch._functorch.partitioners: helpers that the reference's replay partitioner imports.
    import torch._functorch.partitioners as partitioners

    if not hasattr(partitioners, "_is_assert_only_symbool"):
        # newer torch: True for symbolic booleans that only feed runtime asserts (they need not be saved
        # for the backward).  Answering False keeps every symbolic node, which is always correct.
        partitioners._is_assert_only_symbool = lambda node: False
        _note("torch._functorch.partitioners._is_assert_only_symbool -> False")
    if not hasattr(partitioners, "is_opaque_node"):
        def is_opaque_node(node):
            val = node.meta.get("val") if hasattr(node, "meta") else None
            try:
                from torch._library.fake_class_registry import FakeScriptObject

                opaque = (torch.ScriptObject, FakeScriptObject)
            except Exception:
                opaque = (torch.ScriptObject,)
            return isinstance(val, opaque)

        partitioners.is_opaque_node = is_opaque_node
        _note("torch._functorch.partitioners.is_opaque_node (script-object values)")
    ext = partitioners._extract_fwd_bwd_modules
    if "saved_opaque_nodes" not in inspect.signature(ext).parameters and not getattr(ext, "_apb_compat", False):

        @functools.wraps(ext)
        def _extract_fwd_bwd_modules(joint_module, saved_values, saved_sym_nodes, *args, saved_opaque_nodes=None, **kwargs):
            if saved_opaque_nodes:
                saved_values = list(saved_values) + [n for n in saved_opaque_nodes if n not in saved_values]
            return ext(joint_module, saved_values, saved_sym_nodes, *args, **kwargs)

        _extract_fwd_bwd_modules._apb_compat = True
        partitioners._extract_fwd_bwd_modules = _extract_fwd_bwd_modules
        _note("torch._functorch.partitioners._extract_fwd_bwd_modules(saved_opaque_nodes=) merged into saved_values")
    return SHIMMED
