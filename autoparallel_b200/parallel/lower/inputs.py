"""Runtime input checking and sample-input helpers for the simple API.

``input_fn`` describes *global* tensors; the parallel module is called with *local* shards.
This module derives the expected local shapes from the solved input placements, validates each
call (count, type, rank, shape, dtype, equality of non-tensor arguments) and builds an
``input_fn`` from sample inputs that may be DTensors.  Reference:
autoparallel/input_validation.py:27-324.
"""
from __future__ import annotations

from typing import Any, Optional, Sequence

import torch
from torch.distributed.tensor import DTensor
from torch.utils._pytree import tree_flatten, tree_unflatten

from ..frontend.trace import ForwardInputs
from ..strategies.dtensor_adapter import my_local_shape


def expected_local_inputs(traced: ForwardInputs, placements: Sequence[Optional[tuple]], mesh) -> list:
    """Per flat input: ``("tensor", local_shape, dtype)`` or ``("value", v)``."""
    flat, _ = tree_flatten((traced.args, traced.kwargs))
    out = []
    for v, pl in zip(flat, list(placements) + [None] * (len(flat) - len(placements))):
        if isinstance(v, torch.Tensor):
            shape = list(v.shape)
            if pl is not None:
                shape = my_local_shape(shape, mesh, pl)
            out.append(("tensor", tuple(shape), v.dtype))
        else:
            out.append(("value", v))
    return out


def check_forward_args(flat_args: Sequence[Any], expected: Sequence[tuple]) -> None:
    if len(flat_args) != len(expected):
        raise ValueError(f"expected {len(expected)} (flattened) inputs, got {len(flat_args)}")
    for i, (a, e) in enumerate(zip(flat_args, expected)):
        if e[0] == "tensor":
            if not isinstance(a, torch.Tensor):
                raise TypeError(f"input {i}: expected a tensor, got {type(a).__name__}")
            if a.ndim != len(e[1]):
                raise ValueError(f"input {i}: expected {len(e[1])} dims (local shape {e[1]}), got shape {tuple(a.shape)}")
            if tuple(a.shape) != tuple(e[1]):
                raise ValueError(
                    f"input {i}: expected local shape {e[1]}, got {tuple(a.shape)} – the parallel module takes "
                    "this rank's shard, not the global tensor"
                )
            if a.dtype != e[2]:
                raise TypeError(f"input {i}: expected dtype {e[2]}, got {a.dtype}")
        else:
            if isinstance(a, torch.Tensor) or a != e[1]:
                raise ValueError(f"input {i}: non-tensor argument must equal the traced value {e[1]!r}, got {a!r}")


def flatten_call(traced: ForwardInputs, args: tuple, kwargs: dict) -> list:
    """Flatten a runtime call in the traced ``tree_flatten((args, kwargs))`` order, accepting
    keyword arguments in any order."""
    ordered = {k: kwargs[k] for k in traced.kwargs if k in kwargs}
    extra = [k for k in kwargs if k not in traced.kwargs]
    if extra:
        raise TypeError(f"unexpected keyword arguments {extra}; traced with {list(traced.kwargs)}")
    flat, _ = tree_flatten((tuple(args), ordered))
    return flat


def input_fn_from_samples(sample_args: tuple, sample_kwargs: Optional[dict] = None):
    """``(input_fn, flat input placements)`` from sample inputs.  DTensor leaves contribute their
    global shape and placements; plain tensors are taken as global and replicated."""
    sample_kwargs = sample_kwargs or {}
    flat, spec = tree_flatten((tuple(sample_args), dict(sample_kwargs)))
    metas, placements = [], []
    for v in flat:
        if isinstance(v, DTensor):
            metas.append(("t", tuple(v.shape), v.dtype, v.requires_grad))
            placements.append(tuple(v.placements))
        elif isinstance(v, torch.Tensor):
            metas.append(("t", tuple(v.shape), v.dtype, v.requires_grad))
            placements.append(None)
        else:
            metas.append(("v", v))
            placements.append(None)

    def input_fn():
        leaves = []
        for m in metas:
            if m[0] == "t":
                if m[2].is_floating_point or m[2].is_complex:
                    leaves.append(torch.randn(m[1], dtype=m[2], requires_grad=m[3]))
                else:
                    leaves.append(torch.zeros(m[1], dtype=m[2]))
            else:
                leaves.append(m[1])
        a, k = tree_unflatten(leaves, spec)
        return ForwardInputs(tuple(a), dict(k))

    return input_fn, placements


def flatten_out_shardings(out_shardings, num_outputs: int, mesh) -> list:
    """Normalise ``out_shardings`` (one placement tuple, or a pytree of them) to a flat list."""
    if out_shardings is None:
        return [None] * num_outputs

    def is_placement_tuple(x):
        from torch.distributed.tensor.placement_types import Placement

        return isinstance(x, (tuple, list)) and len(x) > 0 and all(isinstance(p, Placement) for p in x)

    if is_placement_tuple(out_shardings):
        return [tuple(out_shardings)] * num_outputs
    flat, _ = tree_flatten(out_shardings, is_leaf=lambda x: x is None or is_placement_tuple(x))
    if len(flat) != num_outputs:
        raise ValueError(f"out_shardings has {len(flat)} leaves for {num_outputs} outputs")
    return [tuple(x) if x is not None else None for x in flat]
