"""Mixed-precision parametrisation.

While the joint graph is traced every floating-point parameter *read* goes through
``apb200::dtype_cast(param, param_dtype)``: the cast becomes a graph node, so the planner can
decide on which side of it the FSDP all-gather goes (gather bf16, not fp32) and on which
side of the gradient up-cast the reduce-scatter goes (reduce fp32 when ``reduce_dtype`` is
wider).  Reference behaviour: autoparallel/cast_parametrization.py:71-204.

Mechanism (ours): each module that owns parameters is re-classed into a one-off subclass
whose ``__getattr__`` intercepts names found in ``_parameters``; nothing else about the
module changes, and the interception is only live inside ``cast_reads()``.
"""
from __future__ import annotations

import contextlib
import dataclasses
from typing import Any, Optional

import torch
import torch.nn as nn
from torch.utils._pytree import tree_map_only

from ...ops import dtype_cast

_STATE = {"on": False}


@dataclasses.dataclass(frozen=True)
class MPPolicy:
    """Canonical mixed-precision policy (same fields as FSDP2's ``MixedPrecisionPolicy``)."""

    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: Optional[torch.dtype] = None
    output_dtype: Optional[torch.dtype] = None
    cast_forward_inputs: bool = True


def canonicalize_mp(policy: Any) -> Optional[MPPolicy]:
    """Accept ``None``, our ``MPPolicy`` or anything with the four FSDP2 attribute names.

    ``reduce_dtype`` defaults to ``param_dtype`` (reference: cast_parametrization.py:116-125).
    """
    if policy is None:
        return None
    pd = getattr(policy, "param_dtype", None)
    rd = getattr(policy, "reduce_dtype", None)
    od = getattr(policy, "output_dtype", None)
    cfi = getattr(policy, "cast_forward_inputs", True)
    if rd is None:
        rd = pd
    return MPPolicy(pd, rd, od, cfi)


@contextlib.contextmanager
def cast_reads(enabled: bool = True):
    prev = _STATE["on"]
    _STATE["on"] = enabled
    try:
        yield
    finally:
        _STATE["on"] = prev


def _make_cast_class(cls: type, param_dtype: torch.dtype) -> type:
    def __getattr__(self, name):  # only reached for params / buffers / submodules
        value = super(new_cls, self).__getattr__(name)
        if (
            _STATE["on"]
            and isinstance(value, torch.Tensor)
            and name in self.__dict__["_parameters"]
            and value.is_floating_point()
            and value.dtype != param_dtype
        ):
            return dtype_cast(value, param_dtype)
        return value

    new_cls = type(cls.__name__, (cls,), {"__getattr__": __getattr__, "_apb200_cast_base": cls})
    new_cls.__module__ = cls.__module__
    new_cls.__qualname__ = cls.__qualname__
    return new_cls


class _CastIO:
    """Mixin installed on the root: casts floating inputs / outputs around ``forward``."""

    def __call__(self, *args, **kwargs):
        pol: MPPolicy = self.__dict__["_apb200_mp_policy"]
        if _STATE["on"] and pol.cast_forward_inputs and pol.param_dtype is not None:
            cast = lambda t: t.to(pol.param_dtype) if t.is_floating_point() else t  # noqa: E731
            args, kwargs = tree_map_only(torch.Tensor, cast, (args, kwargs))
        out = super().__call__(*args, **kwargs)
        if _STATE["on"] and pol.output_dtype is not None:
            cast = lambda t: t.to(pol.output_dtype) if t.is_floating_point() else t  # noqa: E731
            out = tree_map_only(torch.Tensor, cast, out)
        return out


def apply_dtype_cast(model: nn.Module, policy: MPPolicy) -> nn.Module:
    """Re-class ``model`` in place (callers pass a private deep copy)."""
    if policy.param_dtype is not None:
        for mod in model.modules():
            if len(mod._parameters) > 0:
                mod.__class__ = _make_cast_class(mod.__class__, policy.param_dtype)
    root_cls = model.__class__
    io_cls = type(root_cls.__name__, (_CastIO, root_cls), {"_apb200_cast_base": getattr(root_cls, "_apb200_cast_base", root_cls)})
    io_cls.__module__ = root_cls.__module__
    io_cls.__qualname__ = root_cls.__qualname__
    model.__class__ = io_cls
    model.__dict__["_apb200_mp_policy"] = policy
    return model


def original_class(mod: nn.Module) -> type:
    """The user's class of a (possibly re-classed) module."""
    return getattr(type(mod), "_apb200_cast_base", type(mod))
