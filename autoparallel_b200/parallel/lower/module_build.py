"""Reconstruction of the user's module around sharded parameters.

The returned object is an instance of a one-off subclass of the *user's own class* (so
``isinstance``, methods, properties and class attributes keep working) whose ``__init__`` never
ran: instance attributes are copied from the traced model, the module tree is rebuilt from
shells of the original sub-modules (container types such as ``ModuleDict`` survive), parameters
and buffers are replaced by their sharded ``DTensor`` versions with aliasing (tied weights,
shared buffers, shared sub-modules) preserved, and ``forward`` is the generated parallel
function.  Reference: autoparallel/module_construction.py:17-246.
"""
from __future__ import annotations

import copy
from typing import Callable

import torch
import torch.nn as nn

from ..frontend.mp_cast import original_class


def _shell(old: nn.Module, cls: type) -> nn.Module:
    new = cls.__new__(cls)
    nn.Module.__init__(new)
    skip = {"_parameters", "_buffers", "_modules", "_non_persistent_buffers_set", "_apb200_mp_policy"}
    for k, v in old.__dict__.items():
        if k in skip or k in new.__dict__ and k.startswith("_") and k.endswith("hooks"):
            continue
        if k in ("training",):
            new.__dict__[k] = v
            continue
        if k.startswith("_") and k in new.__dict__:
            continue  # nn.Module internals already initialised
        try:
            new.__dict__[k] = copy.copy(v)
        except Exception:
            new.__dict__[k] = v
    new._non_persistent_buffers_set = set(old._non_persistent_buffers_set)
    return new


def make_parallel_module(
    model: nn.Module,
    sharded_params: dict[str, nn.Parameter],
    sharded_buffers: dict[str, torch.Tensor],
    forward_fn: Callable,
) -> nn.Module:
    user_cls = original_class(model)

    def forward(self, *args, **kwargs):
        return forward_fn(self, *args, **kwargs)

    root_cls = type(user_cls.__name__, (user_cls,), {"forward": forward, "_apb200_parallel": True})
    root_cls.__module__ = user_cls.__module__
    root_cls.__qualname__ = user_cls.__qualname__

    # canonical fqn for every (possibly aliased) tensor object
    canon_p: dict[int, str] = {}
    for fqn, p in model.named_parameters(remove_duplicate=False):
        canon_p.setdefault(id(p), fqn)
    canon_b: dict[int, str] = {}
    for fqn, b in model.named_buffers(remove_duplicate=False):
        canon_b.setdefault(id(b), fqn)

    memo: dict[int, nn.Module] = {}

    def build(old: nn.Module, is_root: bool) -> nn.Module:
        if id(old) in memo:
            return memo[id(old)]
        cls = root_cls if is_root else original_class(old)
        new = _shell(old, cls)
        memo[id(old)] = new
        for name, p in old._parameters.items():
            if p is None:
                new._parameters[name] = None
                continue
            fqn = canon_p[id(p)]
            if fqn not in sharded_params:
                raise KeyError(f"parameter {fqn} missing from the sharded state")
            new._parameters[name] = sharded_params[fqn]
        for name, b in old._buffers.items():
            if b is None:
                new._buffers[name] = None
                continue
            new._buffers[name] = sharded_buffers[canon_b[id(b)]]
        for name, child in old._modules.items():
            new._modules[name] = build(child, False) if child is not None else None
        return new

    return build(model, True)
