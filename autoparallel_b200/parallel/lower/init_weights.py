"""Making the user's ``init_weights`` work on a sharded module.

Two mechanisms:

``materialize`` – every DTensor parameter/buffer is temporarily replaced by a full-size plain
tensor on the target device, the user's initialiser runs unchanged (identical on every rank when
the ranks share a seed, so the result does not depend on the plan), and each rank then keeps its
own shard.  Exact, but needs room for the full model once.

``intercept`` – parameters stay DTensors while the initialiser runs.  Assigning a plain tensor or
``nn.Parameter`` to a DTensor slot copies it (interpreted as the *global* value, redistributed to
the slot's placement) instead of replacing the slot; ``dtensor.copy_(plain)`` does the same;
``param.data = x`` is rejected because it would silently drop the sharding.  In-place
initialisers (``normal_`` …) run as DTensor ops.  This is the reference's mechanism
(autoparallel/init_weights.py:13-156) and the only option for models that do not fit on one GPU.
"""
from __future__ import annotations

import contextlib
import functools
import logging
import warnings

import torch
import torch.nn as nn
from torch.distributed.tensor import DTensor, distribute_tensor
from torch.utils._python_dispatch import TorchDispatchMode

logger = logging.getLogger(__name__)

_BIG = 1 << 28  # elements; materialising more than this per tensor earns a warning


def _distribute(full: torch.Tensor, mesh, placements) -> DTensor:
    """``distribute_tensor`` that also understands a re-nested shard order (``_StridedShard``)."""
    from .ordered import local_shard, order_of_dtensor_placements

    order = order_of_dtensor_placements(placements, mesh.ndim)
    if order is None:
        return distribute_tensor(full, mesh, placements, src_data_rank=None)
    coord = mesh.get_coordinate()
    local = local_shard(full, placements, coord, tuple(mesh.shape), order)
    return DTensor.from_local(local, mesh, placements, run_check=False, shape=full.shape, stride=full.contiguous().stride())


def _shard_like(full: torch.Tensor, like: DTensor) -> DTensor:
    if full.numel() >= _BIG and any(p.is_shard() for p in like.placements):
        warnings.warn(
            f"init_weights materialised a full tensor of {full.numel()} elements for a sharded slot; "
            "use in-place initialisers on the parameter to avoid the full copy",
            stacklevel=3,
        )
    full = full.detach().to(device=like.device, dtype=like.dtype)
    return _distribute(full, like.device_mesh, like.placements)


class _CopyFromPlain(TorchDispatchMode):
    """``dtensor.copy_(plain)`` → copy of the redistributed global value."""

    def __torch_dispatch__(self, func, types_, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.ops.aten.copy_.default and isinstance(args[0], DTensor) and not isinstance(args[1], DTensor):
            src = _shard_like(args[1].expand(args[0].shape) if args[1].shape != args[0].shape else args[1], args[0])
            return func(args[0], src, *args[2:], **kwargs)
        return func(*args, **kwargs)


@contextlib.contextmanager
def _intercept_assignments():
    orig_setattr = nn.Module.__setattr__

    def setattr_(self, name, value):
        cur = self._parameters.get(name) if "_parameters" in self.__dict__ else None
        is_param_slot = cur is not None
        if not is_param_slot and "_buffers" in self.__dict__:
            cur = self._buffers.get(name)
        if isinstance(cur, DTensor) and isinstance(value, torch.Tensor) and not isinstance(value, DTensor):
            with torch.no_grad():
                cur.copy_(_shard_like(value, cur))
            if is_param_slot and isinstance(value, nn.Parameter):
                cur.requires_grad_(value.requires_grad)
            return
        orig_setattr(self, name, value)

    nn.Module.__setattr__ = setattr_
    try:
        with _CopyFromPlain():
            yield
    finally:
        nn.Module.__setattr__ = orig_setattr


def _guard_data_assignment(t: torch.Tensor):
    # ``p.data = x`` cannot be intercepted per instance without a subclass; DTensor parameters
    # created by apply_placement carry this marker subclass.
    return t


class ShardedParameter(nn.Parameter):
    """Marker type for parameters of a parallel module (a DTensor inside ``nn.Parameter``)."""


def _full_like(dt: DTensor, device) -> torch.Tensor:
    return torch.empty(dt.shape, dtype=dt.dtype, device=device)


def _run_materialized(module: nn.Module, user_init, args, kwargs):
    slots = []  # (owner module, name, is_param, dtensor, plain)
    seen: dict[int, torch.Tensor] = {}
    for mod in module.modules():
        for store, is_param in ((mod._parameters, True), (mod._buffers, False)):
            for name, t in list(store.items()):
                if not isinstance(t, DTensor):
                    continue
                if id(t) not in seen:
                    plain = _full_like(t, t.device)
                    if is_param:
                        plain = nn.Parameter(plain, requires_grad=t.requires_grad)
                    seen[id(t)] = plain
                slots.append((mod, name, is_param, t, seen[id(t)]))
                store[name] = seen[id(t)]
    try:
        out = user_init(*args, **kwargs)
    finally:
        done = set()
        for mod, name, is_param, dt, _ in slots:
            store = mod._parameters if is_param else mod._buffers
            cur = store[name]  # user may have re-assigned the slot
            if id(dt) not in done:
                done.add(id(dt))
                with torch.no_grad():
                    src = cur.detach().to(dt.dtype)
                    if tuple(src.shape) != tuple(dt.shape):
                        raise RuntimeError(f"init_weights changed the shape of {name}: {tuple(src.shape)} vs {tuple(dt.shape)}")
                    shard = _distribute(src, dt.device_mesh, dt.placements)
                    dt._local_tensor.copy_(shard._local_tensor)
            store[name] = dt
    return out


def wrap_init_weights(module: nn.Module, mode: str = "auto") -> None:
    """Replace ``module.init_weights`` (if any) by a sharding-aware version."""
    if not hasattr(module, "init_weights"):
        return
    user_init = module.init_weights

    @functools.wraps(user_init)
    def init_weights(*args, **kwargs):
        m = mode
        if m == "auto":
            total = sum(p.numel() * p.element_size() for p in module.parameters())
            dev = next((p.device for p in module.parameters()), torch.device("cpu"))
            if dev.type == "cuda":
                free, _ = torch.cuda.mem_get_info(dev)
                m = "materialize" if total < 0.5 * free else "intercept"
            else:
                m = "materialize"
        if m == "materialize":
            return _run_materialized(module, user_init, args, kwargs)
        with _intercept_assignments():
            return user_init(*args, **kwargs)

    module.__dict__["init_weights"] = init_weights
