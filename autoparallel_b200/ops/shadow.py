"""Low-precision shadows of parameters, written by the optimizer and read by ``apb200::dtype_cast``.

Under a mixed-precision policy every step casts each fp32 parameter shard to bf16 once in the forward pass and
once more where the backward pass re-gathers it.  The multi-tensor AdamW kernel already has the new fp32 value
in registers, so it can store the bf16 copy on the way out (``optim.AdamW(emit_bf16=True)``); the cast operator
then hands that copy out instead of launching a kernel.  A shadow is used only while the parameter still has the
version it had when the shadow was written: any in-place update made outside the optimizer (``init_weights``,
loading a checkpoint, a manual ``p.mul_()``) bumps the version and the cast falls back to the kernel.
"""
from __future__ import annotations

import weakref

import torch

#: data_ptr of the fp32 local shard -> (shadow tensor, version of the shard when the shadow was written, weak
#: reference to the shard: while it is alive nothing else can own that address)
_shadows: dict[int, tuple] = {}
hits = 0  # casts answered from a shadow (for tests and launch accounting)


def publish(param_local: torch.Tensor, shadow: torch.Tensor) -> None:
    """Called by the optimizer after it has written ``shadow`` = ``param_local`` in low precision."""
    _shadows[param_local.data_ptr()] = (shadow, param_local._version, weakref.ref(param_local))


def lookup(x: torch.Tensor, dtype: torch.dtype):
    global hits
    ent = _shadows.get(x.data_ptr())
    if ent is None:
        return None
    shadow, version, ref = ent
    owner = ref()
    if owner is None:
        del _shadows[x.data_ptr()]
        return None
    if (shadow.dtype != dtype or version != x._version or owner._version != version or owner.shape != x.shape
            or owner.data_ptr() != x.data_ptr() or shadow.device != x.device):
        return None
    hits += 1
    return shadow


def clear() -> None:
    _shadows.clear()
