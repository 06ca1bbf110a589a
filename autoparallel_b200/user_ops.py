"""Small functional helpers for model code (reference: autoparallel/ops.py:9-41)."""
from __future__ import annotations

import torch


def permutation(n: int, *, generator=None, device=None, dtype=torch.int64, independent: bool = False, batch: int = 1):
    """Random permutation(s) of ``range(n)`` built from sortable noise (shards like any other
    tensor program, unlike ``randperm``).  ``independent=True`` returns ``[batch, n]`` permutations."""
    shape = (batch, n) if independent else (n,)
    noise = torch.rand(shape, generator=generator, device=device)
    return torch.argsort(noise, dim=-1).to(dtype)
