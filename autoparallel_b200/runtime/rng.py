"""Random numbers for sharded tensors.

A random operator whose output the plan shards runs once per rank on that rank's shard.  With one
seed for the whole job (the usual ``torch.manual_seed(s)`` on every rank) all ranks would draw the
same numbers, so the global tensor would be one local draw tiled across the mesh - dropout masks
repeating from shard to shard.  Replicated random tensors, on the other hand, MUST be drawn
identically everywhere.  The lowering therefore routes every random operator with a sharded output
through this module: the draw comes from a generator that is seeded from the job's seed and from the
rank's coordinates along exactly those mesh dims the output is sharded on.  Ranks that hold the
same shard (they differ only along replicated mesh dims) share coordinates, hence the stream;
ranks that hold different shards draw different numbers.  Replicated outputs keep using the default
generator.  All ranks run the same sequence of operators, so the per-key generators stay in step.

Reference: the reference lowers through DTensor, whose offset-based RNG tracker makes a sharded draw
equal the single-device draw (torch/distributed/tensor/_random.py); here the draws are
independent per shard rather than bit-identical to a single-device run.
"""
from __future__ import annotations

import torch

_generators: dict = {}


def _generator(device, key) -> torch.Generator:
    """``key`` = ((mesh dim, coordinate), ...) of the sharded mesh dims."""
    device = torch.device(device)
    full = (device.type, device.index, key, torch.initial_seed())
    g = _generators.get(full)
    if g is None:
        g = torch.Generator(device=device)
        seed = torch.initial_seed() & 0x7FFFFFFFFFFFFFFF
        for dim, coord in key:
            seed = (seed * 6364136223846793005 + 1442695040888963407 + 1000003 * (dim + 1) + coord) & 0x7FFFFFFFFFFFFFFF
        g.manual_seed(seed)
        _generators[full] = g
    return g


def reset() -> None:
    _generators.clear()


def sharded_rand(size, key, normal: bool, dtype=None, layout=None, device=None, pin_memory=None):
    device = device if device is not None else "cpu"
    fn = torch.randn if normal else torch.rand
    return fn(list(size), generator=_generator(device, key), dtype=dtype, device=device)


def sharded_dropout(x: torch.Tensor, p: float, train, key):
    """``aten.native_dropout`` on a shard: (output, mask) with a mask drawn from the shard's own stream."""
    if train is False or p == 0.0:
        return x.clone(), torch.ones_like(x, dtype=torch.bool)
    if p >= 1.0:
        return torch.zeros_like(x), torch.zeros_like(x, dtype=torch.bool)
    noise = torch.rand(x.shape, generator=_generator(x.device, key), dtype=torch.float32, device=x.device)
    mask = noise >= p
    return x * mask.to(x.dtype) * (1.0 / (1.0 - p)), mask


def sharded_like(op, key, x: torch.Tensor, *args, **kwargs):
    """``uniform`` / ``normal`` / ``bernoulli`` / ``rand_like`` / ``randn_like`` on a shard, drawn from the shard's stream."""
    aten = torch.ops.aten
    g = _generator(x.device, key)
    kwargs = {k: v for k, v in kwargs.items() if k != "generator"}
    if op is aten.uniform.default:
        lo = args[0] if len(args) > 0 else kwargs.get("from", 0.0)
        hi = args[1] if len(args) > 1 else kwargs.get("to", 1.0)
        return torch.empty_like(x).uniform_(lo, hi, generator=g)
    if op is aten.normal_functional.default:
        mean = args[0] if len(args) > 0 else kwargs.get("mean", 0.0)
        std = args[1] if len(args) > 1 else kwargs.get("std", 1.0)
        return torch.empty_like(x).normal_(mean, std, generator=g)
    if op is aten.bernoulli.p:
        p = args[0] if args else kwargs.get("p", 0.5)
        return torch.empty_like(x).bernoulli_(p, generator=g)
    if op is aten.bernoulli.default:
        return torch.bernoulli(x, generator=g)
    dtype = kwargs.get("dtype") or x.dtype
    fn = torch.randn if op is aten.randn_like.default else torch.rand
    return fn(x.shape, generator=g, dtype=dtype, device=x.device)
