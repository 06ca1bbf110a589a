"""Numerics debugging helpers: hashing interpreter, per-run numerics log, rank-ordered printing.
Reference: autoparallel/shardings/placement_options.py:672-813 (DebugInterpreter, NumericsLogger,
print_rank_by_rank)."""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import Optional

import torch
import torch.distributed as dist
import torch.fx as fx


def tensor_hash(t: torch.Tensor) -> str:
    b = t.detach().to(torch.float32).cpu().contiguous().numpy().tobytes() if t.dtype.is_floating_point else t.detach().cpu().contiguous().numpy().tobytes()
    return hashlib.sha1(b).hexdigest()[:12]


class DebugInterpreter(fx.Interpreter):
    """Runs a graph node by node, recording a hash and the norm of every tensor output and raising at
    the first NaN/Inf.  Results of ``*_start`` collectives are not read before their ``comm_wait``."""

    def __init__(self, gm: fx.GraphModule, check_finite: bool = True):
        super().__init__(gm)
        self.records: list[dict] = []
        self.check_finite = check_finite

    def run_node(self, n: fx.Node):
        out = super().run_node(n)
        from ..runtime import comm_ops

        if n.op == "call_function" and n.target not in comm_ops.START_OPS:
            vals = out if isinstance(out, (tuple, list)) else [out]
            for i, v in enumerate(vals):
                if isinstance(v, torch.Tensor) and v.numel() > 0:
                    rec = {"node": n.name, "out": i, "shape": list(v.shape), "hash": tensor_hash(v)}
                    if v.dtype.is_floating_point:
                        rec["norm"] = float(v.float().norm())
                        if self.check_finite and not torch.isfinite(v).all():
                            raise FloatingPointError(f"non-finite values produced by {n.name} ({n.target})")
                    self.records.append(rec)
        return out


class NumericsLogger:
    """Writes weight hashes, per-step losses and intermediate hashes of one run into its own directory
    so two runs (two plans, two ranks, two builds) can be diffed."""

    def __init__(self, root: str, tag: Optional[str] = None):
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.dir = os.path.join(root, f"{tag or time.strftime('%Y%m%d-%H%M%S')}", f"rank{rank}")
        os.makedirs(self.dir, exist_ok=True)

    def log_weights(self, module: torch.nn.Module, name: str = "weights") -> None:
        from torch.distributed.tensor import DTensor

        rows = {k: tensor_hash(v._local_tensor if isinstance(v, DTensor) else v) for k, v in module.state_dict().items()}
        with open(os.path.join(self.dir, f"{name}.json"), "w") as f:
            json.dump(rows, f, indent=1)

    def log_records(self, records: list, name: str) -> None:
        with open(os.path.join(self.dir, f"{name}.json"), "w") as f:
            json.dump(records, f)

    def log_scalar(self, key: str, step: int, value: float) -> None:
        with open(os.path.join(self.dir, "scalars.jsonl"), "a") as f:
            f.write(json.dumps({"key": key, "step": step, "value": value}) + "\n")

    @staticmethod
    def diff(dir_a: str, dir_b: str, name: str) -> list:
        a = json.load(open(os.path.join(dir_a, f"{name}.json")))
        b = json.load(open(os.path.join(dir_b, f"{name}.json")))
        if isinstance(a, dict):
            return [k for k in a if a.get(k) != b.get(k)]
        return [x["node"] for x, y in zip(a, b) if x.get("hash") != y.get("hash")]


def print_rank_by_rank(*args, group=None) -> None:
    """Print from every rank in rank order (a barrier between ranks)."""
    if not dist.is_initialized():
        print(*args, flush=True)
        return
    for r in range(dist.get_world_size(group)):
        if dist.get_rank(group) == r:
            print(f"[rank {r}]", *args, flush=True)
        dist.barrier(group)
