"""Failures made on the host: damaged plan files, a rank that leaves before a collective, mismatched calls.
(Device waits that run out are covered by tests/test_kernels_gpu.py and the protocol model.)"""
import json
import os

import pytest
from conftest import free_port
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
from torch.distributed.tensor.placement_types import Shard

from autoparallel_b200 import AutoParallel


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.w1 = nn.Linear(64, 128, bias=False)
        self.w2 = nn.Linear(128, 64, bias=False)

    def forward(self, x):
        return self.w2(torch.relu(self.w1(x)))


def test_damaged_placement_files_are_refused(mesh_1d, tmp_path):
    with torch.device("meta"):
        m = MLP()
    with AutoParallel(m, lambda: torch.randn(16, 8, 64), mesh_1d) as ap:
        ap.add_parameter_memory_constraint()
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        opt = ap.sharding_optimizer
        good = tmp_path / "plan.json"
        opt.save_placements(str(good))
        data = json.loads(good.read_text())

        def write(mutate):
            d = json.loads(json.dumps(data))
            mutate(d)
            p = tmp_path / "bad.json"
            p.write_text(json.dumps(d))
            return str(p)

        with pytest.raises(ValueError, match="version"):
            opt.load_placements(write(lambda d: d.update(version=-1)))
        with pytest.raises(ValueError, match="does not match the graph"):
            opt.load_placements(write(lambda d: d["placements"].pop(next(iter(d["placements"])))))
        with pytest.raises(ValueError, match="does not match the graph"):
            opt.load_placements(write(lambda d: d["placements"].update(no_such_node=0)))
        some = next(iter(data["placements"]))
        with pytest.raises(ValueError, match="is not option"):
            opt.load_placements(write(lambda d: d["placements"].update({some: 10 ** 6})))
        with pytest.raises(ValueError, match="is not option"):
            opt.load_placements(write(lambda d: d["readable"].update({some: "S(7)"})))
        truncated = tmp_path / "cut.json"
        truncated.write_text(good.read_text()[: len(good.read_text()) // 2])
        with pytest.raises(json.JSONDecodeError):
            opt.load_placements(str(truncated))
        assert len(opt.load_placements(str(good))) == len(opt.nodes)  # the intact file still loads afterwards


def _leaving_worker(rank, ws, port, q):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(ws))
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=5))
    from autoparallel_b200.runtime import comm_ops

    name = dist.group.WORLD.group_name
    x = torch.full((4,), float(rank))
    out = comm_ops.ops.all_gather(x, 0, name, ws)  # one good step first
    ok_first = torch.equal(out, torch.arange(ws, dtype=torch.float32).repeat_interleave(4))
    if rank == 1:
        # leaves between steps, with nothing of its own in flight; the others learn of it from their next collective
        q.put(("left", rank, ok_first))
        os._exit(0)
    try:
        comm_ops.ops.all_gather(x, 0, name, ws)
        q.put(("no error", rank, ok_first))
    except Exception as e:  # the process group reports the missing peer instead of waiting for ever
        q.put(("error", rank, ok_first, type(e).__name__))
    os._exit(0)


def test_a_rank_that_leaves_is_reported_by_the_next_collective():
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode is not None, "a rank is still waiting: the missing peer was not detected"
    got = sorted(q.get() for _ in range(2))
    kinds = {g[1]: g[0] for g in got}
    assert kinds[1] == "left" and kinds[0] == "error"
    assert all(g[2] for g in got)  # the step before the departure was correct on both ranks


def test_parallel_module_rejects_calls_that_do_not_match_the_plan(mesh_1d):
    with torch.device("meta"):
        m = MLP()
    with AutoParallel(m, lambda: torch.randn(16, 8, 64), mesh_1d) as ap:
        ap.add_input_constraints([(Shard(0),)])
        ap.optimize_placement()
        pm = ap.apply_placement()
    pm.to_empty(device="cpu")
    with pytest.raises(ValueError, match="shard, not the global"):
        pm(torch.randn(16, 8, 64))
    with pytest.raises(TypeError, match="unexpected keyword"):
        pm(torch.randn(2, 8, 64), extra=1)
    with pytest.raises(RuntimeError, match="not re-entrant|exited|inside"):
        ap.optimize_placement()  # the planning context is closed
