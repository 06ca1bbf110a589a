"""Shared helper of the examples: a fake process group of N ranks in one process (planning,
lowering and even executing rank 0's graph need no GPU and no real communication)."""
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.testing._internal.distributed.fake_pg import FakeStore


def fake_mesh(shape, names):
    world = 1
    for s in shape:
        world *= s
    if not dist.is_initialized():
        dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=world)
    return init_device_mesh("cpu", tuple(shape), mesh_dim_names=tuple(names))
