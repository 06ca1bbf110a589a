import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def free_port() -> int:
    """A TCP port that is free right now (multi-process tests rendezvous on 127.0.0.1; fixed ports collide when test
    workers run side by side)."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def fake_world():
    """8 fake ranks in one process: collectives are shape-only no-ops, so planning, lowering and
    even execution of rank 0's graph run without any device (the reference's test harness does the
    same, tests/conftest.py:43-82 there)."""
    import torch.distributed as dist
    from torch.testing._internal.distributed.fake_pg import FakeStore

    if not dist.is_initialized():
        dist.init_process_group("fake", store=FakeStore(), rank=0, world_size=8)
    yield
    # left initialised for the whole session


@pytest.fixture()
def mesh_1d(fake_world):
    from torch.distributed.device_mesh import init_device_mesh

    return init_device_mesh("cpu", (8,), mesh_dim_names=("dp",))


@pytest.fixture()
def mesh_2d(fake_world):
    from torch.distributed.device_mesh import init_device_mesh

    return init_device_mesh("cpu", (2, 4), mesh_dim_names=("dp", "tp"))


@pytest.fixture(autouse=True)
def _reset_planner_caches():
    yield
    from autoparallel_b200.parallel.cost import comm, compute
    from autoparallel_b200.parallel.strategies import options

    options.reset_caches()
    compute.reset_cache()
    comm.reset_cache()
