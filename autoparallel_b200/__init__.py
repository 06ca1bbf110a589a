"""autoparallel_b200 – automatic sharding of PyTorch models for NVLink-connected B200 GPUs.

Public surface (mirrors the reference's ``autoparallel/__init__.py:6-17``):
``AutoParallel``, ``auto_parallel``, ``autoparallel_backend``, ``ForwardInputs``,
``with_sharding_constraint``; user collectives live in ``autoparallel_b200.collectives``.
"""
from . import ops  # noqa: F401  (registers the apb200 operator library)
from .runtime import comm_ops  # noqa: F401  (registers the apb200_comm collectives)
from .api import AutoParallel, auto_parallel  # noqa: E402
from .collectives import with_sharding_constraint  # noqa: E402
from .compile import autoparallel_backend  # noqa: E402
from .parallel.frontend.trace import ForwardInputs  # noqa: E402

__all__ = ["AutoParallel", "auto_parallel", "autoparallel_backend", "ForwardInputs", "with_sharding_constraint"]
__version__ = "0.1.0"
