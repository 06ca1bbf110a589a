"""Operator library (schemas + CPU reference + sm_100a kernels)."""
from .library import (  # noqa: F401
    attention,
    cross_entropy,
    dtype_cast,
    lib,
    ops,
    reference_impls,
    register_cuda_impl,
    rms_norm,
    rope,
    swiglu,
)
from . import moe_ops  # noqa: F401,E402  (registers the planner-visible MoE operators)
from .moe_ops import grouped_mm, moe_combine, moe_dispatch, moe_slots  # noqa: F401,E402
