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
