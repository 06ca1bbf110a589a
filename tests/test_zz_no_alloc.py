"""The allocation-free RMSNorm-backward entry point, called the way its intended users call it:
through the exported C symbol with raw device pointers (no torch binding in between).

It exists for hosts that may not touch the CUDA allocator around a launch – runtimes with a fixed
arena, code inside stream callbacks, real-time loops – so the kernel's fp32 work buffer is a fixed
array inside the library.  The checks: the result equals the regular entry point's (which gets its
work buffer from the caller) on two calls in a row with different data, proving that the shared
array is cleared between calls; and widths beyond the built-in array are refused, not truncated.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    from autoparallel_b200.ops import build, cuda_impl

    cuda_impl.ensure_loaded()
    so = ctypes.CDLL(build.so_path())
    fn = so.apb_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    so.apb_noalloc_strerror.restype = ctypes.c_char_p
    so.apb_noalloc_strerror.argtypes = [ctypes.c_int]
    return so


def _call(so, dy, x, w, rstd):
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    stream = torch.cuda.current_stream().cuda_stream
    rc = so.apb_rms_norm_bwd_noalloc(
        dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
        x.shape[0], x.shape[1], int(x.dtype == torch.bfloat16), stream,
    )
    assert rc == 0, so.apb_noalloc_strerror(rc).decode()
    return dx, dw


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_matches_regular_entry_point_twice(lib, dtype):
    from autoparallel_b200.ops import library as L

    torch.manual_seed(0)
    rows, D = 300, 4096
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for call in range(2):  # second call: new data, same built-in array
        x = torch.randn(rows, D, device="cuda", dtype=dtype) * (1 + call)
        w = torch.randn(D, device="cuda", dtype=dtype)
        dy = torch.randn(rows, D, device="cuda", dtype=dtype)
        _, rstd = L.ops.rms_norm(x, w, 1e-5)
        ref_dx, ref_dw = L.ops.rms_norm_bwd(dy, x, w, rstd)
        dx, dw = _call(lib, dy, x, w, rstd)
        torch.cuda.synchronize()
        assert torch.allclose(dx.float(), ref_dx.float(), rtol=tol, atol=tol)
        # both paths add per-block partial sums with atomics, so order-of-summation noise only
        assert torch.allclose(dw.float(), ref_dw.float(), rtol=tol, atol=tol * 8 if dtype == torch.bfloat16 else 1e-3)


def test_rejects_width_beyond_builtin_array(lib):
    D = 16384 + 8
    x = torch.zeros(1, D, device="cuda")
    rc = lib.apb_rms_norm_bwd_noalloc(
        x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, D, 0,
        torch.cuda.current_stream().cuda_stream,
    )
    assert rc == 7
    assert b"16384" in lib.apb_noalloc_strerror(rc)


def _reference(dy, x, w, rstd):
    from autoparallel_b200.ops import library as L

    return L.ops.rms_norm_bwd(dy, x, w, rstd)


def test_no_rows_gives_zero_weight_gradient(lib):
    """An empty batch must still clear what an earlier call left in the built-in array."""
    from autoparallel_b200.ops import library as L

    D = 1024
    x = torch.randn(64, D, device="cuda")
    w = torch.randn(D, device="cuda")
    _, rstd = L.ops.rms_norm(x, w, 1e-5)
    _call(lib, torch.randn_like(x), x, w, rstd)  # leaves non-zero sums behind
    empty = torch.empty(0, D, device="cuda")
    _, dw = _call(lib, empty, empty, w, torch.empty(0, device="cuda"))
    torch.cuda.synchronize()
    assert torch.count_nonzero(dw).item() == 0


def test_width_changes_between_calls(lib):
    """4096 -> 1024 -> 4096 on one stream: every call only trusts the part of the array it cleared."""
    from autoparallel_b200.ops import library as L

    torch.manual_seed(1)
    for D in (4096, 1024, 4096):
        x = torch.randn(257, D, device="cuda")
        w = torch.randn(D, device="cuda")
        dy = torch.randn(257, D, device="cuda")
        _, rstd = L.ops.rms_norm(x, w, 1e-5)
        ref_dx, ref_dw = _reference(dy, x, w, rstd)
        dx, dw = _call(lib, dy, x, w, rstd)
        torch.cuda.synchronize()
        assert torch.allclose(dx, ref_dx, rtol=1e-5, atol=1e-5)
        assert torch.allclose(dw, ref_dw, rtol=1e-3, atol=1e-3)


def test_widest_supported_row_in_bf16(lib):
    """D = 16384 is the last width the built-in array covers; bf16 takes the cast path on the way out."""
    from autoparallel_b200.ops import library as L

    torch.manual_seed(2)
    rows, D = 33, 16384
    x = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(D, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(rows, D, device="cuda", dtype=torch.bfloat16)
    _, rstd = L.ops.rms_norm(x, w, 1e-5)
    ref_dx, ref_dw = _reference(dy, x, w, rstd)
    dx, dw = _call(lib, dy, x, w, rstd)
    torch.cuda.synchronize()
    assert torch.allclose(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2)
    assert torch.allclose(dw.float(), ref_dw.float(), rtol=2e-2, atol=0.16)
