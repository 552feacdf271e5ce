"""The allocation-free squared-norm entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they need a
gradient norm (for example a plug-in hook that must not allocate, or a process that has frozen its
memory pool). ``ajb_sumsq_f32_static`` serves them with scratch space that is built into the library.
This test checks that it returns what the regular entry point returns, twice in a row (the built-in
scratch keeps the previous call's contents, so the second call proves nothing stale leaks through),
and that it refuses sizes beyond its stated maximum. The file name sorts last on purpose: a run that
stops at the first failure has then already executed every other test.
"""

import ctypes

import pytest
import torch

from ajllm_b200.ops import native

pytestmark = pytest.mark.gpu


def _static_entry():
    lib = native.lib()
    fn = lib.ajb_sumsq_f32_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    limit = lib.ajb_sumsq_f32_static_max_elements
    limit.argtypes = []
    limit.restype = ctypes.c_longlong
    return fn, limit


def _regular(x: torch.Tensor) -> torch.Tensor:
    scratch = torch.empty(native.lib().ajb_sumsq_scratch_floats(), dtype=torch.float32, device=x.device)
    out = torch.full((1,), -1.0, dtype=torch.float32, device=x.device)
    native.call("ajb_sumsq_f32", x.data_ptr(), x.numel(), scratch.data_ptr(), out.data_ptr(), native.stream_ptr())
    return out


def test_static_scratch_entry_matches_regular_entry_twice():
    device = torch.device("cuda", 0)
    fn, _ = _static_entry()
    torch.manual_seed(123)
    # a large input first, then a small one: the second call reads fewer partial sums than the first wrote
    for numel in (3_000_001, 1_237):
        x = torch.randn(numel, device=device, dtype=torch.float32)
        want = _regular(x)
        out = torch.full((1,), -1.0, dtype=torch.float32, device=device)   # caller-owned output, made beforehand
        status = fn(x.data_ptr(), x.numel(), out.data_ptr(), native.stream_ptr())
        assert status == 0, native.lib().ajb_last_error()
        torch.cuda.synchronize()
        exact = float(x.double().square().sum())
        assert abs(float(out) - float(want)) <= 1e-5 * abs(float(want))
        assert abs(float(out) - exact) <= 1e-5 * exact


def test_static_scratch_entry_rejects_oversized_input():
    device = torch.device("cuda", 0)
    fn, limit = _static_entry()
    x = torch.zeros(16, device=device, dtype=torch.float32)
    out = torch.zeros(1, device=device, dtype=torch.float32)
    status = fn(x.data_ptr(), limit() + 1, out.data_ptr(), native.stream_ptr())
    assert status != 0
    message = native.lib().ajb_last_error().decode()
    assert "outside the supported range" in message


def test_static_scratch_entry_accepts_an_empty_input():
    device = torch.device("cuda", 0)
    fn, _ = _static_entry()
    empty = torch.empty(0, device=device, dtype=torch.float32)
    assert empty.data_ptr() == 0
    out = torch.full((1,), -1.0, dtype=torch.float32, device=device)
    status = fn(empty.data_ptr() or None, 0, out.data_ptr(), native.stream_ptr())
    assert status == 0, native.lib().ajb_last_error()
    torch.cuda.synchronize()
    assert float(out) == 0.0
