"""The allocation-free C entry point against the regular operator path.

Some callers cannot allocate device memory when they need the clip coefficient
(a frozen memory pool, a guest plugin in a process that owns the context, a full
device); ``gefenx_clip_coef_noalloc`` serves them from a fixed array inside the
library.  It is called here through its exported C symbol, twice in a row with
different data, and must agree with the tensor-based path each time.  The file
name sorts last so that a run that stops at the first failure has already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gefen_x_b200 import build
    from gefen_x_b200.ops import _ext

    _ext.available(required=True)
    lib = ctypes.CDLL(str(build.cuda_lib_path()))
    lib.gefenx_clip_coef_noalloc.restype = ctypes.c_int
    lib.gefenx_clip_coef_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                             ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    lib.gefenx_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _regular(grad, max_norm):
    from gefen_x_b200.ops import update as U

    partials = torch.zeros(2048, dtype=torch.float32, device=grad.device)
    coef = torch.zeros(2, dtype=torch.float32, device=grad.device)
    U.reduce_sources(None, [grad.data_ptr()], grad.numel(), 1.0, partials, grad.dtype, grad.device)
    U.clip_coef(partials, max_norm, coef)
    return coef


def test_no_alloc_clip_coef_matches_regular_path_twice():
    lib = _lib()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    out = torch.zeros(2, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev)
    cases = [((3_000_001,), torch.bfloat16, 2e-3, 0.5), ((777, 129), torch.float32, 5.0, 1.0)]
    # warm-up call: the driver loads the library's device image on first use (lazy module loading),
    # which takes device memory once; the calls measured below come after it
    warm = torch.ones(64, dtype=torch.float32, device=dev)
    assert lib.gefenx_clip_coef_noalloc(warm.data_ptr(), 64, 0, 1.0, out.data_ptr(), stream.cuda_stream) == 0
    torch.cuda.synchronize(dev)
    for shape, dtype, scale, max_norm in cases:      # two calls in a row, the second on less data
        grad = (torch.randn(shape, device=dev, generator=g) * scale).to(dtype)
        torch.cuda.synchronize(dev)
        # free bytes as the driver sees them: a raw cudaMalloc inside the entry point (which torch's own
        # counters cannot see) would lower this figure
        free_before, _total = torch.cuda.mem_get_info(dev)
        rc = lib.gefenx_clip_coef_noalloc(grad.data_ptr(), grad.numel(), {torch.float32: 0, torch.bfloat16: 1}[dtype],
                                          max_norm, out.data_ptr(), stream.cuda_stream)
        assert rc == 0, lib.gefenx_noalloc_last_error()
        torch.cuda.synchronize(dev)
        free_after, _total = torch.cuda.mem_get_info(dev)
        assert free_after >= free_before, (free_before, free_after)
        want = _regular(grad, max_norm)
        torch.cuda.synchronize(dev)
        exact = grad.float().norm().item()
        assert abs(out[1].item() - exact) <= 1e-4 * exact
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-7), (out, want)


def test_no_alloc_rejects_oversize_and_bad_arguments():
    lib = _lib()
    dev = torch.device("cuda", 0)
    out = torch.zeros(2, dtype=torch.float32, device=dev)
    x = torch.ones(16, dtype=torch.float32, device=dev)
    s = torch.cuda.current_stream(dev).cuda_stream
    too_many = 65536 * 16384 + 1
    assert lib.gefenx_clip_coef_noalloc(x.data_ptr(), too_many, 0, 1.0, out.data_ptr(), s) == 2
    assert b"exceed" in lib.gefenx_noalloc_last_error()
    assert lib.gefenx_clip_coef_noalloc(None, 16, 0, 1.0, out.data_ptr(), s) == 1
    assert lib.gefenx_clip_coef_noalloc(x.data_ptr(), 16, 7, 1.0, out.data_ptr(), s) == 1
    host = torch.ones(16, dtype=torch.float32)                       # not device memory of the current GPU
    assert lib.gefenx_clip_coef_noalloc(host.data_ptr(), 16, 0, 1.0, out.data_ptr(), s) == 1
    assert b"current device" in lib.gefenx_noalloc_last_error()
    assert lib.gefenx_clip_coef_noalloc(x.data_ptr(), 16, 0, 1.0, out.data_ptr(), s) == 0
    torch.cuda.synchronize(dev)
    assert abs(out[1].item() - 4.0) < 1e-5 and abs(out[0].item() - 0.25) < 1e-5
