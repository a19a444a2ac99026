"""The allocation-free linear entry point (dq_linear_w4a4_int4_static), called straight through
the C ABI with ctypes.

It exists for callers that cannot give the library scratch memory (their HBM is already carved
up, or they sit inside a callback where allocating would stall the device), so the test hands it
nothing but inputs and outputs and checks that it returns exactly what the scratch-taking entry
point returns - twice in a row, because the built-in scratch keeps the previous call's bytes.
This file sorts last on purpose: a run that stops at the first failure has then already
exercised everything else.
"""
import ctypes

import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _vp(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _call_static(lib, x, a, pw, r, y, scale_fp16=True):
    M, K = x.shape
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    return lib.dq_linear_w4a4_int4_static(_vp(x), x.stride(0) if M > 1 else K, _vp(a), None,
                                          _vp(pw.w_packed), _vp(pw.sw_t), _vp(r), M, pw.N, K,
                                          pw.group, _vp(y), _lib.DTYPE_F32, int(scale_fp16), stream)


def _weights(N, K, seed):
    codes, sw = ops.quant_w_int4(synthetic.make_w(N, K, seed).to(DEV))
    return ops.pack_w_int4(codes, sw)


def test_static_scratch_matches_caller_scratch_twice():
    torch.cuda.set_device(0)
    _lib.ensure_init(0)
    lib = _lib.load()
    N, K = 384, 1024
    pw = _weights(N, K, 21)
    r, c = synthetic.make_scales(N, K, 21)
    r, a = r.to(DEV), (1.0 / c).to(DEV)
    # two different batches back to back: the second call finds the first call's codes and
    # scales in the shared scratch and must not be affected by them
    for M, seed in ((16, 1), (5, 2)):
        x = synthetic.make_x(M, K, seed).to(DEV)
        want = ops.linear_w4a4_int4(x, a, None, pw, r, scale_fp16=True)
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
        if M == 16:
            # the first call on a device resolves the built-in scratch's address (no allocation,
            # but outside the measured window all the same)
            assert _call_static(lib, x, a, pw, r, got) == 0, _lib.last_error()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(0)
        reserved_before = torch.cuda.memory_reserved(0)
        rc = _call_static(lib, x, a, pw, r, got)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(0)
        assert rc == 0, _lib.last_error()
        # the driver's free-memory figure is what a cudaMalloc inside the call would move; torch's
        # own pool did not grow either, so nothing was allocated on the library's behalf
        assert free_after == free_before
        assert torch.cuda.memory_reserved(0) == reserved_before
        _lib.device_status(0)
        assert torch.equal(got, want)  # same kernels, same inputs: identical bits


def test_static_scratch_rejects_oversize_batch():
    torch.cuda.set_device(0)
    _lib.ensure_init(0)
    lib = _lib.load()
    limit = lib.dq_linear_w4a4_int4_static_max_bytes()
    assert limit == 2 * 1024 * 1024 + 16 * 1024
    N, K = 128, 4096
    M = limit // K + 8  # scratch need exceeds the built-in array
    pw = _weights(N, K, 3)
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    rc = _call_static(lib, x, None, pw, None, y)
    assert rc == 6  # DQ_ERR_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
