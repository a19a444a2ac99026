"""Failure detection of the all-reduce fused into the decode GEMM, without a second rank and without
a fault: a world-2 context whose "peer" buffers are local arrays that nobody ever flags makes the
bounded wait run out; the kernel returns, the status word reports DQ_ERR_TIMEOUT with the all-reduce
site code, and the library keeps working afterwards."""
import ctypes

import pytest
import torch

from dualquant_b200 import _lib, ops, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_missing_peer_times_out_and_reports_site():
    M, N, K = 8, 512, 1024
    w = synthetic.make_w(N, K, 2)
    codes_w, sw = ops.quant_w_int4(w.to(DEV))
    pw = ops.pack_w_int4(codes_w, sw)
    x = synthetic.make_x(M, K, 2)
    codes, sx = ops.quant_act_int4(x.to(DEV), None, None, False)
    cap, units = 16 * 4096, 1024
    bufs = torch.zeros(2, 2 * cap, dtype=torch.float32, device=DEV)
    flags = torch.zeros(2, units * 8, dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = _lib.AllReduceCtx()
    ctx.world, ctx.rank = 2, 0
    for p in range(2):
        ctx.buf_ptrs[p] = bufs[p].data_ptr()
        ctx.flag_ptrs[p] = flags[p].data_ptr()
    ctx.seq = seq.data_ptr()
    ctx.buf_capacity_floats = cap
    ctx.flag_units = units
    y = torch.full((M, N), 7.0, dtype=torch.float32, device=DEV)
    lib = _lib.load()
    _lib.set_tuning("ar_wait_log2", 25)  # about 17 ms instead of half a second
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.dq_gemm_w4a4_int4_ar(ctypes.c_void_p(codes.data_ptr()), ctypes.c_void_p(sx.data_ptr()),
                                      ctypes.c_void_p(pw.w_packed.data_ptr()), ctypes.c_void_p(pw.sw_t.data_ptr()),
                                      None, M, N, K, 128, ctypes.c_void_p(y.data_ptr()), _lib.DTYPE_F32,
                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.byref(ctx))
        t1.record()
        assert rc == 0  # the launch itself succeeds; the expiry is reported through the status word
        with pytest.raises(RuntimeError, match="DQ_ERR_TIMEOUT.*site 23"):
            _lib.device_status(0)
        assert t0.elapsed_time(t1) < 2000.0  # the wait is bounded
    finally:
        _lib.set_tuning("ar_wait_log2", 0)
    assert torch.all(y == 7.0)       # rows of a tile whose peers never arrived are not written
    assert int(seq.item()) == 1      # the call counter still advanced
    _lib.device_status(0)            # the word was cleared: clean status
    # and the context is usable: a plain GEMM right after gives the right answer
    y2 = ops.gemm_w4a4_int4(codes, sx, pw, None)
    _lib.device_status(0)
    from oracle import dq_oracle as O

    qx, sxo, _ = O.quant_act_int4(x, None, None, False)
    ref = O.dequant_matmul(qx, sxo, *O.quant_w_int4(w))
    assert ((y2.double().cpu() - ref).abs().max() / ref.abs().max()) < 1e-5


def test_exchange_barrier_without_peer_times_out_once():
    """The device-side barrier of the token-sharded prompt pass, same construction: the "peer" of a
    world-2 context is a local array nobody writes.  The first barrier gives up after the (lowered)
    limit and records site 24; a second barrier issued while the word is still set does not wait
    again; the status call reports and clears the word; nothing faults."""
    T, H = 512, 128
    part = torch.zeros(2, 2, T // 2, H, dtype=torch.bfloat16, device=DEV)
    codes = torch.zeros(2, T, H, dtype=torch.uint8, device=DEV)
    sx = torch.zeros(2, T, dtype=torch.float32, device=DEV)
    flags = torch.zeros(2, 8, dtype=torch.int32, device=DEV)
    ctx = _lib.ExchangeCtx()
    ctx.world, ctx.rank = 2, 0
    for p in range(2):
        ctx.part_ptrs[p] = part[p].data_ptr()
        ctx.codes_ptrs[p] = codes[p].data_ptr()
        ctx.sx_ptrs[p] = sx[p].data_ptr()
        ctx.flag_ptrs[p] = flags[p].data_ptr()
    ctx.tokens_per_rank, ctx.hidden = T // 2, H
    lib = _lib.load()
    _lib.ensure_init(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.set_tuning("ar_wait_log2", 26)  # about 35 ms
    try:
        t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        t0.record()
        assert lib.dq_exchange_barrier(ctypes.byref(ctx), 1, stream) == 0
        t1.record()
        assert lib.dq_exchange_barrier(ctypes.byref(ctx), 2, stream) == 0
        t2.record()
        with pytest.raises(RuntimeError, match="DQ_ERR_TIMEOUT.*site 24"):
            _lib.device_status(0)
        first, second = t0.elapsed_time(t1), t1.elapsed_time(t2)
        assert 5.0 < first < 2000.0      # waited, but not for long
        assert second < first / 4        # the second barrier saw the word and returned at once
    finally:
        _lib.set_tuning("ar_wait_log2", 0)
    assert int(flags[1, 0].item()) == 2  # this rank's word did reach the "peer" both times
    _lib.device_status(0)                # cleared
    # epoch 0: the kernel counts this rank's barriers itself (the form a captured graph can replay)
    count = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx.barrier_count = count.data_ptr()
    flags.zero_()
    _lib.set_tuning("ar_wait_log2", 22)
    try:
        for _ in range(3):
            assert lib.dq_exchange_barrier(ctypes.byref(ctx), 0, stream) == 0
        with pytest.raises(RuntimeError, match="DQ_ERR_TIMEOUT.*site 24"):
            _lib.device_status(0)
    finally:
        _lib.set_tuning("ar_wait_log2", 0)
    assert int(count.item()) == 3 and int(flags[1, 0].item()) == 3
