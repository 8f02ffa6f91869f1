"""The failure path of the cross-GPU kernels, on ONE GPU and without any fault: a device-side wait on a peer that never
signals runs into its clock limit, the kernel returns with a status bit set, later launches return at once, and the
device stays usable. The "peer" is this GPU itself: the context's peer addresses alias local buffers, so no other rank
exists that could signal, and no kernel here waits on another kernel.
"""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from vyre_b200 import ffi, synth

pytestmark = pytest.mark.gpu

LIMIT_CLOCKS = 4_000_000  # about 2 ms at boost clocks


def test_allgather_push_wait_runs_out_and_device_stays_usable():
    L = ffi.lib()
    m, n, world = 1, 1024, 2
    data_bytes = 2 * world * m * n * 2
    buf = torch.zeros(data_bytes + 256, dtype=torch.uint8, device="cuda")
    local = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctx = ffi.AllGatherCtx()
    ctx.world, ctx.rank = world, 0
    for r in range(world):  # both "ranks" are this buffer: the peer's counters are our own, and nobody bumps the one we poll
        ctx.peer_out[r] = buf.data_ptr()
        ctx.peer_flag[r] = buf.data_ptr() + data_bytes
    ctx.epoch = local.data_ptr()
    ctx.wait_clocks = LIMIT_CLOCKS
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def push(half):
        ffi.check(L.vyb_k_allgather_push(C.byref(ctx), half, m, n, stream, C.c_void_p(status.data_ptr())))

    push(0)  # first push: nothing to wait for
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    t0 = time.perf_counter()
    push(1)  # must see one push from the peer first: it never comes
    torch.cuda.synchronize()
    first = time.perf_counter() - t0
    assert status.cpu()[0].item() & 128, "the wait did not report running out"
    assert first < 1.0, "the wait limit of the context was not honoured"
    t0 = time.perf_counter()
    for half in (0, 1, 0, 1):  # a wait that has run out is not repeated: these return at once
        push(half)
    ffi.check(L.vyb_k_allgather_wait(C.byref(ctx), stream, C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < max(0.05, 2 * first)
    # the status word turns into DispatchFailed on the contract path (vyb_submission_wait); here: the device still works
    status.zero_()
    x, w, s = synth.int4_linear_inputs(1, 256, 4096, seed=1)
    tx, tw, ts = (torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
    y = torch.zeros((1, 256), dtype=torch.bfloat16, device="cuda")
    ffi.check(L.vyb_k_int4_gemv(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), y.data_ptr(), 1, 256, 4096, 128, ffi.DT_BF16,
                                stream, C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0] and torch.isfinite(y.float()).all()


def test_gathering_gemv_single_rank_matches_plain_kernel_and_keeps_its_books():
    """vyb_k_int4_gemv_allgather with a one-rank context: the outputs land in this rank's slice of the named half and
    equal the plain kernel's bit for bit; the launch index passes from half to half; the wait kernel settles the signal."""
    from vyre_b200 import sharding

    L = ffi.lib()
    for m, n, k in [(1, 14336, 4096), (3, 1000, 2048), (4, 333, 4096)]:
        x, w, s = synth.int4_linear_inputs(m, n, k, seed=m)
        tx, tw, ts = (torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        want = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ffi.check(L.vyb_k_int4_gemv(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), want.data_ptr(), m, n, k, 128, ffi.DT_BF16,
                                    C.c_void_p(stream), C.c_void_p(status.data_ptr())))
        pag = sharding.PeerAllGather.__new__(sharding.PeerAllGather)
        pag.ffi, pag.torch, pag.world, pag.rank, pag.m, pag.n = ffi, torch, 1, 0, m, n
        pag.data_bytes = (2 * m * n * 2 + 255) & ~255
        pag.buf = torch.zeros(pag.data_bytes + 256, dtype=torch.uint8, device="cuda")
        pag.local = torch.zeros(64, dtype=torch.int32, device="cuda")
        pag.ctx = ffi.AllGatherCtx()
        pag.ctx.world, pag.ctx.rank = 1, 0
        pag.ctx.peer_out[0], pag.ctx.peer_flag[0] = pag.buf.data_ptr(), pag.buf.data_ptr() + pag.data_bytes
        pag.ctx.epoch = pag.local.data_ptr()
        for step in range(5):
            pag.gemv(step & 1, tx, tw, ts, k, stream, status, ffi.LAUNCH_CONSTANT_WEIGHTS)
        pag.wait(stream, status)
        torch.cuda.synchronize()
        assert status.cpu().tolist() == [0, 0, 0, 0]
        for half in (0, 1):
            assert torch.equal(pag.halves()[half][0].view(torch.int16), want.view(torch.int16)), (m, n, k, half)
        words = pag.local.cpu().tolist()
        assert words[0] == 5 and words[10] == 4 and words[11] == 5 and words[12] == 0, words[:16]
        # the pipelined form keeps its outputs local until the next launch (or the wait) carries them over
        pag.halves().zero_()
        for step in range(5, 8):
            pag.gemv(step & 1, tx, tw, ts, k, stream, status, ffi.LAUNCH_CONSTANT_WEIGHTS | ffi.LAUNCH_PIPELINED_GATHER)
        torch.cuda.synchronize()
        assert pag.local.cpu().tolist()[13] == 2  # launch 7 wrote half 1 (marker = half + 1) and left it to its successor
        pag.wait(stream, status)
        torch.cuda.synchronize()
        assert status.cpu().tolist() == [0, 0, 0, 0] and pag.local.cpu().tolist()[13] == 0
        for half in (0, 1):
            assert torch.equal(pag.halves()[half][0].view(torch.int16), want.view(torch.int16)), (m, n, k, half, "pipelined")


def test_gathering_gemv_wait_on_a_silent_peer_runs_out():
    """Two ranks in the context, both this GPU, nobody else to signal: the second launch's check of its peer runs into
    the clock limit, raises status bit 128, and the device stays usable (no fault, no hang)."""
    L = ffi.lib()
    m, n, k, world = 1, 2048, 4096, 2
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=9)
    tx, tw, ts = (torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
    data_bytes = 2 * world * m * n * 2
    buf = torch.zeros(data_bytes + 256, dtype=torch.uint8, device="cuda")
    local = torch.zeros(64, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ctx = ffi.AllGatherCtx()
    ctx.world, ctx.rank = world, 0
    for r in range(world):
        ctx.peer_out[r] = buf.data_ptr()
        ctx.peer_flag[r] = buf.data_ptr() + data_bytes
    ctx.epoch = local.data_ptr()
    ctx.wait_clocks = LIMIT_CLOCKS
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def gemv(half):
        ffi.check(L.vyb_k_int4_gemv_allgather(C.byref(ctx), half, tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), m, n, k, 128, 0,
                                              stream, C.c_void_p(status.data_ptr())))

    gemv(0)  # launch 0 needs nothing from its peer
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    t0 = time.perf_counter()
    gemv(1)  # launch 1 needs the peer's signal for launch 0: it never comes
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert status.cpu()[0].item() & 128
    t0 = time.perf_counter()
    gemv(0)  # not waited for again
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    status.zero_()
    y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    ffi.check(L.vyb_k_int4_gemv(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), y.data_ptr(), m, n, k, 128, ffi.DT_BF16, stream,
                                C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0] and torch.isfinite(y.float()).all()
