"""The allocation-free dynamic int8 linear (fixed device scratch array) against the regular kernel-level entry points.

Collected last on purpose: it must pass both alone and after every other GPU test has used the library.
All calls go through the C ABI (ctypes), never through the oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _ffi():
    from vyre_b200 import ffi

    return ffi


def _inputs(m, n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn(m, k, generator=g) * 1.7).to(torch.bfloat16).cuda()
    w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda()
    return x, w


def _regular(ffi, x, w, m, n, k):
    """Existing entry points with a caller-owned buffer for the quantised activations."""
    xq = torch.empty(m, k, dtype=torch.int8, device="cuda")
    sc = torch.empty(m, dtype=torch.float32, device="cuda")
    y = torch.empty(m, n, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ffi.check(ffi.lib().vyb_k_quantize_per_token_int8(x.data_ptr(), xq.data_ptr(), sc.data_ptr(), m, k, stream))
    ffi.check(ffi.lib().vyb_k_int8_gemm_i32(xq.data_ptr(), w.data_ptr(), y.data_ptr(), m, n, k, stream, status.data_ptr()))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    return sc, y


def _static(ffi, x, w, m, n, k):
    sc = torch.empty(m, dtype=torch.float32, device="cuda")
    y = torch.empty(m, n, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    before = torch.cuda.mem_get_info()[0]
    ffi.check(
        ffi.lib().vyb_k_linear_int8_dynamic_static_scratch(
            x.data_ptr(), w.data_ptr(), sc.data_ptr(), y.data_ptr(), m, n, k, stream, status.data_ptr()
        )
    )
    torch.cuda.synchronize()
    after = torch.cuda.mem_get_info()[0]
    assert status.cpu().tolist() == [0, 0, 0, 0]
    return sc, y, before - after


def test_static_scratch_matches_regular_entry_points_twice_in_a_row():
    ffi = _ffi()
    # set-up call: the first call on a device resolves the scratch array's address
    x0, w0 = _inputs(16, 64, 64, seed=1)
    _static(ffi, x0, w0, 16, 64, 64)
    # two calls in a row with different shapes and data: the second must not see leftovers of the first
    for (m, n, k, seed) in [(512, 1024, 4096, 11), (300, 777, 2048, 12)]:
        x, w = _inputs(m, n, k, seed)
        sc_ref, y_ref = _regular(ffi, x, w, m, n, k)
        sc, y, grew = _static(ffi, x, w, m, n, k)
        assert torch.equal(sc, sc_ref)
        assert torch.equal(y, y_ref)  # int32 results are bit-exact
        if m * k >= (2 << 20):  # an allocated activation buffer of this size would show in the device's free memory
            assert grew < (1 << 20), f"device memory in use grew by {grew} bytes across the call"
    # and the first shape again, now after a smaller problem has overwritten part of the array
    x, w = _inputs(512, 1024, 4096, seed=11)
    sc_ref, y_ref = _regular(ffi, x, w, 512, 1024, 4096)
    sc, y, _ = _static(ffi, x, w, 512, 1024, 4096)
    assert torch.equal(sc, sc_ref) and torch.equal(y, y_ref)


def test_static_scratch_largest_shape_and_refusal_beyond_it():
    ffi = _ffi()
    limit = 8 << 20
    m, k, n = 1024, 8192, 512  # m * k == limit exactly
    assert m * k == limit
    x, w = _inputs(m, n, k, seed=21)
    sc_ref, y_ref = _regular(ffi, x, w, m, n, k)
    sc, y, _ = _static(ffi, x, w, m, n, k)
    assert torch.equal(sc, sc_ref) and torch.equal(y, y_ref)

    m2 = m + 1
    x2, w2 = _inputs(m2, n, k, seed=22)
    sc2 = torch.empty(m2, dtype=torch.float32, device="cuda")
    y2 = torch.full((m2, n), -7, dtype=torch.int32, device="cuda")
    rc = ffi.lib().vyb_k_linear_int8_dynamic_static_scratch(
        x2.data_ptr(), w2.data_ptr(), sc2.data_ptr(), y2.data_ptr(), m2, n, k, 0, None
    )
    assert rc == ffi.ERR_INVALID_PROGRAM
    msg = ffi.lib().vyb_last_error_message().decode()
    assert "8388608" in msg and "Fix:" in msg
    torch.cuda.synchronize()
    assert int((y2 != -7).sum()) == 0  # refused before anything was launched
