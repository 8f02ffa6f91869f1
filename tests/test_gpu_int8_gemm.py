"""GPU parity of the int8 x int8 -> int32 tensor-core GEMM and the per-token quantiser (benchmark config 5):
bit-exact against the CPU oracle on every output (integer arithmetic has no tolerance)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import vyre_b200 as vb
from vyre_b200 import ffi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def gemm_raw(a, w):
    m, k = a.shape
    n = w.shape[0]
    ta, tw = torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda()
    out = torch.full((m, n), -7, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ffi.check(ffi.lib().vyb_k_int8_gemm_i32(ta.data_ptr(), tw.data_ptr(), out.data_ptr(), m, n, k,
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream),
                                            C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    return out.cpu().numpy()


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (1, 1, 16), (5, 7, 48), (127, 255, 112), (129, 257, 144),
                                   (300, 520, 1024), (64, 1000, 4096), (256, 512, 8192)])
def test_int8_gemm_bit_exact(m, n, k):
    rng = np.random.default_rng(m * 131 + n * 7 + k)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    got = gemm_raw(a, w)
    want = oracle.int8_gemm_i32(a, w, m, n, k)
    assert np.array_equal(got, want)


def test_int8_gemm_cta_pair_kernel_ragged_shape_bit_exact():
    """Enough 256 x 256 tiles for the CTA-pair kernel (two waves on 74 pairs), ragged in every dimension: checked on
    the first, a middle and the last rows against the oracle, and on every element against torch's int64 matmul."""
    m, n, k = 2050, 4500, 272
    rng = np.random.default_rng(99)
    a = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    w = rng.integers(-127, 128, size=(n, k), dtype=np.int8)
    assert ((m + 255) // 256) * ((n + 255) // 256) >= 148
    got = gemm_raw(a, w)
    for lo, hi in ((0, 8), (1020, 1030), (m - 6, m)):
        assert np.array_equal(got[lo:hi], oracle.int8_gemm_i32(a, w, m, n, k, row_begin=lo, row_end=hi))
    full = (torch.from_numpy(a).cuda().to(torch.float64) @ torch.from_numpy(w).cuda().to(torch.float64).T).to(torch.int32)
    assert np.array_equal(got, full.cpu().numpy())  # |sum| < 2^53: the f64 product is exact


def test_int8_gemm_extremes_do_not_wrap():
    m, n, k = 128, 256, 8192
    a = np.full((m, k), -127, dtype=np.int8)
    w = np.full((n, k), -127, dtype=np.int8)
    w[::2] = 127
    got = gemm_raw(a, w)
    assert got.max() == 8192 * 127 * 127 and got.min() == -8192 * 127 * 127


def test_linear_int8_dynamic_contract_path(dev):
    m, n, k = 200, 384, 1024
    x, w, _ = synth.int8_dynamic_inputs(m, n, k, seed=3)
    prog = vb.linear_int8_dynamic("x", "w", "x_scale", "out", m, k, n)
    sess = vb.ArtifactSession.compile(prog, dev)
    outs = sess.run_host([x, w, np.zeros(m, np.float32)])
    scales = np.frombuffer(outs[0], np.float32)  # x_scale (ReadWrite, slot 2) comes first in buffer order
    acc = np.frombuffer(outs[1], np.int32).reshape(m, n)
    q_want, s_want = oracle.quantize_per_token_int8(x, m, k)
    assert np.array_equal(scales.view(np.uint32), s_want.view(np.uint32))
    assert np.array_equal(acc, oracle.int8_gemm_i32(q_want, w, m, n, k))


def test_config5_sampled_rows_bit_exact(dev):
    # full K and N of the column-parallel config, a 256-row slab of its 4096 tokens (the CPU check is O(m n k))
    m, n, k = 256, 28672, 8192
    x, w, _ = synth.int8_dynamic_inputs(m, n, k, seed=0)
    q, s = oracle.quantize_per_token_int8(x, m, k)
    got = gemm_raw(q, w)
    rows = [0, 1, 127, 128, 255]
    for r in rows:
        want = oracle.int8_gemm_i32(q, w, m, n, k, row_begin=r, row_end=r + 1)
        assert np.array_equal(got[r:r + 1], want)
    # checksum of the whole slab against int64 numpy on a column sample
    cols = np.arange(0, n, 97)
    ref = q.astype(np.int64) @ w[cols].astype(np.int64).T
    assert np.array_equal(got[:, cols].astype(np.int64), ref)
