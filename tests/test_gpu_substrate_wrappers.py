"""The scratch-reusing int4 wrappers on the device, against the CPU oracle and against the reference's own small cases
(vyre-self-substrate/src/math/quantized_dispatch/tests.rs builds its expectations with the `*_cpu` functions the oracle
restates). Integer and dyadic cases bit for bit; a repeated shape is served from the scratch (no second compilation)."""
import numpy as np
import pytest

import oracle
import vyre_b200 as vb

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


@pytest.fixture()
def scratch(dev):
    s = vb.QuantizedScratch(dev)
    yield s
    s.close()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).tolist()


def pack_rows(rng, rows, cols):
    vals = rng.integers(-8, 8, size=(rows, cols))
    return np.concatenate([oracle.pack_i4x8(vals[r]) for r in range(rows)]), vals


def test_unpack_and_dot(scratch):
    rng = np.random.default_rng(1)
    for lanes in (1, 7, 8, 9, 96, 1000):
        vals = rng.integers(-8, 8, size=lanes)
        packed = oracle.pack_i4x8(vals)
        assert vb.unpack_i4x8_via(scratch, packed, lanes).tolist() == vals.tolist()
        other = oracle.pack_i4x8(rng.integers(-8, 8, size=lanes))
        got = vb.i4x8_dot_f32_scaled_via(scratch, packed, other, 0.5, 0.25, lanes)
        assert bits([got]) == bits([oracle.i4x8_dot_f32_scaled(packed, other, 0.5, 0.25, lanes)])
    st = scratch.stats()
    assert st["cached"] == 12 and st["misses"] == 12 and st["hits"] == 0
    # the same shape again: served from the scratch
    vb.unpack_i4x8_via(scratch, oracle.pack_i4x8(np.arange(-4, 3)), 7)
    assert scratch.stats()["hits"] == 1 and scratch.stats()["cached"] == 12


@pytest.mark.parametrize("batch,rows,cols", [(1, 5, 9), (3, 17, 40), (8, 4096, 4096)])
def test_matvec_and_batched_matvec(scratch, batch, rows, cols):
    rng = np.random.default_rng(rows + cols)
    w, _ = pack_rows(rng, rows, cols)
    x = ((rng.integers(0, 32, size=batch * cols) - 16.0) * 0.0625).astype(np.float32)  # exact sums in any order
    scales = (0.0625 * rng.integers(1, 14, size=rows)).astype(np.float32)
    got = vb.i4x8_batched_matvec_f32_scaled_via(scratch, w, x, scales, batch, rows, cols)
    assert bits(got) == bits(oracle.i4x8_batched_matvec_f32_scaled(w, x, scales, batch, rows, cols))
    one = vb.i4x8_matvec_f32_scaled_via(scratch, w, x[:cols], scales, rows, cols)
    assert bits(one) == bits(oracle.i4x8_batched_matvec_f32_scaled(w, x[:cols], scales, 1, rows, cols))
    again = vb.i4x8_batched_matvec_f32_scaled_via(scratch, w, x, scales, batch, rows, cols)
    assert bits(again) == bits(got) and scratch.stats()["hits"] == 1


@pytest.mark.parametrize("batch,rows,cols", [(1, 3, 8), (4, 9, 33), (16, 96, 96)])
def test_batched_matmul_and_top1(scratch, batch, rows, cols):
    rng = np.random.default_rng(batch * 100 + rows)
    w, _ = pack_rows(rng, rows, cols)
    a, _ = pack_rows(rng, batch, cols)
    rs = (0.25 * rng.integers(1, 9, size=rows)).astype(np.float32)
    bs = (0.5 * rng.integers(1, 5, size=batch)).astype(np.float32)
    got = vb.i4x8_batched_matmul_f32_scaled_via(scratch, w, a, rs, bs, batch, rows, cols)
    want = oracle.i4x8_batched_matmul_f32_scaled(w, a, rs, bs, batch, rows, cols)
    assert bits(got) == bits(want)
    scores, idx = vb.i4x8_batched_matmul_top1_f32_scaled_via(scratch, w, a, rs, bs, batch, rows, cols)
    both = oracle.i4x8_batched_matmul_top1_f32_scaled(w, a, rs, bs, batch, rows, cols)
    assert bits(scores) == bits(both[:batch])
    assert idx.tolist() == both[batch:].astype(np.uint32).tolist()
    # the winner is the first maximum of the full product
    full = want.reshape(batch, rows)
    assert idx.tolist() == np.argmax(full, axis=1).tolist()


def test_errors_leave_the_scratch_usable(scratch):
    with pytest.raises(vb.BackendError):
        vb.i4x8_matvec_f32_scaled_via(scratch, np.zeros(5, np.uint32), np.zeros(9, np.float32), np.zeros(3, np.float32), 3, 9)
    w = oracle.pack_i4x8(np.array([1, -2, 3, -4, 5, -6, 7, -8, 1]))
    out = vb.i4x8_matvec_f32_scaled_via(scratch, w, np.ones(9, np.float32), np.array([2.0], np.float32), 1, 9)
    assert out.tolist() == [-6.0]


def test_scratch_keeps_its_device_alive():
    # the caller may release its device handle first; the scratch is a second owner until it is closed
    d = vb.Device.acquire(0)
    s = vb.QuantizedScratch(d)
    d.release()
    w = oracle.pack_i4x8(np.array([1, -2, 3, -4, 5, -6, 7, -8, 1]))
    out = vb.i4x8_matvec_f32_scaled_via(s, w, np.ones(9, np.float32), np.array([2.0], np.float32), 1, 9)
    assert out.tolist() == [-6.0]
    s.close()
