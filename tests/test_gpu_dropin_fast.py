"""The reference's own operator ids at the sizes it benchmarks and at decode-GEMV sizes. From a size threshold on these
programs are served by kernels shaped for the reference's layouts (kernel variants 5 and 6 of the target payload) rather
than by the kernels that replay the reference's evaluation order. Same contract path as every other op
(compile -> target_compile -> materialize -> submit -> wait), checked against the CPU oracle:

  * bit for bit where every partial sum is exactly representable (dyadic scales, small integer activations: the value
    set of the reference's generated sweep, vyre-libs/src/nn/linear/inner/linear_4bit.rs:1611-1702), because then no
    summation order can change the result;
  * within the reference's drift window for this operator on random data
    (LINEAR_4BIT_AFFINE_GROUPED_OUTPUT_DRIFT_ABS_TOLERANCE = 1e-4, linear_4bit.rs:26; relative 1e-4 for f32
    accumulation where outputs exceed 1).
"""
import numpy as np
import pytest

import oracle
import vyre_b200 as vb

pytestmark = pytest.mark.gpu

DRIFT = 1.0e-4
KV_AFFINE_GROUPED_OUTPUT_MAJOR, KV_I4_MATVEC_WARP_ROWS = 5, 6


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def as_f32(b):
    return np.frombuffer(b, dtype=np.float32)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def affine_inputs(rng, k, n, g, b, dyadic):
    groups = k // g
    packed = rng.integers(0, 2**32, size=(k // 8) * n, dtype=np.uint32)
    zp = rng.integers(0, 16, size=groups * n, dtype=np.uint32)
    if dyadic:
        x = rng.integers(0, 19, size=b * k).astype(np.float32)
        scale = np.array([0.25, 0.5, 1.0, 2.0], dtype=np.float32)[rng.integers(0, 4, size=groups * n)]
        bias = rng.integers(0, 8, size=n).astype(np.float32)
    else:
        x = rng.standard_normal(b * k).astype(np.float32)
        scale = rng.uniform(1e-3, 2e-2, size=groups * n).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
    return x, packed, scale, zp, bias


def affine_program(k, n, g, b):
    if b == 1:
        return vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", k, n, g)
    return vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", k, n, g, b)


# (in_dim, out_dim, group, batch): the reference's benchmark row (1m: K=256, N=4096, g=64, B=256), the decode GEMV shape
# through this operator at 1, 4 and 8 rows, and ragged shapes (outputs, batch and k that fill no tile)
AFFINE_SHAPES = [(256, 4096, 64, 256), (4096, 14336, 128, 1), (4096, 14336, 128, 4), (4096, 14336, 128, 8),
                 (264, 4100, 24, 19), (4096, 1000, 128, 5), (2048, 72, 8, 130)]


@pytest.mark.parametrize("shape", AFFINE_SHAPES)
def test_affine_grouped_large_shapes_take_the_layout_kernel_and_match_the_oracle(dev, shape):
    k, n, g, b = shape
    sess = vb.ArtifactSession.compile(affine_program(k, n, g, b), dev)
    assert sess.kernel_variant() == KV_AFFINE_GROUPED_OUTPUT_MAJOR
    rng = np.random.default_rng(k * 31 + n * 7 + b)
    # exact sums: any order gives the same bits
    args = affine_inputs(rng, k, n, g, b, dyadic=True)
    got = as_f32(sess.run_host(list(args))[0])
    want = oracle.linear_4bit_affine_grouped(*args, k, n, g, batch=b)
    assert np.abs(want).max() < 2**22  # the premise: every partial sum is a multiple of 1/4 below 2^24 quarter-units
    assert bits(got).tolist() == bits(want).tolist()
    # random data: the operator's drift window
    args = affine_inputs(rng, k, n, g, b, dyadic=False)
    got = as_f32(sess.run_host(list(args))[0])
    want = oracle.linear_4bit_affine_grouped(*args, k, n, g, batch=b)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= DRIFT * np.maximum(1.0, np.abs(want))).all(), float(err.max())


def test_affine_grouped_small_shapes_keep_the_reference_order_kernel(dev):
    sess = vb.ArtifactSession.compile(affine_program(256, 512, 64, 8), dev)
    assert sess.kernel_variant() == 0
    # a group that is no multiple of 8 never takes the layout kernel, whatever the size
    sess = vb.ArtifactSession.compile(affine_program(4096, 4096, 4, 8), dev)
    assert sess.kernel_variant() == 0


def pack_rows(values, rows, cols):
    wpr = (cols + 7) // 8
    padded = np.zeros((rows, wpr * 8), dtype=np.int64)
    padded[:, :cols] = values
    nib = (padded & 0xF).astype(np.uint32).reshape(rows, wpr, 8)
    return (nib << (4 * np.arange(8, dtype=np.uint32))).sum(axis=2, dtype=np.uint64).astype(np.uint32).reshape(-1)


def exact_matvec(w, x, scales, batch, rows, cols):
    wpr = (cols + 7) // 8
    nib = ((w.reshape(rows, wpr, 1) >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(rows, wpr * 8)[:, :cols].astype(np.int8)
    signed = np.where(nib >= 8, nib - 16, nib).astype(np.float64)
    xs = x.reshape(batch, cols).astype(np.float64)
    return ((xs @ signed.T) * scales.astype(np.float64)[None, :]).reshape(-1)


# (batch, rows, cols): decode shapes, then rows / batch that fill no tile, a row whose last word is partial (cols % 8 = 4)
# and rows that are not 16-byte multiples (cols % 4 = 2: the scalar path for every word)
MATVEC_SHAPES = [(1, 14336, 4096), (8, 4096, 4096), (11, 1001, 4100), (3, 777, 4102), (64, 256, 256)]


@pytest.mark.parametrize("shape", MATVEC_SHAPES)
@pytest.mark.parametrize("lib_op_id", [False, True])
def test_i4_matvec_large_shapes_take_the_warp_row_kernel_and_match_the_oracle(dev, shape, lib_op_id):
    batch, rows, cols = shape
    if batch == 1:
        prog = vb.i4x8_matvec_f32_scaled("w", "x", "s", "o", rows, cols, lib_op_id=lib_op_id)
    else:
        prog = vb.i4x8_batched_matvec_f32_scaled("w", "x", "s", "o", batch, rows, cols, lib_op_id=lib_op_id)
    sess = vb.ArtifactSession.compile(prog, dev)
    assert sess.kernel_variant() == KV_I4_MATVEC_WARP_ROWS
    rng = np.random.default_rng(rows + cols + batch)
    w = pack_rows(rng.integers(-8, 8, size=(rows, cols)), rows, cols)
    scales = (0.0625 * rng.integers(1, 14, size=rows)).astype(np.float32)
    # the reference generator's value set (multiples of 1/16 in [-1, 1)): exact sums, bit for bit
    x = ((rng.integers(0, 32, size=batch * cols) - 16.0) * 0.0625).astype(np.float32)
    got = as_f32(sess.run_host([w, x, scales])[0])
    want = oracle.i4x8_batched_matvec_f32_scaled(w, x, scales, batch, rows, cols)
    assert bits(got).tolist() == bits(want).tolist()
    # random data. The reference order is one f32 chain over the whole row, which by itself sits up to ~1e-3 from the
    # exact sum at 4096 columns (partial sums of a few hundred, 4096 roundings); a per-element 1e-4 window around THAT
    # value would measure the oracle's rounding, not this kernel's. So: (a) max error relative to the largest output
    # within 1e-4 (f32 accumulation), and (b) against the exact f64 result this kernel is about as close as the reference order or closer
    x = rng.standard_normal(batch * cols).astype(np.float32)
    got = as_f32(sess.run_host([w, x, scales])[0]).astype(np.float64)
    want = oracle.i4x8_batched_matvec_f32_scaled(w, x, scales, batch, rows, cols).astype(np.float64)
    assert np.abs(got - want).max() <= DRIFT * max(1.0, np.abs(want).max())
    exact = exact_matvec(w, x, scales, batch, rows, cols)
    assert np.abs(got - exact).max() <= 1.5 * np.abs(want - exact).max() + 4 * np.spacing(np.float32(np.abs(want).max()))
