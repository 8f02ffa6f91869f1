"""The operators either side of the feed-forward block (learned / gated RMSNorm, residual add) and the GGML K-quant
unpack / fused linear programs, through the contract path on the device against the CPU oracle. Everything is evaluated
in the reference interpreter's order, so results are bit-identical; where exp is involved (the gated norm) the
reference's 128-ULP window applies (vyre-foundation/src/fp_parity.rs:14-16)."""
import numpy as np
import pytest

import oracle
import vyre_b200 as vb
from vyre_b200 import ffi

pytestmark = pytest.mark.gpu
DT = {ffi.DT_F32: oracle.DT_F32, ffi.DT_BF16: oracle.DT_BF16, ffi.DT_F16: oracle.DT_F16}


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def run(dev, program, inputs):
    return vb.ArtifactSession.compile(program, dev).run_host(inputs)


def typed(values, tag):
    v = np.asarray(values, dtype=np.float32)
    if tag == ffi.DT_BF16:
        return oracle.f32_to_bf16_bits(v)
    if tag == ffi.DT_F16:
        return v.astype(np.float16).view(np.uint16)
    return v


def out_of(buf, tag):
    return np.frombuffer(buf, dtype=np.float32 if tag == ffi.DT_F32 else np.uint16)


def test_residual_add_fixture_and_dtypes(dev):
    out = run(dev, vb.residual_add("residual", "branch", "output", 4),
              [np.array([1.0, -2.0, 3.5, 0.0], np.float32), np.array([0.5, 4.0, -1.5, -0.0], np.float32)])[0]
    assert np.frombuffer(out, np.float32).tolist() == [1.5, 2.0, 2.0, 0.0]  # residual_add.rs:53-76
    rng = np.random.default_rng(0)
    for tag in (ffi.DT_F32, ffi.DT_BF16, ffi.DT_F16):
        n = 1000
        a, b = typed(rng.standard_normal(n) * 8, tag), typed(rng.standard_normal(n), tag)
        got = out_of(run(dev, vb.residual_add_typed("r", "b", "o", n, tag), [a, b])[0], tag)
        assert np.array_equal(got, oracle.residual_add(a, b, DT[tag]))
    with pytest.raises(vb.BackendError, match="residual_add_typed requires n > 0"):
        vb.residual_add_typed("r", "b", "o", 0, ffi.DT_F32)
    with pytest.raises(vb.BackendError, match="supports F16, BF16, or F32"):
        vb.residual_add_typed("r", "b", "o", 4, ffi.DT_U32)


@pytest.mark.parametrize("rows,hidden", [(1, 1), (3, 37), (5, 1024), (2, 4096), (4, 1500)])
@pytest.mark.parametrize("tag", [ffi.DT_F32, ffi.DT_BF16, ffi.DT_F16])
def test_learned_rms_norm_against_the_oracle(dev, rows, hidden, tag):
    rng = np.random.default_rng(rows * 7 + hidden)
    x, w = typed(rng.standard_normal(rows * hidden) * 3, tag), typed(1.0 + 0.1 * rng.standard_normal(hidden), tag)
    got = out_of(run(dev, vb.learned_rms_norm("input", "weight", "output", rows, hidden, 1e-6, tag), [x, w])[0], tag)
    want = oracle.rms_norm(x, w, rows, hidden, 1e-6, dtype=DT[tag])
    sess_variant = vb.ArtifactSession.compile(vb.learned_rms_norm("input", "weight", "output", rows, hidden, 1e-6, tag), dev).kernel_variant()
    if hidden < 2048:
        assert sess_variant == 0
        assert np.array_equal(got.view(np.uint32 if tag == ffi.DT_F32 else np.uint16),
                              want.view(np.uint32 if tag == ffi.DT_F32 else np.uint16))
    else:
        # rows of 2048 elements and more: the sum of squares is a tree, not the reference's chain (kernel variant 8); the sum
        # differs by f32 rounding, so f32 outputs agree to a few ulp and 16-bit outputs except for rare one-ulp flips
        assert sess_variant == 8
        if tag == ffi.DT_F32:
            # the chain of 4096 additions carries about sqrt(4096) * 2^-24 = 4e-6 of rounding itself
            assert np.abs(got - want).max() <= 3e-5 * np.abs(want).max()
        else:
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            # a relative difference of a few 1e-6 in 1/rms moves a value across a rounding boundary of an 11-bit (f16) or
            # 8-bit (bf16) significand about once in a thousand
            # (a flipped normalised value times a weight above one can land two ulp away)
            assert diff.max() <= 2 and np.mean(diff != 0) < 0.01


def test_gated_rms_norm_within_the_exp_window(dev):
    rng = np.random.default_rng(9)
    rows, hidden = 3, 640
    x = rng.standard_normal(rows * hidden).astype(np.float32)
    w = rng.standard_normal(hidden).astype(np.float32)
    g = (rng.standard_normal(rows * hidden) * 2).astype(np.float32)
    got = np.frombuffer(run(dev, vb.gated_rms_norm("input", "weight", "gate", "output", rows, hidden, 1e-5, ffi.DT_F32),
                            [x, w, g])[0], np.float32)
    want = oracle.rms_norm(x, w, rows, hidden, 1e-5, gate=g)
    ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    assert ulp.max() <= 128


def test_gated_rms_norm_contract_vectors_on_the_device(dev):
    # vyre-libs/tests/gated_rms_norm_contract.rs: the reference's own known answers
    f = lambda a: np.array(a, np.float32)  # noqa: E731
    u = lambda a: np.array(a, np.uint16)  # noqa: E731
    gated = lambda rows, hidden, eps, tag, ins: run(dev, vb.gated_rms_norm("i", "w", "g", "o", rows, hidden, eps, tag), ins)[0]  # noqa: E731
    got = np.frombuffer(gated(2, 4, 1e-6, ffi.DT_F32, [f([1.0, -2.0, 3.0, -4.0, 0.25, -0.5, 2.0, 1.0]), f([0.5, 1.5, -1.0, 2.0]),
                                                        f([-3.0, 0.0, 2.0, 8.0, -1.0, 1.0, -8.0, 3.0])]), np.float32)
    want = f([-0.025976218, 0.0, -1.9297296, -23.361658, -0.029170781, -0.47576645, 0.0046558483, 4.9594145])
    assert np.abs(got - want).max() <= 3e-6  # :72-101, the reference's tolerance
    got = np.frombuffer(gated(2, 4, 1e-6, ffi.DT_F32, [np.zeros(8, np.float32), f([1, -2, 3, -4]),
                                                        f([-100, -1, 0, 100, 1, 2, 3, 4])]), np.float32)
    assert np.all(got == 0.0)  # :104-116
    small = np.frombuffer(gated(1, 2, 1e-12, ffi.DT_F32, [f([1e-8, -1e-8]), f([1, 1]), f([1, 1])]), np.float32)
    large = np.frombuffer(gated(1, 2, 1e-4, ffi.DT_F32, [f([1e-8, -1e-8]), f([1, 1]), f([1, 1])]), np.float32)
    assert 0.007 < small[0] < 0.008 and 7e-7 < large[0] < 8e-7 and small[0] > large[0] * 9000.0  # :119-129
    got = np.frombuffer(gated(2, 2, 1e-6, ffi.DT_F32, [f([np.nan, 1.0, 3.0, 4.0]), f([1, 1]), f([1, 1, 1, 1])]), np.float32)
    assert np.isnan(got[0]) and np.isnan(got[1]) and np.abs(got[2:] - f([0.6203238, 0.8270984])).max() <= 3e-6  # :132-144
    got = np.frombuffer(gated(1, 2, 1e-6, ffi.DT_F16, [u([0x3C00, 0xC000]), u([0x3C00, 0x3800]), u([0x3C00, 0xBC00])]), np.uint16)
    assert got.tolist() == [0x3765, 0x3171]  # :170-212, exact words
    got = np.frombuffer(gated(1, 2, 1e-6, ffi.DT_BF16, [u([0x3F80, 0xC000]), u([0x3F80, 0x3F00]), u([0x3F80, 0xBF80])]), np.uint16)
    assert got.tolist() == [0x3EED, 0x3E2E]
    prog = vb.gated_rms_norm_with_weight_dtype("x", "w", "g", "y", 1, 2, 1e-6, ffi.DT_BF16, ffi.DT_F32)  # :214-246
    assert [b["dtype"] for b in prog.buffers()] == [ffi.DT_BF16, ffi.DT_F32, ffi.DT_BF16, ffi.DT_BF16]
    got = np.frombuffer(run(dev, prog, [u([0x3F80, 0xC000]), f([1.0, 0.5]), u([0x3F80, 0xBF80])])[0], np.uint16)
    assert got.tolist() == [0x3EED, 0x3E2E]
    with pytest.raises(vb.BackendError, match="supports F16, BF16, or F32 source tensors"):  # :248-257
        vb.gated_rms_norm_with_weight_dtype("x", "w", "g", "y", 1, 2, 1e-6, ffi.DT_BF16, ffi.DT_U32)


def test_rms_norm_construction_errors():
    with pytest.raises(vb.BackendError, match="requires nonzero rows and hidden size; got rows=0, hidden=8"):
        vb.learned_rms_norm("i", "w", "o", 0, 8, 1e-6, ffi.DT_F32)
    with pytest.raises(vb.BackendError, match="supports F16, BF16, or F32 source tensors"):
        vb.learned_rms_norm("i", "w", "o", 2, 8, 1e-6, ffi.DT_U32)
    with pytest.raises(vb.BackendError, match="rows\\*hidden overflows u32"):
        vb.learned_rms_norm("i", "w", "o", 1 << 20, 1 << 13, 1e-6, ffi.DT_F32)


def test_k_quant_reference_fixtures_on_the_device(dev):
    # ggml.rs:392-474
    out = run(dev, vb.q4_k_unpack("packed", "scales", "mins", "out", 16),
              [np.array([0x76543210, 0xFEDCBA98, 0, 0], np.uint32), np.array([1.0], np.float32), np.array([0.0], np.float32)])[0]
    assert np.frombuffer(out, np.float32).tolist() == [float(i) for i in range(16)]
    out = run(dev, vb.q2_k_unpack("packed", "scales", "mins", "out", 16),
              [np.array([0xE4E4E4E4], np.uint32), np.array([1.0], np.float32), np.array([0.0], np.float32)])[0]
    assert np.frombuffer(out, np.float32).tolist() == [0.0, 1.0, 2.0, 3.0] * 4
    x = np.zeros(32, np.float32)
    x[31] = 1.0
    out = run(dev, vb.q4_k_linear("x", "packed", "scales", "mins", "b", "out", 32, 2),
              [x, np.full(8, 0x11111111, np.uint32), np.array([1.0, 2.0], np.float32), np.zeros(2, np.float32),
               np.array([0.5, 1.5], np.float32)])[0]
    assert np.frombuffer(out, np.float32).tolist() == [2.5, 3.5]


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("in_dim,out_dim", [(1, 1), (7, 5), (32, 2), (96, 33), (256, 1024), (1000, 130)])
def test_k_quant_unpack_and_linear_bit_identical(dev, bits, in_dim, out_dim):
    rng = np.random.default_rng(bits * 1000 + in_dim + out_dim)
    block, wpb = (32, 4) if bits == 4 else (16, 1)
    n = in_dim * out_dim
    blocks = -(-n // block)
    packed = rng.integers(0, 2**32, size=blocks * wpb, dtype=np.uint32)
    scales = rng.uniform(0.01, 0.2, size=blocks).astype(np.float32)
    mins = (-rng.uniform(0.0, 1.0, size=blocks)).astype(np.float32)
    unpack = vb.q4_k_unpack if bits == 4 else vb.q2_k_unpack
    got = np.frombuffer(run(dev, unpack("p", "s", "m", "o", n), [packed, scales, mins])[0], np.float32)
    want = oracle.k_quant_unpack(packed, scales, mins, n, bits)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    x, b = rng.standard_normal(in_dim).astype(np.float32), rng.standard_normal(out_dim).astype(np.float32)
    linear = vb.q4_k_linear if bits == 4 else vb.q2_k_linear
    got = np.frombuffer(run(dev, linear("x", "p", "s", "m", "b", "o", in_dim, out_dim), [x, packed, scales, mins, b])[0], np.float32)
    want = oracle.k_quant_linear(x, packed, scales, mins, b, in_dim, out_dim, bits)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # against dequantise-then-matmul in f64: the fused form computes the same linear map
    deq = oracle.k_quant_unpack(packed, scales, mins, n, bits).astype(np.float64).reshape(in_dim, out_dim)
    assert np.allclose(got, x.astype(np.float64) @ deq + b, rtol=1e-4, atol=1e-4 * max(1.0, np.abs(want).max()))


def test_k_quant_construction_errors():
    with pytest.raises(vb.BackendError, match="vyre-libs::quant::q4_k_unpack n=0 is invalid"):
        vb.q4_k_unpack("p", "s", "m", "o", 0)
    with pytest.raises(vb.BackendError, match="vyre-libs::quant::q2_k_linear all dims must be > 0"):
        vb.q2_k_linear("x", "p", "s", "m", "b", "o", 0, 4)
    with pytest.raises(vb.BackendError, match="vyre-libs::quant::q4_k_linear dimensions overflow u32"):
        vb.q4_k_linear("x", "p", "s", "m", "b", "o", 1 << 17, 1 << 17)


@pytest.mark.parametrize("bits,in_dim,out_dim", [(4, 4096, 4096), (2, 4096, 4096), (4, 1100, 1056), (2, 2048, 576), (4, 14336, 4096)])
def test_k_quant_linear_large_shapes_take_the_word_column_kernel(dev, bits, in_dim, out_dim):
    rng = np.random.default_rng(bits + in_dim)
    block, wpb = (32, 4) if bits == 4 else (16, 1)
    blocks = -(-(in_dim * out_dim) // block)
    linear = vb.q4_k_linear if bits == 4 else vb.q2_k_linear
    sess = vb.ArtifactSession.compile(linear("x", "p", "s", "m", "b", "o", in_dim, out_dim), dev)
    assert sess.kernel_variant() == 7
    packed = rng.integers(0, 2**32, size=blocks * wpb, dtype=np.uint32)
    # exact sums (dyadic scales and minimums, small integer activations): any order gives the same bits
    scales = np.array([0.25, 0.5, 1.0, 2.0], np.float32)[rng.integers(0, 4, size=blocks)]
    mins = -np.array([0.0, 0.5, 1.0, 4.0], np.float32)[rng.integers(0, 4, size=blocks)]
    x, b = rng.integers(-4, 5, size=in_dim).astype(np.float32), rng.integers(0, 8, size=out_dim).astype(np.float32)
    got = np.frombuffer(sess.run_host([x, packed, scales, mins, b])[0], np.float32)
    want = oracle.k_quant_linear(x, packed, scales, mins, b, in_dim, out_dim, bits)
    assert np.abs(want).max() < 2**22
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # random data: f32 accumulation in another order
    scales = rng.uniform(0.01, 0.2, size=blocks).astype(np.float32)
    mins = (-rng.uniform(0.0, 1.0, size=blocks)).astype(np.float32)
    x, b = rng.standard_normal(in_dim).astype(np.float32), rng.standard_normal(out_dim).astype(np.float32)
    got = np.frombuffer(sess.run_host([x, packed, scales, mins, b])[0], np.float32)
    want = oracle.k_quant_linear(x, packed, scales, mins, b, in_dim, out_dim, bits)
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())


def test_k_quant_linear_small_or_unaligned_shapes_keep_the_reference_order(dev):
    assert vb.ArtifactSession.compile(vb.q4_k_linear("x", "p", "s", "m", "b", "o", 256, 1024), dev).kernel_variant() == 0
    assert vb.ArtifactSession.compile(vb.q2_k_linear("x", "p", "s", "m", "b", "o", 4096, 1056), dev).kernel_variant() == 0
