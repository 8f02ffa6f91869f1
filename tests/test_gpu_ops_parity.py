"""GPU parity of the reference operator surface: every op runs through the C-ABI contract path
(compile -> target_compile -> materialize -> submit -> wait) on the device and is compared with the CPU
oracle / the reference's golden fixtures. Bit-exact for integer outputs and for f32 ops evaluated in the
reference order; the reference's 128-ULP window where exp is involved (vyre-foundation/src/fp_parity.rs:14-16).
"""
import numpy as np
import pytest

import oracle
import vyre_b200 as vb
from vyre_b200 import ffi

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)  # a missing device is a loud failure, never a skip
    yield d
    d.release()


def f32(*v):
    return np.array(v, dtype=np.float32)


def u32(*v):
    return np.array(v, dtype=np.uint32)


def run(dev, program, inputs):
    return vb.ArtifactSession.compile(program, dev).run_host(inputs)


def as_f32(b):
    return np.frombuffer(b, dtype=np.float32)


def as_u32(b):
    return np.frombuffer(b, dtype=np.uint32)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def max_ulp(a, b):
    L = oracle.lib()
    return max((L.vyo_ulp_distance(float(x), float(y)) for x, y in zip(a, b)), default=0)


# ---- reference generators (vyre-driver-cuda/tests/int4_quantized_gpu_parity.rs:209-245) -------------------------
def generated_i4_values(n, seed):
    state = (seed ^ 0x9E3779B9) & 0xFFFFFFFF
    out = []
    for index in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        r = index % 17
        state = ((state << r) | (state >> (32 - r))) & 0xFFFFFFFF if r else state
        out.append((state >> 28) - 8)
    return np.array(out, dtype=np.int32)


def generated_f32_values(n, seed):
    state = (seed ^ 0xA5A55A5A) & 0xFFFFFFFF
    out = []
    for index in range(n):
        state = (state * 747796405 + 2891336453) & 0xFFFFFFFF
        r = index % 11
        state = ((state >> r) | (state << (32 - r))) & 0xFFFFFFFF if r else state
        out.append((((state >> 27) & 0x1F) - 16.0) * 0.0625)
    return np.array(out, dtype=np.float32)


def generated_positive_scales(n, seed):
    return np.array([0.0625 * (1 + ((seed + i * 3) % 13)) for i in range(n)], dtype=np.float32)


def pack_rows(rows):
    return np.concatenate([oracle.pack_i4x8(r) for r in rows])


# ---- registry fixtures -------------------------------------------------------------------------------------------
def test_linear_4bit_registry_fixture(dev):
    out = run(dev, vb.linear_4bit("x", "w", "b", "out", 8, 4),
              [np.arange(8, dtype=np.float32), u32(0x76543210, 0xFEDCBA98, 0x11111111, 0), np.zeros(4, np.float32)])
    assert as_f32(out[0]).tolist() == [140.0, 364.0, 28.0, 0.0]


def test_affine_grouped_registry_fixtures(dev):
    x = np.arange(1, 9, dtype=np.float32)
    args = [u32(0x87654321, 0), f32(0.5, 1.0, 2.0, 1.0), u32(1, 0, 4, 0), f32(0.0, 3.0)]
    out = run(dev, vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 8, 2, 4), [x] + args)
    assert as_f32(out[0]).tolist() == [150.0, 3.0]  # trimmed by output_byte_range
    xb = np.concatenate([x, np.zeros(8, np.float32)])
    out = run(dev, vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", 8, 2, 4, 2), [xb] + args)
    assert as_f32(out[0]).tolist() == [150.0, 3.0, 0.0, 3.0]
    act = np.repeat(np.arange(1, 9, dtype=np.float32), 256)
    out = run(dev, vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", 256, 8, 64, 8),
              [act, np.full(256, 0x11111111, np.uint32), np.ones(32, np.float32), np.zeros(32, np.uint32),
               np.arange(8, dtype=np.float32)])
    assert as_f32(out[0]).tolist() == [256.0 * (b + 1) + o for b in range(8) for o in range(8)]
    out = run(dev, vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 8, 2, 8),
              [np.ones(8, np.float32), np.zeros(2, np.uint32), f32(2.0, 0.5), u32(15, 14), f32(0.0, 1.0)])
    assert as_f32(out[0]).tolist() == [-240.0, -55.0]


def test_affine_grouped_generated_sweep_matches_oracle_bit_for_bit(dev):
    # linear_4bit.rs:1611-1702 shapes, every seed third; plus non-dyadic inputs where order matters
    rng = np.random.default_rng(7)
    for out_dim in [1, 3, 8, 13, 32]:
        for group in [1, 4, 8, 32]:
            prog = vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 32, out_dim, group)
            sess = vb.ArtifactSession.compile(prog, dev)
            groups = 32 // group
            for seed in range(0, 48, 3):
                x = np.array([((k * 3 + seed) % 19) for k in range(32)], dtype=np.float32)
                packed = rng.integers(0, 2**32, size=4 * out_dim, dtype=np.uint32)
                scale = np.array([[0.25, 0.5, 1.0, 2.0][(g + o + seed) & 3] for g in range(groups)
                                  for o in range(out_dim)], dtype=np.float32)
                zp = np.array([(g * 5 + o + seed) & 0xF for g in range(groups) for o in range(out_dim)], np.uint32)
                bias = np.array([(o + seed) & 7 for o in range(out_dim)], dtype=np.float32)
                got = as_f32(sess.run_host([x, packed, scale, zp, bias])[0])
                want = oracle.linear_4bit_affine_grouped(x, packed, scale, zp, bias, 32, out_dim, group)
                assert bits(got).tolist() == bits(want).tolist()
    # the case the reference benchmarks (K=256, N=4096, g=64) with random non-dyadic data, batch 8
    k, n, g, b = 256, 512, 64, 8
    x = rng.standard_normal(b * k).astype(np.float32)
    packed = rng.integers(0, 2**32, size=(k // 8) * n, dtype=np.uint32)
    scale = rng.uniform(0.01, 1.0, size=(k // g) * n).astype(np.float32)
    zp = rng.integers(0, 16, size=(k // g) * n, dtype=np.uint32)
    bias = rng.standard_normal(n).astype(np.float32)
    got = as_f32(run(dev, vb.linear_4bit_affine_grouped_batched("x", "w", "s", "zp", "b", "out", k, n, g, b),
                     [x, packed, scale, zp, bias])[0])
    want = oracle.linear_4bit_affine_grouped(x, packed, scale, zp, bias, k, n, g, batch=b)
    assert bits(got).tolist() == bits(want).tolist()


def test_int4_primitive_fixtures_and_boundary_shapes(dev):
    w = u32(0x76210F98)
    out = run(dev, vb.unpack_i4x8("p", "o", 8), [w, np.zeros(8, np.int32)])
    assert np.frombuffer(out[0], np.int32).tolist() == [-8, -7, -1, 0, 1, 2, 6, 7]
    assert np.frombuffer(run(dev, vb.i4x8_dot_i32("l", "r", "o", 8), [w, w])[0], np.int32).tolist() == [204]
    assert np.frombuffer(run(dev, vb.i4x8_dot_i32("l", "r", "o", 8, lib_op_id=True),
                             [u32(0xCDEF4321), u32(0xFEDC1234)])[0], np.int32).tolist() == [40]
    assert as_f32(run(dev, vb.i4x8_dot_f32_scaled("l", "r", "ls", "rs", "o", 8),
                      [u32(0xCDEF4321), u32(0xFEDC1234), f32(0.5), f32(0.25)])[0]).tolist() == [5.0]
    # lanes 1,7,8,9,...,96 (int4_quantized_gpu_parity dot contracts)
    for lanes in [1, 7, 8, 9, 15, 16, 17, 31, 33, 64, 65, 96]:
        a, b = generated_i4_values(lanes, 11 + lanes), generated_i4_values(lanes, 97 + lanes)
        pa, pb = oracle.pack_i4x8(a), oracle.pack_i4x8(b)
        got = np.frombuffer(run(dev, vb.i4x8_dot_i32("l", "r", "o", lanes), [pa, pb])[0], np.int32)[0]
        assert got == oracle.i4x8_dot_i32(pa, pb, lanes) == int(np.sum(a * b))
        got = as_f32(run(dev, vb.i4x8_dot_f32_scaled("l", "r", "ls", "rs", "o", lanes),
                         [pa, pb, f32(0.125), f32(0.5)])[0])[0]
        assert bits(f32(got))[0] == bits(f32(oracle.i4x8_dot_f32_scaled(pa, pb, 0.125, 0.5, lanes)))[0]


def test_int4_matvec_matmul_top1_sweeps(dev):
    for rows, cols, batch in [(1, 1, 1), (3, 9, 2), (4, 8, 2), (7, 65, 3), (5, 33, 1), (16, 96, 4)]:
        wrows = [generated_i4_values(cols, 5 + r * 97) for r in range(rows)]
        w = pack_rows(wrows)
        x = generated_f32_values(batch * cols, 3 + rows)
        scales = generated_positive_scales(rows, 1)
        got = as_f32(run(dev, vb.i4x8_batched_matvec_f32_scaled("w", "x", "s", "o", batch, rows, cols), [w, x, scales])[0])
        want = oracle.i4x8_batched_matvec_f32_scaled(w, x, scales, batch, rows, cols)
        assert bits(got).tolist() == bits(want).tolist()
        if batch == 1:
            got = as_f32(run(dev, vb.i4x8_matvec_f32_scaled("w", "x", "s", "o", rows, cols), [w, x, scales])[0])
            assert bits(got).tolist() == bits(want).tolist()
        acts = pack_rows([generated_i4_values(cols, 1000 + b * 13) for b in range(batch)])
        bs = generated_positive_scales(batch, 4)
        got = as_f32(run(dev, vb.i4x8_batched_matmul_f32_scaled("w", "a", "rs", "bs", "o", batch, rows, cols),
                         [w, acts, scales, bs])[0])
        want = oracle.i4x8_batched_matmul_f32_scaled(w, acts, scales, bs, batch, rows, cols)
        assert bits(got).tolist() == bits(want).tolist()
        got = as_f32(run(dev, vb.i4x8_batched_matmul_top1_f32_scaled("w", "a", "rs", "bs", "o", batch, rows, cols),
                         [w, acts, scales, bs])[0])
        want = oracle.i4x8_batched_matmul_top1_f32_scaled(w, acts, scales, bs, batch, rows, cols)
        assert bits(got).tolist() == bits(want).tolist()
    # registry fixture: ties keep the first row, out = [scores | f32(index)]
    w4, act = u32(*[0x76210F98] * 4), u32(0x76210F98, 0x76210F98)
    got = as_f32(run(dev, vb.i4x8_batched_matmul_top1_f32_scaled("w", "a", "rs", "bs", "o", 2, 4, 8),
                     [w4, act, np.ones(4, np.float32), np.ones(2, np.float32)])[0])
    assert got.tolist() == [204.0, 204.0, 0.0, 0.0]


def test_int8_and_matmul_and_linear_rows(dev):
    assert as_f32(run(dev, vb.int8_unpack("p", "s", "o", 4, 2), [u32(10, 20, 30, 40), f32(0.5, 2.0)])[0]).tolist() == [
        5.0, 10.0, 60.0, 80.0]
    assert as_u32(run(dev, vb.int8_pack("i", "o", 4), [u32(255, 256, 1, 0)])[0]).tolist() == [255, 0, 1, 0]
    rng = np.random.default_rng(5)
    a = rng.integers(0, 2**32, size=(5, 9), dtype=np.uint32)
    b = rng.integers(0, 2**32, size=(9, 7), dtype=np.uint32)
    got = as_u32(run(dev, vb.matmul("a", "b", "o", 5, 9, 7), [a, b])[0])
    assert got.tolist() == oracle.matmul_u32(a, b, None, 5, 9, 7).tolist()
    # registry fixtures: matmul_bias (vyre-libs/src/math/linalg/matmul.rs:708-731), nn::linear (nn/linear/inner/tiled.rs:150-186)
    assert as_u32(run(dev, vb.matmul_bias("a", "b", "bias", "out", 2, 2, 2), [u32(1, 2, 3, 4), u32(5, 6, 7, 8), u32(10, 20)])[0]
                  ).tolist() == [29, 42, 53, 70]
    assert as_u32(run(dev, vb.matmul_bias_tiled("a", "b", "bias", "out", 2, 2, 2, 2), [u32(1, 2, 3, 4), u32(5, 6, 7, 8), u32(10, 20)])[0]
                  ).tolist() == [29, 42, 53, 70]
    assert as_u32(run(dev, vb.linear("x", "w", "b", "out", 4, 4), [np.arange(4, dtype=np.uint32), np.arange(16, dtype=np.uint32),
                                                                   u32(0, 0, 0, 0)])[0]).tolist() == [56, 62, 68, 74]
    # wrapping products at sizes that fill no tile, through the flat, the tiled and the linear builders
    for m, k, n in [(1, 1, 1), (33, 65, 31), (70, 100, 129), (1, 300, 257)]:
        a = rng.integers(0, 2**32, size=(m, k), dtype=np.uint32)
        b = rng.integers(0, 2**32, size=(k, n), dtype=np.uint32)
        bias = rng.integers(0, 2**32, size=n, dtype=np.uint32)
        want = oracle.matmul_u32(a, b, bias, m, k, n).tolist()
        assert as_u32(run(dev, vb.matmul_bias("a", "b", "bias", "out", m, k, n), [a, b, bias])[0]).tolist() == want
        assert as_u32(run(dev, vb.matmul_bias_tiled("a", "b", "bias", "out", m, k, n, 32), [a, b, bias])[0]).tolist() == want
        if m == 1:
            assert as_u32(run(dev, vb.linear("x", "w", "b", "out", k, n), [a, b, bias])[0]).tolist() == want
    for dt, odt in [(ffi.DT_F32, oracle.DT_F32), (ffi.DT_BF16, oracle.DT_BF16), (ffi.DT_F16, oracle.DT_F16)]:
        x = rng.standard_normal((3, 40)).astype(np.float32)
        w = rng.standard_normal((40, 6)).astype(np.float32)
        if dt == ffi.DT_F32:
            xe, we = x, w
        elif dt == ffi.DT_BF16:
            xe, we = oracle.f32_to_bf16_bits(x), oracle.f32_to_bf16_bits(w)
        else:
            xe, we = x.astype(np.float16).view(np.uint16), w.astype(np.float16).view(np.uint16)
        for out_in in (False, True):
            wl = np.ascontiguousarray(we.reshape(40, 6).T) if out_in else we
            build = vb.linear_rows_no_bias_out_in_typed if out_in else vb.linear_rows_no_bias_typed
            got = run(dev, build("x", "w", "o", 3, 40, 6, dt), [xe, wl])[0]
            want = oracle.linear_rows(xe, wl, None, 3, 40, 6, dtype=odt, weight_out_in=out_in)
            assert got == want.tobytes()
    bias = rng.standard_normal(6).astype(np.float32)
    got = run(dev, vb.linear_rows("x", "w", "b", "o", 3, 40, 6), [x, w, bias])[0]
    assert got == oracle.linear_rows(x, w, bias, 3, 40, 6).tobytes()
    # vyre-libs/tests/linear_rows_contract.rs:24-75: the reference's hand-computed projections
    got = run(dev, vb.linear_rows("x", "w", "b", "o", 2, 3, 2), [f32(1, 2, 3, -1, 0, 2), f32(1, 0, 0, 1, 1, 1), f32(0.5, -0.5)])[0]
    assert as_f32(got).tolist() == [4.5, 4.5, 1.5, 1.5]
    got = run(dev, vb.linear_rows("x", "w", "b", "o", 2, 2, 1), [f32(0, 0, 4, -1), f32(2, 3), f32(0.0)])[0]
    assert as_f32(got).tolist() == [0.0, 5.0]
    got = run(dev, vb.linear_rows_no_bias_out_in_typed("x", "w", "o", 1, 2, 2, ffi.DT_F32), [f32(2, 3), f32(1, 10, 100, 1000)])[0]
    assert as_f32(got).tolist() == [32.0, 3200.0]


def test_moe_ops(dev):
    scores = f32(0.5, 1.0, 0.1, 2.0, 0.3, 3.0, 0.2, 0.4)
    out = run(dev, vb.moe_gate("s", "i", "w", 8, 2), [scores, np.zeros(2, np.uint32)])
    oi, ow = oracle.moe_gate(scores, 2)
    assert as_u32(out[0]).tolist() == [5, 3] == oi.tolist()
    assert max_ulp(as_f32(out[1]), ow) <= 128
    s8 = np.arange(1, 9, dtype=np.float32)
    out = run(dev, vb.softmax_top_k("s", "oi", "ow", 8, 2), [s8, np.zeros(2, np.float32), np.zeros(2, np.float32),
                                                           np.zeros(2, np.uint32)])
    oi, ow, bv, bi = oracle.softmax_top_k(s8, 2)
    assert as_u32(out[0]).tolist() == [7, 6] and as_u32(out[3]).tolist() == [7, 6]
    assert max_ulp(as_f32(out[1]), ow) <= 128 and max_ulp(as_f32(out[2]), bv) <= 128
    out = run(dev, vb.top_k("s", "o", 8, 3), [f32(3, 1, 4, 1, 5, 9, 2, 6), np.zeros(3, np.float32), np.zeros(3, np.uint32)])
    assert as_u32(out[0]).tolist() == [5, 7, 4]
    # random gates incl. ties: indices identical to the oracle
    rng = np.random.default_rng(9)
    for _ in range(20):
        sc = rng.integers(-4, 5, size=16).astype(np.float32) * np.float32(0.25)
        out = run(dev, vb.moe_gate("s", "i", "w", 16, 4), [sc, np.zeros(4, np.uint32)])
        oi, ow = oracle.moe_gate(sc, 4)
        assert as_u32(out[0]).tolist() == oi.tolist() and max_ulp(as_f32(out[1]), ow) <= 128
    gate, up = f32(0.0, 1.0, -1.0, 2.0), f32(1.0, 2.0, 3.0, 4.0)
    assert max_ulp(as_f32(run(dev, vb.swiglu("g", "u", "o", 4), [gate, up])[0]), oracle.swiglu(gate, up)) <= 128
    g = rng.standard_normal(1000).astype(np.float32)
    u = rng.standard_normal(1000).astype(np.float32)
    gb, ub = oracle.f32_to_bf16_bits(g), oracle.f32_to_bf16_bits(u)
    got = np.frombuffer(run(dev, vb.swiglu_typed("g", "u", "o", 1000, ffi.DT_BF16), [gb, ub])[0], np.uint16)
    want = oracle.swiglu(gb, ub, dtype=oracle.DT_BF16)
    # bf16 outputs: equal up to one bf16 ulp where exp differs in its last bits
    assert np.max(np.abs(got.astype(np.int32) - want.astype(np.int32))) <= 1
    args = [f32(1.0, 2.0), f32(0.5, -0.25, 1.0, 0.75), f32(0.1, -0.2), f32(0.25, 0.5, -0.5, 1.25), f32(0.0, 0.3),
            f32(1.0, -0.5, 0.25, 0.75), f32(0.2, -0.1)]
    got = as_f32(run(dev, vb.expert_mlp("x", "wg", "bg", "wu", "bu", "wd", "bd", "o", 2, 2, 2), args)[0])
    assert max_ulp(got, oracle.expert_mlp(*args, 2, 2, 2)) <= 128
    # larger experts under the reference's transcendental window (128 ULP, vyre-foundation/src/fp_parity.rs:14-16):
    # dyadic weights and inputs keep every product and partial sum exact, so that only exp differs between the two sides
    for (i, h, o, seed) in [(16, 24, 8, 1), (64, 96, 32, 2), (33, 130, 7, 3), (128, 256, 64, 4)]:
        r = np.random.default_rng(seed)
        dy = lambda *shape: (r.integers(-8, 9, size=shape) * 0.125).astype(np.float32)
        args = [dy(i), dy(i * h) * np.float32(0.25), dy(h), dy(i * h) * np.float32(0.25), dy(h), dy(h * o) * np.float32(0.25), dy(o)]
        got = as_f32(run(dev, vb.expert_mlp("x", "wg", "bg", "wu", "bu", "wd", "bd", "o", i, h, o), args)[0])
        want = oracle.expert_mlp(*args, i, h, o)
        # outputs that cancel to (almost) nothing carry no ULP information: the window applies from 1e-3 of the largest
        big = np.abs(want) >= 1e-3 * np.max(np.abs(want))
        assert big.sum() >= o // 2 and max_ulp(got[big], want[big]) <= 128, (i, h, o)
        assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))
    got = as_f32(run(dev, vb.moe_layer_route_and_accumulate("x", "wr", "br", "ei", "ew", "eo", "o", 2, 4, 2, 2),
                     [np.zeros(2, np.float32), np.zeros(8, np.float32), np.zeros(4, np.float32), u32(0, 1),
                      f32(0.6, 0.4), f32(1.0, 2.0, 3.0, 4.0)])[0])
    assert bits(got).tolist() == bits(oracle.moe_layer_accumulate(f32(0.6, 0.4), f32(1, 2, 3, 4), 2, 2)).tolist()


# ---- contract behaviour on a live device ---------------------------------------------------------------------------
def test_resident_buffer_rules_and_binding_validation(dev):
    with pytest.raises(vb.BackendError, match="0 bytes"):
        dev.allocate_resident(0)
    h = dev.resident_from(np.arange(16, dtype=np.uint32))
    assert np.array_equal(dev.download_resident(h, 64).view(np.uint32), np.arange(16, dtype=np.uint32))
    dev.upload_resident_at(h, 8, u32(7, 9))
    assert dev.download_resident(h, 8, offset=8).view(np.uint32).tolist() == [7, 9]
    with pytest.raises(vb.BackendError, match="exceeds"):
        dev.upload_resident_at(h, 60, u32(1, 2))
    foreign = ffi.ResidentHandle(h.owner + 1000, h.id)
    with pytest.raises(vb.BackendError, match="owned by backend instance") as e:
        dev.download_resident(foreign, 4)
    assert e.value.code == ffi.ERR_INVALID_PROGRAM
    dev.free_resident(h)
    with pytest.raises(vb.BackendError, match="unknown or already freed"):
        dev.free_resident(h)

    sess = vb.ArtifactSession.compile(vb.linear_4bit("x", "w", "b", "out", 8, 4), dev)
    good = [np.arange(8, dtype=np.float32), u32(0x76543210, 0xFEDCBA98, 0x11111111, 0), np.zeros(4, np.float32)]
    with pytest.raises(vb.BackendError, match="declares 32"):
        sess.run_host([good[0][:7], good[1], good[2]])
    with pytest.raises(vb.BackendError, match="missing input"):
        bs = vb.BindingSet(sess.artifact.digest())
        bs.insert_host(0, good[0])
        sess.submit_and_wait(bs)
    with pytest.raises(vb.BackendError, match="different artifact"):
        bs = sess.host_bindings(good)
        bs.artifact = bytes(32)
        sess.submit_and_wait(bs)
    # resident inputs + resident output left on the device; mixed with a host input
    hw, hb = dev.resident_from(good[1]), dev.resident_from(good[2])
    hout = dev.allocate_resident(16)
    bs = vb.BindingSet(sess.artifact.digest())
    bs.insert_host(0, good[0])
    bs.insert_resident(1, hw)
    bs.insert_resident(2, hb)
    bs.insert_resident(3, hout)
    sub = sess.submit(bs, leave_resident=True)
    c = sub.wait()
    with pytest.raises(vb.BackendError, match="consumed only once"):
        sub.wait()
    with pytest.raises(vb.BackendError, match="left resident"):
        c.output(3)
    assert c.device_ns is not None
    assert dev.download_resident(hout, 16).view(np.float32).tolist() == [140.0, 364.0, 28.0, 0.0]
    for hh in (hw, hb, hout):
        dev.free_resident(hh)


def test_payload_admission_fails_closed(dev):
    a1 = vb.compile(vb.linear_4bit("x", "w", "b", "out", 8, 4))
    a2 = vb.compile(vb.linear_4bit("x", "w", "b", "out", 16, 4))
    with pytest.raises(vb.BackendError, match="not authenticated for the supplied neutral artifact"):
        dev.materialize(a1, vb.target_compile(a2))
    inst = dev.materialize(a1, vb.target_compile(a1))
    assert inst.artifact() == a1.digest() and inst.device()["backend"] == "cuda-b200"


def test_device_loss_is_structured_and_recoverable():
    # host-injected loss: no device fault is provoked (vyre-runtime/src/recovery.rs:13-25)
    d = vb.Device.acquire(0)
    try:
        sess = vb.ArtifactSession.compile(vb.int8_pack("i", "o", 4), d)
        assert as_u32(sess.run_host([u32(255, 256, 1, 0)])[0]).tolist() == [255, 0, 1, 0]
        gen = d.identity()["generation"]
        envelope = sess.envelope_bytes()
        d.mark_lost("simulated context loss")
        assert not d.is_healthy()
        with pytest.raises(vb.BackendError) as e:
            sess.run_host([u32(1, 2, 3, 4)])
        assert e.value.code == ffi.ERR_DEVICE_LOST and "rematerialize" in e.value.message
        d.reacquire()
        assert d.is_healthy() and d.identity()["generation"] == gen + 1
        with pytest.raises(vb.BackendError) as e:  # stale instance of the lost generation
            sess.run_host([u32(1, 2, 3, 4)])
        assert e.value.code == ffi.ERR_DEVICE_LOST
        sess.rematerialize()  # same authenticated payload bytes, no recompilation
        assert sess.envelope_bytes() == envelope
        assert as_u32(sess.run_host([u32(511, 2, 3, 4)])[0]).tolist() == [255, 2, 3, 4]
    finally:
        d.release()
