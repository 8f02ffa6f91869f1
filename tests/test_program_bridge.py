"""The bridge a TargetCompiler facet calls: a program rebuilt from a reference op id plus BufferDecl counts
(vyb_program_from_op), with and without an op spec, must equal the program the builder produced; declarations that
contradict the recovered shape are refused. CPU only: building and compiling programs needs no device.
"""
import pytest

import vyre_b200 as vb
from vyre_b200 import api, ffi


def roundtrip(prog, spec):
    bufs = [b for b in prog.buffers() if b["access"] != ffi.ACCESS_WORKGROUP]
    from_counts = api.program_from_op(prog.op_id, bufs)
    from_spec = api.program_from_op(prog.op_id, bufs, spec)
    assert from_counts.fingerprint() == prog.fingerprint() == from_spec.fingerprint()
    assert from_counts.buffers() == prog.buffers()
    # the rebuilt program compiles to the same artifact digest
    assert vb.compile(from_counts).digest() == vb.compile(prog).digest()
    return bufs


def test_affine_grouped_program_from_op_id_and_counts():
    # the reference's published case (vyre-bench/src/cases/quantized_linear.rs:26-37): K=256, N=4096, g=64, B=256
    prog = vb.linear_4bit_affine_grouped_batched("x", "w", "scale", "zp", "b", "out", 256, 4096, 64, 256)
    bufs = roundtrip(prog, [256, 4096, 64, 256])
    assert prog.op_id == "vyre-libs::nn::linear_4bit_affine_grouped"
    # C2-sized single row, group 128
    roundtrip(vb.linear_4bit_affine_grouped("x", "w", "scale", "zp", "b", "out", 4096, 14336, 128), [4096, 14336, 128, 1])
    # a declaration that contradicts the shape: one scale word too few
    broken = [dict(b) for b in bufs]
    broken[2]["count"] -= 1
    with pytest.raises(vb.BackendError) as e:
        api.program_from_op(prog.op_id, broken)
    assert e.value.code == ffi.ERR_INVALID_PROGRAM and "Fix:" in str(e.value)
    # an op spec that contradicts the declarations: authoritative spec, cross-check fails
    with pytest.raises(vb.BackendError, match="disagrees"):
        api.program_from_op(prog.op_id, bufs, [256, 4096, 32, 256])


def test_int4_matvec_and_gate_programs_from_op_ids():
    roundtrip(vb.i4x8_batched_matvec_f32_scaled("w", "x", "s", "o", 4, 3, 65, lib_op_id=True), [4, 3, 65])
    roundtrip(vb.i4x8_batched_matvec_f32_scaled("w", "x", "s", "o", 8, 14336, 4096), [8, 14336, 4096])
    roundtrip(vb.i4x8_matvec_f32_scaled("w", "x", "s", "o", 3, 65, lib_op_id=True), [1, 3, 65])
    roundtrip(vb.moe_gate("scores", "idx", "wts", 8, 2), [8, 2])
    roundtrip(vb.swiglu("g", "u", "o", 1000), [1000])
    with pytest.raises(vb.BackendError) as e:
        api.program_from_op("vyre-libs::nn::attention", [dict(name="q", binding=0, access=0, dtype=ffi.DT_F32, count=4)])
    assert e.value.code == ffi.ERR_UNSUPPORTED_FEATURE


def test_matmul_bias_and_linear_programs_from_op_ids():
    # vyre-libs/src/math/linalg/matmul.rs:252-268 (a, b, bias, out), vyre-libs/src/nn/linear/inner/builder.rs:139-162
    prog = vb.matmul_bias("a", "b", "bias", "out", 5, 9, 7)
    assert prog.op_id == "vyre-libs::math::matmul_bias" and [b["binding"] for b in prog.buffers()] == [0, 1, 2, 3]
    roundtrip(prog, [5, 9, 7])
    small = vb.linear("x", "w", "b", "out", 4, 4)  # the registry fixture's shape stays on the flat form
    assert small.op_id == "vyre-libs::nn::linear" and [b["count"] for b in small.buffers()] == [4, 16, 4, 4]
    roundtrip(small, [4, 4])
    # from in_dim * out_dim >= 1024 the builder hands over to the tiled form (builder.rs:147-152, tiled.rs:13-14):
    # two workgroup tiles of 32 x 16 and an output padded to whole 16 x 16 tiles, read back over its logical bytes
    big = vb.linear("x", "w", "b", "out", 64, 40)
    assert big.op_id == "vyre-libs::nn::linear_tiled"
    bufs = {b["name"]: b for b in big.buffers()}
    assert bufs["matmul_a_tile"]["count"] == 512 and bufs["matmul_b_tile"]["count"] == 512
    assert bufs["out"]["count"] == 3 * 256 and bufs["out"]["output_byte_range"] == (0, 40 * 4) and bufs["out"]["binding"] == 3
    roundtrip(big, [64, 40, 32])
    assert vb.linear_tiled("x", "w", "b", "out", 64, 40, 32).fingerprint() == big.fingerprint()
    for bad in [(0, 4), (4, 0), (1 << 17, 1 << 16)]:
        with pytest.raises(vb.BackendError) as e:
            vb.linear("x", "w", "b", "out", *bad)
        assert e.value.code == ffi.ERR_INVALID_PROGRAM and "Fix:" in str(e.value)
    with pytest.raises(vb.BackendError, match="needs the op spec"):
        api.program_from_op("vyre-libs::math::matmul", [b for b in vb.matmul("a", "b", "o", 2, 3, 4).buffers()])


def test_norm_residual_and_k_quant_programs_from_op_ids():
    import struct

    eps_bits = struct.unpack("<I", struct.pack("<f", 1e-6))[0]
    cases = [(vb.residual_add_typed("r", "b", "o", 96, ffi.DT_BF16), None),
             (vb.learned_rms_norm("i", "w", "o", 3, 64, 1e-6, ffi.DT_F16), [eps_bits]),
             (vb.gated_rms_norm("i", "w", "g", "o", 2, 128, 1e-6, ffi.DT_F32), [eps_bits]),
             (vb.q4_k_unpack("p", "s", "m", "o", 100), None), (vb.q2_k_unpack("p", "s", "m", "o", 100), None),
             (vb.q4_k_linear("x", "p", "s", "m", "b", "o", 96, 33), None), (vb.q2_k_linear("x", "p", "s", "m", "b", "o", 96, 33), None)]
    for prog, spec in cases:
        again = api.program_from_op(prog.op_id, prog.buffers(), spec)
        assert again.fingerprint() == prog.fingerprint(), prog.op_id
    with pytest.raises(vb.BackendError, match="eps"):  # the norm's eps is not recoverable from buffer counts
        api.program_from_op("vyre-libs::nn::learned_rms_norm", vb.learned_rms_norm("i", "w", "o", 3, 64, 1e-6, ffi.DT_F32).buffers())
