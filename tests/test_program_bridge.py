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
