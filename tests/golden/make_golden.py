"""Generates tests/golden/vectors.npz: seeded inputs -> outputs of the CPU oracle for a few small cases of the path.

The reference is Rust and cannot run here, so these vectors are not reference outputs; they freeze the oracle (whose
semantics are pinned against the reference's own fixtures in tests/test_oracle_golden.py) so that a later change of the
oracle or of a kernel shows up as a diff against committed bytes. Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from vyre_b200 import synth  # noqa: E402


def build() -> dict:
    out = {}
    # int4 decode GEMV, f32 and bf16 outputs (group 128, k multiple of 1024)
    m, n, k = 2, 64, 1024
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=101)
    out["gemv_x"], out["gemv_w"], out["gemv_s"] = x, w, s
    out["gemv_y_f32"] = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32, mode=0)
    out["gemv_y_bf16"] = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_BF16, mode=0)
    # int8 dynamic linear: per-token quantiser + int32 GEMM (bit-exact path)
    rows, kk, nn = 48, 128, 96
    xa, wa = synth.int8_dynamic_inputs(rows, nn, kk, seed=102)[:2]
    q, sc = oracle.quantize_per_token_int8(xa, rows, kk)
    out["i8_x"], out["i8_w"], out["i8_q"], out["i8_scale"] = xa, wa, q, sc
    out["i8_y"] = oracle.int8_gemm_i32(q, wa, rows, nn, kk)
    # MoE FFN layer, bf16-weight mode (what the tensor-core path computes)
    t, h, i, e, topk = 24, 256, 256, 2, 2
    mx, mwr, mw13, ms13, mw2, ms2 = synth.moe_ffn_inputs(t, h, i, e, seed=103)
    mo, midx, mwts = oracle.moe_ffn_int4(mx, mwr, mw13, ms13, mw2, ms2, np.arange(t), h, i, e, topk, mode=1)
    out.update(moe_x=mx, moe_wr=mwr, moe_w13=mw13, moe_s13=ms13, moe_w2=mw2, moe_s2=ms2, moe_out=mo, moe_idx=midx,
               moe_wts=mwts)
    # residual add (bf16), learned RMSNorm (f32 and bf16, rows short enough for the chain-order sum), K-quant unpack and
    # fused linear (4-bit and 2-bit): all bit-exact on the device
    rng = np.random.default_rng(104)
    ra = oracle.f32_to_bf16_bits((rng.standard_normal(300) * 8).astype(np.float32))
    rb = oracle.f32_to_bf16_bits(rng.standard_normal(300).astype(np.float32))
    out["res_a"], out["res_b"], out["res_out"] = ra, rb, oracle.residual_add(ra, rb, oracle.DT_BF16)
    rows, hidden = 3, 200
    nx = (rng.standard_normal(rows * hidden) * 3).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    out["norm_x"], out["norm_w"] = nx, nw
    out["norm_out_f32"] = oracle.rms_norm(nx, nw, rows, hidden, 1e-6).reshape(rows, hidden)
    nxb, nwb = oracle.f32_to_bf16_bits(nx), oracle.f32_to_bf16_bits(nw)
    out["norm_out_bf16"] = oracle.rms_norm(nxb, nwb, rows, hidden, 1e-6, dtype=oracle.DT_BF16).reshape(rows, hidden)
    in_dim, out_dim = 96, 33
    for bits, block, wpb in ((4, 32, 4), (2, 16, 1)):
        blocks = -(-(in_dim * out_dim) // block)
        kp = rng.integers(0, 2**32, size=blocks * wpb, dtype=np.uint32)
        ks = rng.uniform(0.01, 0.2, size=blocks).astype(np.float32)
        km = (-rng.uniform(0.0, 1.0, size=blocks)).astype(np.float32)
        kx, kb = rng.standard_normal(in_dim).astype(np.float32), rng.standard_normal(out_dim).astype(np.float32)
        pre = f"q{bits}k_"
        out[pre + "packed"], out[pre + "scales"], out[pre + "mins"], out[pre + "x"], out[pre + "b"] = kp, ks, km, kx, kb
        out[pre + "unpacked"] = oracle.k_quant_unpack(kp, ks, km, in_dim * out_dim, bits)
        out[pre + "y"] = oracle.k_quant_linear(kx, kp, ks, km, kb, in_dim, out_dim, bits)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vectors.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
