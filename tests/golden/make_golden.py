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
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vectors.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
