"""CPU checker for the quantized-linear / MoE hot path (TEST INFRASTRUCTURE ONLY).

`oracle.lib()` loads `oracle/_build/libvyre_oracle.so` (built by `oracle/Makefile`) and the thin
numpy wrappers below call it. Only the tests, the smoke run and the benchmark's CPU-baseline leg
import this package; the product library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libvyre_oracle.so")
_BASE_SO = os.path.join(_HERE, "_build", "libvyre_cpu_baseline.so")
_LIB = None
_BASE = None

DT_F32, DT_BF16, DT_F16 = 0, 1, 2


def build(force: bool = False) -> str:
    stale = force
    for so, src in ((_SO, "vyre_oracle.cpp"), (_BASE_SO, "cpu_baseline.cpp")):
        stale = stale or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(_HERE, src))
    if stale:
        subprocess.run(["make", "-C", _HERE, "all"], check=True, stdout=subprocess.DEVNULL)
    return _SO


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not os.path.exists(_SO):
            build()
        _LIB = C.CDLL(_SO)
        _LIB.vyo_canonical_f32.restype = C.c_float
        _LIB.vyo_canonical_f32.argtypes = [C.c_float]
        _LIB.vyo_bf16_to_f32.restype = C.c_float
        _LIB.vyo_bf16_to_f32.argtypes = [C.c_uint16]
        _LIB.vyo_f32_to_bf16.restype = C.c_uint16
        _LIB.vyo_f32_to_bf16.argtypes = [C.c_float]
        _LIB.vyo_f16_to_f32.restype = C.c_float
        _LIB.vyo_f16_to_f32.argtypes = [C.c_uint16]
        _LIB.vyo_f32_to_f16.restype = C.c_uint16
        _LIB.vyo_f32_to_f16.argtypes = [C.c_float]
        _LIB.vyo_ulp_distance.restype = C.c_uint32
        _LIB.vyo_ulp_distance.argtypes = [C.c_float, C.c_float]
        _LIB.vyo_i4x8_dot_i32.restype = C.c_int32
        _LIB.vyo_i4x8_dot_f32_scaled.restype = C.c_float
        _LIB.vyo_i4x8_dot_f32_scaled.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_uint32]
        _LIB.vyo_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().vyo_num_threads())


def cpu_baseline_int4_gemv(x_f32, w_packed, scale_bf16, m: int, n: int, k: int, group: int = 128, zp: int = 8) -> np.ndarray:
    """The reference bench's CPU loop (f32, sequential k, one task per output; vyre-bench/src/cases/
    quantized_linear.rs:447-463) for the row-major int4 GEMV, built -O3: the thing bench.py TIMES on the host cores.
    Not the checker."""
    global _BASE
    if _BASE is None:
        if not os.path.exists(_BASE_SO):
            build()
        _BASE = C.CDLL(_BASE_SO)
    x = _c(x_f32, np.float32)
    w = _c(w_packed, np.uint8)
    s = _c(scale_bf16, np.uint16)
    out = np.empty((m, n), np.float32)
    _BASE.vyo_cpu_baseline_int4_gemv(_p(x), _p(w), _p(s), _p(out), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k),
                                     C.c_uint32(group), C.c_int32(zp))
    return out


# ---- bf16 helpers (numpy has no bf16: carried as uint16 bit patterns) -------------------------
def f32_to_bf16_bits(a) -> np.ndarray:
    """RNE conversion, NaN -> 0x7fc0, subnormal flushed (vyre-reference/src/float16.rs:9-16)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).copy()
    exp0 = (bits & 0x7F800000) == 0
    bits[exp0] &= 0x80000000
    nan = ((bits & 0x7F800000) == 0x7F800000) & ((bits & 0x007FFFFF) != 0)
    rounded = (bits.astype(np.uint64) + 0x7FFF + ((bits >> 16) & 1)).astype(np.uint32)
    out = (rounded >> 16).astype(np.uint16)
    out[nan] = 0x7FC0
    return out


def bf16_bits_to_f32(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


# ---- primitives ---------------------------------------------------------------------------------
def pack_i4x8(values) -> np.ndarray:
    v = _c(values, np.int32)
    out = np.zeros((v.size + 7) // 8, dtype=np.uint32)
    lib().vyo_pack_i4x8(_p(v), C.c_uint32(v.size), _p(out))
    return out


def unpack_i4x8(packed, lanes: int) -> np.ndarray:
    p = _c(packed, np.uint32)
    out = np.zeros(lanes, dtype=np.int32)
    lib().vyo_unpack_i4x8(_p(p), C.c_uint32(p.size), C.c_uint32(lanes), _p(out))
    return out


def i4x8_dot_i32(lhs, rhs, lanes: int) -> int:
    l, r = _c(lhs, np.uint32), _c(rhs, np.uint32)
    return int(lib().vyo_i4x8_dot_i32(_p(l), _p(r), C.c_uint32(lanes)))


def i4x8_dot_f32_scaled(lhs, rhs, ls: float, rs: float, lanes: int) -> float:
    l, r = _c(lhs, np.uint32), _c(rhs, np.uint32)
    return float(lib().vyo_i4x8_dot_f32_scaled(_p(l), _p(r), C.c_float(ls), C.c_float(rs), C.c_uint32(lanes)))


def i4x8_batched_matvec_f32_scaled(w, x, scales, batch: int, rows: int, cols: int) -> np.ndarray:
    w, x, s = _c(w, np.uint32), _c(x, np.float32), _c(scales, np.float32)
    out = np.zeros(batch * rows, dtype=np.float32)
    lib().vyo_i4x8_batched_matvec_f32_scaled(_p(w), _p(x), _p(s), C.c_uint32(batch), C.c_uint32(rows),
                                             C.c_uint32(cols), _p(out))
    return out


def i4x8_batched_matmul_f32_scaled(w, act, row_scales, batch_scales, batch, rows, cols) -> np.ndarray:
    w, a = _c(w, np.uint32), _c(act, np.uint32)
    rs, bs = _c(row_scales, np.float32), _c(batch_scales, np.float32)
    out = np.zeros(batch * rows, dtype=np.float32)
    lib().vyo_i4x8_batched_matmul_f32_scaled(_p(w), _p(a), _p(rs), _p(bs), C.c_uint32(batch), C.c_uint32(rows),
                                             C.c_uint32(cols), _p(out))
    return out


def i4x8_batched_matmul_top1_f32_scaled(w, act, row_scales, batch_scales, batch, rows, cols) -> np.ndarray:
    w, a = _c(w, np.uint32), _c(act, np.uint32)
    rs, bs = _c(row_scales, np.float32), _c(batch_scales, np.float32)
    out = np.zeros(2 * batch, dtype=np.float32)
    lib().vyo_i4x8_batched_matmul_top1_f32_scaled(_p(w), _p(a), _p(rs), _p(bs), C.c_uint32(batch),
                                                  C.c_uint32(rows), C.c_uint32(cols), _p(out))
    return out


def linear_4bit(x, w, b, in_dim: int, out_dim: int) -> np.ndarray:
    x, w, b = _c(x, np.float32), _c(w, np.uint32), _c(b, np.float32)
    out = np.zeros(out_dim, dtype=np.float32)
    lib().vyo_linear_4bit(_p(x), _p(w), _p(b), _p(out), C.c_uint32(in_dim), C.c_uint32(out_dim))
    return out


def linear_4bit_affine_grouped(x, w, scale, zp, b, in_dim, out_dim, group_size, batch=1, simple=False):
    x, w, s = _c(x, np.float32), _c(w, np.uint32), _c(scale, np.float32)
    z, b = _c(zp, np.uint32), _c(b, np.float32)
    out = np.zeros(batch * out_dim, dtype=np.float32)
    fn = lib().vyo_linear_4bit_affine_grouped_simple if simple else lib().vyo_linear_4bit_affine_grouped
    fn(_p(x), _p(w), _p(s), _p(z), _p(b), _p(out), C.c_uint32(in_dim), C.c_uint32(out_dim),
       C.c_uint32(group_size), C.c_uint32(batch))
    return out


def int8_unpack(packed, scales, n: int, cols: int) -> np.ndarray:
    p, s = _c(packed, np.uint32), _c(scales, np.float32)
    out = np.zeros(n, dtype=np.float32)
    lib().vyo_int8_unpack(_p(p), _p(s), _p(out), C.c_uint32(n), C.c_uint32(cols))
    return out


def int8_pack(values, n: int) -> np.ndarray:
    v = _c(values, np.uint32)
    out = np.zeros(n, dtype=np.uint32)
    lib().vyo_int8_pack(_p(v), _p(out), C.c_uint32(n))
    return out


_NP_OF = {DT_F32: np.float32, DT_BF16: np.uint16, DT_F16: np.uint16}


def linear_rows(x, w, bias, rows, in_dim, out_dim, dtype=DT_F32, weight_out_in=False) -> np.ndarray:
    nd = _NP_OF[dtype]
    x, w = _c(x, nd), _c(w, nd)
    bias = None if bias is None else _c(bias, nd)
    out = np.zeros(rows * out_dim, dtype=nd)
    lib().vyo_linear_rows(_p(x), _p(w), _p(bias), _p(out), C.c_uint32(rows), C.c_uint32(in_dim),
                          C.c_uint32(out_dim), C.c_uint32(dtype), C.c_uint32(1 if weight_out_in else 0))
    return out


def matmul_u32(a, b, bias, m, k, n) -> np.ndarray:
    a, b = _c(a, np.uint32), _c(b, np.uint32)
    bias = None if bias is None else _c(bias, np.uint32)
    out = np.zeros(m * n, dtype=np.uint32)
    lib().vyo_matmul_u32(_p(a), _p(b), _p(bias), _p(out), C.c_uint32(m), C.c_uint32(k), C.c_uint32(n))
    return out


def moe_gate(scores, k: int):
    s = _c(scores, np.float32)
    idx = np.zeros(k, dtype=np.uint32)
    w = np.zeros(k, dtype=np.float32)
    lib().vyo_moe_gate(_p(s), C.c_uint32(s.size), C.c_uint32(k), _p(idx), _p(w))
    return idx, w


def softmax_top_k(scores, k: int):
    s = _c(scores, np.float32)
    idx = np.zeros(k, dtype=np.uint32)
    w = np.zeros(k, dtype=np.float32)
    bv = np.zeros(k, dtype=np.float32)
    bi = np.zeros(k, dtype=np.uint32)
    lib().vyo_softmax_top_k(_p(s), C.c_uint32(s.size), C.c_uint32(k), _p(idx), _p(w), _p(bv), _p(bi))
    return idx, w, bv, bi


def top_k(values, k: int) -> np.ndarray:
    s = _c(values, np.float32)
    idx = np.zeros(k, dtype=np.uint32)
    lib().vyo_top_k(_p(s), C.c_uint32(s.size), C.c_uint32(k), _p(idx))
    return idx


def swiglu(gate, up, dtype=DT_F32) -> np.ndarray:
    nd = _NP_OF[dtype]
    g, u = _c(gate, nd), _c(up, nd)
    out = np.zeros(g.size, dtype=nd)
    lib().vyo_swiglu(_p(g), _p(u), _p(out), C.c_uint32(g.size), C.c_uint32(dtype))
    return out


def expert_mlp(x, wg, bg, wu, bu, wd, bd, in_dim, hidden, out_dim) -> np.ndarray:
    a = [_c(t, np.float32) for t in (x, wg, bg, wu, bu, wd, bd)]
    out = np.zeros(out_dim, dtype=np.float32)
    lib().vyo_expert_mlp(*[_p(t) for t in a], _p(out), C.c_uint32(in_dim), C.c_uint32(hidden), C.c_uint32(out_dim))
    return out


def moe_layer_accumulate(weights, expert_out, k, out_dim) -> np.ndarray:
    w, e = _c(weights, np.float32), _c(expert_out, np.float32)
    out = np.zeros(out_dim, dtype=np.float32)
    lib().vyo_moe_layer_accumulate(_p(w), _p(e), _p(out), C.c_uint32(k), C.c_uint32(out_dim))
    return out


# ---- benchmark-configuration compositions -------------------------------------------------------
def int4_rowmajor_linear(x_bf16, w_packed, scale_bf16, m, n, k, group=128, zp=8, out_dtype=DT_BF16, mode=0):
    x, w, s = _c(x_bf16, np.uint16), _c(w_packed, np.uint8), _c(scale_bf16, np.uint16)
    out = np.zeros(m * n, dtype=_NP_OF[out_dtype])
    lib().vyo_int4_rowmajor_linear(_p(x), _p(w), _p(s), _p(out), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k),
                                   C.c_uint32(group), C.c_int32(zp), C.c_uint32(out_dtype), C.c_uint32(mode))
    return out.reshape(m, n)


def int8_weight_only_linear(x, w, scale, m, n, k, mode=0) -> np.ndarray:
    x, w, s = _c(x, np.float32), _c(w, np.int8), _c(scale, np.float32)
    out = np.zeros(m * n, dtype=np.float32)
    lib().vyo_int8_weight_only_linear(_p(x), _p(w), _p(s), _p(out), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k),
                                      C.c_uint32(mode))
    return out.reshape(m, n)


def quantize_per_token_int8(x_bf16, m, k):
    x = _c(x_bf16, np.uint16)
    q = np.zeros(m * k, dtype=np.int8)
    s = np.zeros(m, dtype=np.float32)
    lib().vyo_quantize_per_token_int8(_p(x), _p(q), _p(s), C.c_uint32(m), C.c_uint32(k))
    return q.reshape(m, k), s


def int8_gemm_i32(a, w, m, n, k, row_begin=0, row_end=None) -> np.ndarray:
    a, w = _c(a, np.int8), _c(w, np.int8)
    row_end = m if row_end is None else row_end
    out = np.zeros((row_end - row_begin) * n, dtype=np.int32)
    lib().vyo_int8_gemm_i32(_p(a), _p(w), _p(out), C.c_uint32(m), C.c_uint32(n), C.c_uint32(k),
                            C.c_uint32(row_begin), C.c_uint32(row_end))
    return out.reshape(row_end - row_begin, n)


def moe_ffn_int4(x_bf16, w_router_bf16, w13, s13, w2, s2, tokens, hidden, inter, experts, topk, group=128, mode=0):
    x, wr = _c(x_bf16, np.uint16), _c(w_router_bf16, np.uint16)
    w13, s13, w2, s2 = _c(w13, np.uint8), _c(s13, np.uint16), _c(w2, np.uint8), _c(s2, np.uint16)
    tok = _c(tokens, np.uint32)
    out = np.zeros(tok.size * hidden, dtype=np.uint16)
    idx = np.zeros(tok.size * topk, dtype=np.uint32)
    wts = np.zeros(tok.size * topk, dtype=np.float32)
    lib().vyo_moe_ffn_int4(_p(x), _p(wr), _p(w13), _p(s13), _p(w2), _p(s2), _p(tok), C.c_uint32(tok.size),
                           C.c_uint32(hidden), C.c_uint32(inter), C.c_uint32(experts), C.c_uint32(topk),
                           C.c_uint32(group), C.c_uint32(mode), _p(out), _p(idx), _p(wts))
    return out.reshape(tok.size, hidden), idx.reshape(tok.size, topk), wts.reshape(tok.size, topk)


# ---- operators either side of the feed-forward block, GGML K-quant linears ------------------------------------------
def residual_add(residual, branch, dtype=DT_F32) -> np.ndarray:
    nd = _NP_OF[dtype]
    r, b = _c(residual, nd), _c(branch, nd)
    out = np.zeros(r.size, dtype=nd)
    lib().vyo_residual_add(_p(r), _p(b), _p(out), C.c_uint32(r.size), C.c_uint32(dtype))
    return out


def rms_norm(x, weight, rows: int, hidden: int, eps: float, dtype=DT_F32, gate=None, weight_dtype=None) -> np.ndarray:
    """learned_rms_norm (gate=None) and gated_rms_norm."""
    nd = _NP_OF[dtype]
    wd = dtype if weight_dtype is None else weight_dtype
    xv, wv = _c(x, nd), _c(weight, _NP_OF[wd])
    gv = None if gate is None else _c(gate, nd)
    out = np.zeros(rows * hidden, dtype=nd)
    lib().vyo_rms_norm(_p(xv), _p(wv), _p(gv) if gv is not None else None, _p(out), C.c_uint32(rows), C.c_uint32(hidden),
                       C.c_float(eps), C.c_uint32(dtype), C.c_uint32(wd))
    return out


def k_quant_unpack(packed, scales, mins, n: int, bits: int) -> np.ndarray:
    p, s, m = _c(packed, np.uint32), _c(scales, np.float32), _c(mins, np.float32)
    out = np.zeros(n, dtype=np.float32)
    lib().vyo_k_quant_unpack(_p(p), _p(s), _p(m), _p(out), C.c_uint32(n), C.c_uint32(bits))
    return out


def k_quant_linear(x, packed, scales, mins, b, in_dim: int, out_dim: int, bits: int) -> np.ndarray:
    xv, p, s, m, bv = _c(x, np.float32), _c(packed, np.uint32), _c(scales, np.float32), _c(mins, np.float32), _c(b, np.float32)
    out = np.zeros(out_dim, dtype=np.float32)
    lib().vyo_k_quant_linear(_p(xv), _p(p), _p(s), _p(m), _p(bv), _p(out), C.c_uint32(in_dim), C.c_uint32(out_dim), C.c_uint32(bits))
    return out
