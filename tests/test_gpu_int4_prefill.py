"""GPU parity of the int4 prefill GEMM (benchmark config 3) against the CPU oracle.

The kernel dequantises weights to bf16 (one rounding of (q-8)*s) and accumulates in f32 on the tensor cores; the
oracle in mode 1 applies the same bf16 rounding and accumulates exactly, so f32 outputs must agree to 1e-4 and
bf16 outputs to 1e-2 (in practice one bf16 ulp). Mode 0 (no weight rounding) is checked at the bf16 tolerance.
"""
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


def rel_err(got, want, floor_frac=1e-2):
    want = want.astype(np.float64)
    floor = floor_frac * float(np.sqrt(np.mean(want**2))) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))


def prefill_raw(x, w, s, m, n, k, group, out_f32):
    tx, tw, ts = (torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
    ty = torch.full((m, n), 7.0, dtype=torch.float32 if out_f32 else torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ffi.check(ffi.lib().vyb_k_int4_prefill_gemm(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), ty.data_ptr(), m, n, k,
                                                group, ffi.DT_F32 if out_f32 else ffi.DT_BF16,
                                                C.c_void_p(torch.cuda.current_stream().cuda_stream),
                                                C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    return ty.cpu().numpy() if out_f32 else ty.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("m,n,k,group", [(128, 256, 64, 64), (128, 256, 128, 128), (1, 8, 64, 64), (65, 100, 192, 64),
                                         (129, 257, 256, 128), (300, 1000, 1024, 128), (96, 520, 4096, 128),
                                         (200, 264, 512, 256), (77, 31, 1024, 128)])
def test_prefill_shapes_f32_out(m, n, k, group):
    x, w, s = synth.int4_linear_inputs(m, n, k, group=group, seed=m + n + k)
    got = prefill_raw(x, w, s, m, n, k, group, True)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k, group=group, out_dtype=oracle.DT_F32, mode=1)
    # The tensor core aligns every addend to the running sum and drops the bits below its f32 mantissa, so an
    # output that cancels to near zero keeps an absolute error of ~1e-6 of the row's typical magnitude: the
    # relative window is measured against max(|want|, 10% of the output RMS).
    assert rel_err(got, want, floor_frac=0.1) <= 1e-4


def test_prefill_exact_on_dyadic_inputs():
    rng = np.random.default_rng(4)
    m, n, k = 160, 300, 512
    x = synth.f32_to_bf16_bits((rng.integers(-8, 9, size=(m, k)) * 0.25).astype(np.float32))
    w = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    s = synth.f32_to_bf16_bits(np.array([[0.25, 0.5, 1.0, 2.0][(r + g) & 3] for r in range(n)
                                        for g in range(k // 128)], dtype=np.float32).reshape(n, -1))
    got = prefill_raw(x, w, s, m, n, k, 128, True)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32, mode=1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_prefill_config3_sampled_rows(dev):
    m, n, k = 2048, 14336, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=0)
    got = prefill_raw(x, w, s, m, n, k, 128, False)
    rows = np.array([0, 1, 127, 128, 777, 1023, 1024, 2047])
    want1 = oracle.int4_rowmajor_linear(x[rows], w, s, len(rows), n, k, mode=1)
    g, w1 = synth.bf16_bits_to_f32(got[rows]), synth.bf16_bits_to_f32(want1)
    assert rel_err(g, w1) <= 1e-2
    big = np.abs(w1) >= 1e-2 * np.sqrt(np.mean(w1.astype(np.float64) ** 2))
    ulp = np.abs(got[rows].astype(np.int32) - want1.astype(np.int32))
    assert ulp[big].max() <= 1
    # Against the un-rounded weights (the decode path's semantics) every weight differs by its bf16 rounding
    # (2^-9 relative, independent per weight), which moves an output by ~1e-3 of the output RMS whatever its own
    # size; the 1e-2 window is therefore taken relative to max(|want|, output RMS) for this cross-check.
    want0 = oracle.int4_rowmajor_linear(x[rows], w, s, len(rows), n, k, mode=0)
    assert rel_err(g, synth.bf16_bits_to_f32(want0), floor_frac=1.0) <= 1e-2
    # the contract path picks the tensor-core kernel for this batch and returns the same bits
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, k, n, 128, ffi.DT_BF16)
    out = vb.ArtifactSession.compile(prog, dev).run_host([x, w.view(np.uint32), s])[0]
    assert np.array_equal(np.frombuffer(out, np.uint16).reshape(m, n), got)


def test_prefill_and_decode_paths_agree():
    # same inputs through the skinny-GEMM path (8 rows per pass) and the tensor-core path
    m, n, k = 64, 512, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=11)
    a = synth.bf16_bits_to_f32(prefill_raw(x, w, s, m, n, k, 128, False))
    want = synth.bf16_bits_to_f32(oracle.int4_rowmajor_linear(x, w, s, m, n, k, mode=0))
    assert rel_err(a, want, floor_frac=1.0) <= 1e-2  # bf16-rounded vs exact weights: window relative to the RMS
    assert rel_err(a, synth.bf16_bits_to_f32(oracle.int4_rowmajor_linear(x, w, s, m, n, k, mode=1))) <= 1e-2
