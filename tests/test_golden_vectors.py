"""Committed golden vectors (tests/golden/vectors.npz, made by tests/golden/make_golden.py).

CPU: the oracle still reproduces them byte for byte (guards the checker against drift).
GPU: the kernels, called through the C ABI, match them - bit-exact for the integer path, within the stated windows for
floating point - without the oracle being involved at run time.
"""
import ctypes as C
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(GOLDEN))


def test_oracle_reproduces_the_committed_vectors(gold):
    import sys

    sys.path.insert(0, os.path.join(os.path.dirname(GOLDEN)))
    import make_golden

    fresh = make_golden.build()
    assert sorted(fresh) == sorted(gold)
    for k in gold:
        assert fresh[k].dtype == gold[k].dtype and np.array_equal(fresh[k], gold[k]), k


@pytest.mark.gpu
def test_kernels_match_the_committed_vectors(gold):
    import torch

    from vyre_b200 import ffi, synth

    L = ffi.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    dev = lambda a: torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a).cuda()  # noqa: E731

    # int4 decode GEMV: f32 accumulate <= 1e-4, bf16 out <= 1e-2 (relative, against max(|want|, 1% of the RMS))
    x, w, s = dev(gold["gemv_x"]), dev(gold["gemv_w"]), dev(gold["gemv_s"])
    m, n, k = 2, 64, 1024
    for name, dt, tdt, tol in (("gemv_y_f32", ffi.DT_F32, torch.float32, 1e-4), ("gemv_y_bf16", ffi.DT_BF16, torch.bfloat16, 1e-2)):
        y = torch.zeros((m, n), dtype=tdt, device="cuda")
        ffi.check(L.vyb_k_int4_gemv(x.data_ptr(), w.data_ptr(), s.data_ptr(), y.data_ptr(), m, n, k, 128, dt, stream,
                                    C.c_void_p(status.data_ptr())))
        torch.cuda.synchronize()
        want = gold[name].reshape(m, n)
        want = synth.bf16_bits_to_f32(want) if want.dtype == np.uint16 else want
        got = y.float().cpu().numpy()
        floor = 1e-2 * float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
        assert np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)) <= tol, name

    # int8 dynamic linear: quantiser and int32 GEMM are bit-exact
    rows, kk, nn = gold["i8_q"].shape[0], gold["i8_q"].shape[1], gold["i8_w"].shape[0]
    xa, wa = dev(gold["i8_x"]), dev(gold["i8_w"])
    q = torch.empty((rows, kk), dtype=torch.int8, device="cuda")
    sc = torch.empty(rows, dtype=torch.float32, device="cuda")
    y = torch.empty((rows, nn), dtype=torch.int32, device="cuda")
    ffi.check(L.vyb_k_quantize_per_token_int8(xa.data_ptr(), q.data_ptr(), sc.data_ptr(), rows, kk, stream))
    ffi.check(L.vyb_k_int8_gemm_i32(q.data_ptr(), wa.data_ptr(), y.data_ptr(), rows, nn, kk, stream,
                                    C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), gold["i8_q"]) and np.array_equal(sc.cpu().numpy(), gold["i8_scale"])
    assert np.array_equal(y.cpu().numpy(), gold["i8_y"])

    # MoE FFN layer: routing exact, outputs within 2e-2 of max(|want|, output RMS) (single bf16-ulp flips of an
    # expert output, scaled by its gate weight)
    t, h = gold["moe_x"].shape
    e, i = gold["moe_w13"].shape[0], gold["moe_w13"].shape[2]
    topk = gold["moe_idx"].shape[1]
    need = C.c_uint64(0)
    ffi.check(L.vyb_k_moe_ffn_int4_scratch_bytes(t, h, i, e, topk, C.byref(need)))
    ten = [dev(gold[k_]) for k_ in ("moe_x", "moe_wr", "moe_w13", "moe_s13", "moe_w2", "moe_s2")]
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    idx = torch.empty((t, topk), dtype=torch.int32, device="cuda")
    wts = torch.empty((t, topk), dtype=torch.float32, device="cuda")
    scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    ffi.check(L.vyb_k_moe_ffn_int4(*[a.data_ptr() for a in ten], out.data_ptr(), idx.data_ptr(), wts.data_ptr(),
                                   scratch.data_ptr(), need.value, t, h, i, e, topk, 128, stream, C.c_void_p(status.data_ptr())))
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), gold["moe_idx"])
    assert np.allclose(wts.cpu().numpy(), gold["moe_wts"], rtol=2e-5, atol=1e-7)
    want = synth.bf16_bits_to_f32(gold["moe_out"]).astype(np.float64)
    got = out.float().cpu().numpy().astype(np.float64)
    floor = float(np.sqrt(np.mean(want ** 2)))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)) <= 2e-2


@pytest.mark.gpu
def test_operators_around_the_block_match_the_committed_vectors(gold):
    """Residual add, learned RMSNorm (chain-order rows) and the K-quant programs through the contract path: bit-exact."""
    import vyre_b200 as vb
    from vyre_b200 import ffi

    dev = vb.Device.acquire(0)
    try:
        run = lambda program, inputs: vb.ArtifactSession.compile(program, dev).run_host(inputs)[0]  # noqa: E731
        n = gold["res_a"].size
        got = np.frombuffer(run(vb.residual_add_typed("r", "b", "o", n, ffi.DT_BF16), [gold["res_a"], gold["res_b"]]), np.uint16)
        assert np.array_equal(got, gold["res_out"])
        rows, hidden = gold["norm_out_f32"].shape
        got = np.frombuffer(run(vb.learned_rms_norm("i", "w", "o", rows, hidden, 1e-6, ffi.DT_F32),
                                [gold["norm_x"], gold["norm_w"]]), np.uint32)
        assert np.array_equal(got, gold["norm_out_f32"].view(np.uint32).ravel())
        from vyre_b200 import synth

        xb, wb = synth.f32_to_bf16_bits(gold["norm_x"]), synth.f32_to_bf16_bits(gold["norm_w"])
        got = np.frombuffer(run(vb.learned_rms_norm("i", "w", "o", rows, hidden, 1e-6, ffi.DT_BF16), [xb, wb]), np.uint16)
        assert np.array_equal(got, gold["norm_out_bf16"].ravel())
        for bits, unpack, linear in ((4, vb.q4_k_unpack, vb.q4_k_linear), (2, vb.q2_k_unpack, vb.q2_k_linear)):
            g = {k: gold[f"q{bits}k_{k}"] for k in ("packed", "scales", "mins", "x", "b", "unpacked", "y")}
            in_dim, out_dim = g["x"].size, g["b"].size
            got = np.frombuffer(run(unpack("p", "s", "m", "o", in_dim * out_dim), [g["packed"], g["scales"], g["mins"]]), np.uint32)
            assert np.array_equal(got, g["unpacked"].view(np.uint32))
            got = np.frombuffer(run(linear("x", "p", "s", "m", "b", "o", in_dim, out_dim),
                                    [g["x"], g["packed"], g["scales"], g["mins"], g["b"]]), np.uint32)
            assert np.array_equal(got, g["y"].view(np.uint32))
    finally:
        dev.release()
