"""The int4 projection with the learned RMSNorm in front and / or SwiGLU or the residual add behind as ONE node
(`linear_int4_block`) on the device: the node's values are the bits of the three stand-alone operators run one after
the other (every intermediate is rounded where they round), for the shapes whose decode kernel takes the parts into its
own launch (kernel variant 9) and for the shapes that run the stand-alone kernels inside the node; against the CPU
oracle within the projection's bf16 window; the graph pass that forms such nodes leaves the block's output unchanged."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
import vyre_b200 as vb
from vyre_b200 import api, ffi, synth

pytestmark = pytest.mark.gpu
TOL_BF16_OUT = 1e-2  # relative to max(|want|, 1% of the RMS): one bf16 rounding of an f32 sum that differs in its last bits
BF16 = ffi.DT_BF16


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def rel_err(got, want):
    floor = 1e-2 * float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


def run(dev, program, inputs):
    sess = vb.ArtifactSession.compile(program, dev)
    return sess.kernel_variant(), np.frombuffer(sess.run_host(inputs)[0], np.uint16)


def block_inputs(m, n, k, seed):
    x, w, s = synth.int4_linear_inputs(m, n, k, seed=seed)
    rng = np.random.default_rng(seed + 1)
    x = synth.f32_to_bf16_bits(synth.bf16_bits_to_f32(x) * 3.0)  # rows whose RMS is not one
    nw = synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(k)).astype(np.float32))
    res = synth.f32_to_bf16_bits(rng.standard_normal((m, n)).astype(np.float32))
    return x, w.view(np.uint32), s, nw, res


def gate_inputs(m, n, seed):
    return synth.f32_to_bf16_bits((np.random.default_rng(seed + 2).standard_normal((m, n)) * 2).astype(np.float32))


@pytest.mark.parametrize("m,n,k,variant", [
    (1, 1000, 4096, 9), (2, 4736, 4096, 9), (1, 48, 2048, 9), (2, 2400, 2048, 9),  # one launch
    (1, 520, 8192, 9), (4, 300, 14336, 9), (3, 96, 6144, 9),                       # long rows: the residual joins the launch
    (3, 256, 4096, 1), (8, 130, 2048, 1), (1, 200, 3072, 1), (1, 64, 96, 0), (70, 128, 512, 2),  # stand-alone kernels in the node
])
@pytest.mark.parametrize("parts", ["norm", "residual", "both", "swiglu", "norm+swiglu"])
def test_block_node_equals_the_operators_in_sequence(dev, m, n, k, variant, parts):
    group = 128 if k % 128 == 0 else 32
    x, w, s, nw, res = block_inputs(m, n, k, seed=m * 1000 + n + k)
    if group != 128:
        s = synth.f32_to_bf16_bits(np.random.default_rng(5).uniform(1e-3, 2e-2, size=(n, k // group)).astype(np.float32))
    eps = 1e-6
    norm, gated, resid = parts in ("norm", "both", "norm+swiglu"), parts.endswith("swiglu"), parts in ("residual", "both")
    gate = gate_inputs(m, n, seed=n)
    prog = vb.linear_int4_block("x", "nw" if norm else None, "w", "s", "res" if resid else None, "out", m, k, n, group, eps,
                                gate="g" if gated else None)
    got_variant, got = run(dev, prog, [x] + ([nw] if norm else []) + [w, s] + ([gate] if gated else []) + ([res] if resid else []))
    long_rows = k > 4096 and k % 2048 == 0
    if variant == 9 and long_rows and parts == "norm":
        variant = 1  # the norm of a long row is not part of the k-block launch
    assert got_variant == variant
    # the same operators as separate programs
    xin = x
    if norm:
        xin = run(dev, vb.learned_rms_norm("i", "w", "o", m, k, eps, BF16), [x, nw])[1]
    y = run(dev, vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", m, k, n, group), [xin, w, s])[1]
    if gated:
        y = run(dev, vb.swiglu_typed("g", "u", "o", m * n, BF16), [gate, y])[1]
    if resid:
        y = run(dev, vb.residual_add_typed("r", "b", "o", m * n, BF16), [res, y])[1]
    assert np.array_equal(got, y)
    # and the CPU oracle's composition (its norm sums a long row as a chain, the device as a tree: within the projection's window)
    xo = oracle.rms_norm(x, nw, m, k, eps, dtype=oracle.DT_BF16) if norm else x
    # (the tensor-core GEMM of prefill batches multiplies bf16-rounded weights: the oracle's mode 1)
    yo = oracle.int4_rowmajor_linear(xo, w.view(np.uint8), s, m, n, k, group=group, mode=1 if variant == 2 else 0).ravel()
    want = oracle.residual_add(res, yo, oracle.DT_BF16) if resid else yo
    if gated:  # the projection in the window of the stand-alone one, SwiGLU of it in the stand-alone operator's
        want = oracle.swiglu(gate.ravel(), yo, dtype=oracle.DT_BF16)
        a, b = synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)
        up_f = np.abs(synth.bf16_bits_to_f32(yo))
        g_f = synth.bf16_bits_to_f32(gate.ravel())
        slope = np.abs(g_f / (1.0 + np.exp(-g_f.astype(np.float64)))).astype(np.float32)  # |d swiglu / d up|
        floor = 1e-2 * float(np.sqrt(np.mean(up_f.astype(np.float64) ** 2)))
        assert np.all(np.abs(a - b) <= slope * 2 * TOL_BF16_OUT * np.maximum(up_f, floor) + 2.0 ** -7 * np.abs(b) + 1e-30)
        return
    a, b = synth.bf16_bits_to_f32(got), synth.bf16_bits_to_f32(want)
    if resid:  # the add rounds to a bf16 ulp of the sum; the branch's window is relative to the branch
        assert np.max(np.abs(a - b)) <= TOL_BF16_OUT * max(1.0, float(np.abs(synth.bf16_bits_to_f32(yo)).max())) + 2.0 ** -7 * np.abs(b).max()
    else:
        assert rel_err(a, b) <= 2 * TOL_BF16_OUT


def test_outlier_activations_behind_the_norm(dev):
    # one element 2^20 above the rest: after the norm the small elements still need the single-row wide conversion
    m, n, k = 1, 512, 4096
    x, w, s, nw, res = block_inputs(m, n, k, seed=77)
    xf = synth.bf16_bits_to_f32(x).copy()
    xf[0, 1234] = 2.0 ** 20
    x = synth.f32_to_bf16_bits(xf)
    _, got = run(dev, vb.linear_int4_block("x", "nw", "w", "s", "res", "out", m, k, n, 128, 1e-6), [x, nw, w, s, res])
    xin = run(dev, vb.learned_rms_norm("i", "w", "o", m, k, 1e-6, BF16), [x, nw])[1]
    y = run(dev, vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", m, k, n, 128), [xin, w, s])[1]
    y = run(dev, vb.residual_add_typed("r", "b", "o", m * n, BF16), [res, y])[1]
    assert np.array_equal(got, y)


def test_kernel_entry_in_a_captured_chain(dev):
    # the launch pattern of a serving loop: constant weights, programmatic dependent launches, one CUDA graph; the residual
    # of one launch is the output of the launch before
    lib = ffi.lib()
    m, n, k = 1, 4096, 4096
    x, w, s, nw, res = block_inputs(m, n, k, seed=5)
    tx, tw, ts, tnw = (torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a.view(np.int32)).cuda() for a in (x, w, s, nw))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    bufs = [torch.zeros((m, n), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    bufs[0].copy_(tx.view(torch.bfloat16).reshape(m, k))

    def chain(stream):
        for i in range(3):  # h[i+1] = h[i] + W rmsnorm(h[i])
            ffi.check(lib.vyb_k_int4_linear_block(bufs[i].data_ptr(), tnw.data_ptr(), C.c_float(1e-6), tw.data_ptr(), ts.data_ptr(),
                                                  None, bufs[i].data_ptr(), bufs[i + 1].data_ptr(), m, n, k, 128, ffi.LAUNCH_CONSTANT_WEIGHTS,
                                                  C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        chain(side)
    side.synchronize()
    eager = [b.clone() for b in bufs]
    for b in bufs[1:]:
        b.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            chain(side)
        for _ in range(3):
            graph.replay()
    side.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    for a, b in zip(eager, bufs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    # every link against the stand-alone programs
    h = x
    for i in range(3):
        xin = run(dev, vb.learned_rms_norm("i", "w", "o", m, k, 1e-6, BF16), [h, nw])[1]
        y = run(dev, vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", m, k, n, 128), [xin, w, s])[1]
        h = run(dev, vb.residual_add_typed("r", "b", "o", m * n, BF16), [h, y])[1]
        assert np.array_equal(bufs[i + 1].view(torch.int16).cpu().numpy().view(np.uint16).ravel(), h)
    # shapes the kernel does not fuse are refused, not emulated
    rc = lib.vyb_k_int4_linear_block(bufs[0].data_ptr(), tnw.data_ptr(), C.c_float(1e-6), tw.data_ptr(), ts.data_ptr(), None, None,
                                     bufs[1].data_ptr(), 3, n, k, 128, 0, None, None)
    assert rc == ffi.ERR_UNSUPPORTED_FEATURE and b"Fix:" in lib.vyb_last_error_message()
    rc = lib.vyb_k_int4_linear_block(bufs[0].data_ptr(), None, C.c_float(0), tw.data_ptr(), ts.data_ptr(), None, None,
                                     bufs[1].data_ptr(), 1, n, k, 128, 0, None, None)
    assert rc == ffi.ERR_INVALID_PROGRAM
    rc = lib.vyb_k_int4_linear_block(bufs[0].data_ptr(), tnw.data_ptr(), C.c_float(0), tw.data_ptr(), ts.data_ptr(), bufs[2].data_ptr(),
                                     bufs[3].data_ptr(), bufs[1].data_ptr(), 1, n, k, 128, 0, None, None)
    assert rc == ffi.ERR_INVALID_PROGRAM and b"not both" in lib.vyb_last_error_message()


@pytest.mark.parametrize("behind", ["residual", "swiglu"])
def test_long_row_stores_first_use_under_capture(dev, behind):
    # no workspace on a fresh stream while it captures: one launch per k block, then the add / SwiGLU as its own kernel; same bits
    lib = ffi.lib()
    m, n, k = 2, 300, 6144
    x, w, s, _, res = block_inputs(m, n, k, seed=9)
    tx, tw, ts, tres = (torch.from_numpy(a.view(np.int16) if a.dtype == np.uint16 else a.view(np.int32)).cuda() for a in (x, w, s, res))
    ty = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    gate_p, res_p = (tres.data_ptr(), None) if behind == "swiglu" else (None, tres.data_ptr())

    def launch(stream):
        ffi.check(lib.vyb_k_int4_linear_block(tx.data_ptr(), None, C.c_float(0), tw.data_ptr(), ts.data_ptr(), gate_p, res_p,
                                              ty.data_ptr(), m, n, k, 128, 0, C.c_void_p(stream.cuda_stream), C.c_void_p(status.data_ptr())))

    fresh = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(fresh):
        with torch.cuda.graph(graph, stream=fresh):
            launch(fresh)
        graph.replay()
    fresh.synchronize()
    captured = ty.clone()
    ty.zero_()
    with torch.cuda.stream(fresh):
        launch(fresh)  # un-captured: the workspace exists from now on and the stores do it all
    fresh.synchronize()
    assert torch.equal(captured.view(torch.int16), ty.view(torch.int16))
    y = run(dev, vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", m, k, n, 128), [x, w, s])[1]
    if behind == "swiglu":
        y = run(dev, vb.swiglu_typed("g", "u", "o", m * n, BF16), [res, y])[1]
    else:
        y = run(dev, vb.residual_add_typed("r", "b", "o", m * n, BF16), [res, y])[1]
    assert np.array_equal(ty.view(torch.int16).cpu().numpy().view(np.uint16).ravel(), y)
    assert status.cpu().tolist() == [0, 0, 0, 0]


def test_swiglu_in_the_stores_for_every_bf16_gate(dev):
    # Every one of the 65536 bf16 gate values against the stand-alone operator, whole-row and k-block forms. The weights
    # select ONE activation per output (nibble 9 = +1 at position j of row j, 8 = 0 elsewhere, scale 1) and the activations
    # lie in [1, 2), so the projection returns them exactly: up = x.
    for k, n in ((4096, 4096), (6144, 4096)):
        w = np.full((n, k // 2), 0x88, dtype=np.uint8)
        j = np.arange(n)
        w[j, j // 2] = np.where(j % 2 == 0, 0x89, 0x98).astype(np.uint8)
        s = synth.f32_to_bf16_bits(np.ones((n, k // 128), np.float32))
        gates = np.arange(65536, dtype=np.uint16)
        rng = np.random.default_rng(3)
        block = vb.ArtifactSession.compile(vb.linear_int4_block("x", None, "w", "s", None, "out", 1, k, n, 128, gate="g"), dev)
        alone = vb.ArtifactSession.compile(vb.swiglu_typed("g", "u", "o", n, BF16), dev)
        assert block.kernel_variant() == 9
        for c in range(0, 65536, n):
            g = gates[c:c + n]
            x = synth.f32_to_bf16_bits((rng.uniform(1.0, 2.0, k) * rng.choice([-1.0, 1.0], k)).astype(np.float32))
            got = np.frombuffer(block.run_host([x, w.view(np.uint32), s, g])[0], np.uint16)
            want = np.frombuffer(alone.run_host([g, x[:n]])[0], np.uint16)
            nan = (want & 0x7FFF) > 0x7F80
            assert np.array_equal(got[~nan], want[~nan]), (k, c)
            assert np.all((got[nan] & 0x7FFF) > 0x7F80), (k, c)


@pytest.mark.parametrize("rows,hidden,inter", [(1, 4096, 6144), (2, 2048, 4096), (4, 4096, 8192)])
def test_fused_graph_runs_to_the_same_block_output(dev, rows, hidden, inter):
    spec = api.QuantizedGatedMlpSpec(rows, hidden, inter, 128, norm_eps=1e-6)
    graph = api.quantized_gated_mlp_graph(spec)
    fused, taken = graph.fuse_linear_blocks()
    assert taken == (3 if rows <= 2 else 1)
    rng = np.random.default_rng(rows + inter)
    x = synth.f32_to_bf16_bits((rng.standard_normal((rows, hidden)) * 2).astype(np.float32))
    consts = {"post_attention_layernorm.weight": synth.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))}
    for name, (n, k) in {"gate_proj": (inter, hidden), "up_proj": (inter, hidden), "down_proj": (hidden, inter)}.items():
        _, w, s = synth.int4_linear_inputs(1, n, k, seed=len(name) + n)
        consts[f"mlp.{name}.qweight"], consts[f"mlp.{name}.scales"] = w.view(np.uint32), s
    outs = []
    for g in (graph, fused):
        sess = api.GraphSession(g, dev)
        try:
            for name, data in consts.items():
                sess.set_constant(name, data)
            for _ in range(2):
                out = sess.run({"residual": x})["mlp.block_output"]
            outs.append(np.frombuffer(out, np.uint16))
            # the same graph without the host between the nodes: prepared sets, each ordered on the device behind the one before
            x2 = synth.f32_to_bf16_bits((rng.standard_normal((rows, hidden)) * 2).astype(np.float32))
            want2 = sess.run({"residual": x2})["mlp.block_output"]
            for inp, want in ((x, out), (x2, want2), (x, out)):
                assert sess.run_chained({"residual": inp})["mlp.block_output"] == want
            # a constant replaced: the prepared sets are made again over the new buffer
            other = synth.f32_to_bf16_bits(np.ones(hidden, np.float32))
            sess.set_constant("post_attention_layernorm.weight", other)
            assert sess.run_chained({"residual": x})["mlp.block_output"] == sess.run({"residual": x})["mlp.block_output"] != out
            sess.set_constant("post_attention_layernorm.weight", consts["post_attention_layernorm.weight"])
            with pytest.raises(vb.BackendError, match="bind the graph input"):
                sess.run_chained({})
            if g is fused:
                kinds = [s_.kernel_variant() for s_ in sess.sessions]
                assert kinds[-1] == 9 and (rows > 2 or kinds[0] == kinds[1] == 9)
        finally:
            sess.close()
    assert np.array_equal(outs[0], outs[1])
