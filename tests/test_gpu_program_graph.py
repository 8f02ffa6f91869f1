"""ProgramGraphs on the device: GraphSession walks the schedule, one materialised Program per node, values as resident
buffers, constants uploaded once (or loaded from a safetensors shard). Checked against the oracle's composition of the
same nodes: byte-exact for the reference-order dense nodes, within the path's bf16 tolerance for the quantized ones."""
import json
import struct

import numpy as np
import pytest

import oracle
import vyre_b200 as vb
from vyre_b200 import api, ffi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    d = vb.Device.acquire(0)
    yield d
    d.release()


def test_dense_gated_mlp_contract_fixtures_on_the_device(dev):
    # vyre-libs/tests/dense_gated_mlp_graph_contract.rs: the reference's own fixtures of the connected block
    f = lambda a: np.array(a, np.float32)  # noqa: E731

    def block(spec, consts, residual):
        sess = api.GraphSession(api.dense_gated_mlp_graph(spec), dev)
        try:
            for name, data in consts.items():
                sess.set_constant(name, data)
            out = sess.run({"residual": residual})["mlp.block_output"]
            assert sess.run_chained({"residual": residual})["mlp.block_output"] == out
            return out
        finally:
            sess.close()

    silu_one = np.float32(1.0) / (np.float32(1.0) + np.exp(np.float32(-1.0)))
    eye = f([1.0, 0.0, 0.0, 1.0])
    names = ("post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")
    # :124-149
    got = np.frombuffer(block(api.DenseGatedMlpSpec(1, 2, 2, 2, ffi.DT_F32, norm_eps=0.0), dict(zip(names, (f([1.0, 1.0]), eye, eye, eye))),
                              f([1.0, 1.0, 2.0, 2.0])), np.float32)
    assert np.abs(got - f([1 + silu_one, 1 + silu_one, 2 + silu_one, 2 + silu_one])).max() < 1e-6
    # :151-177
    got = np.frombuffer(block(api.DenseGatedMlpSpec(1, 1, 2, 1, ffi.DT_F32, norm_eps=0.0),
                              dict(zip(names, (f([1.0, 1.0]), f([1.0, 0.0]), f([0.0, 1.0]), f([2.0, 3.0])))), f([1.0, 1.0])), np.float32)
    assert abs(got[0] - (1.0 + 2.0 * silu_one)) < 1e-6 and abs(got[1] - (1.0 + 3.0 * silu_one)) < 1e-6
    # :179-206: the exact BF16 word
    b = oracle.f32_to_bf16_bits
    one = b(f([1.0]))
    got = np.frombuffer(block(api.DenseGatedMlpSpec(1, 1, 1, 1, ffi.DT_BF16, norm_eps=0.0), dict(zip(names, (one, one, one, one))),
                              b(f([2.0]))), np.uint16)
    silu_rounded = oracle.bf16_bits_to_f32(b(f([silu_one])))[0]
    assert got.tolist() == b(f([2.0 + silu_rounded])).tolist()


@pytest.mark.parametrize("dtype,odt", [(ffi.DT_F32, oracle.DT_F32), (ffi.DT_BF16, oracle.DT_BF16)])
def test_dense_gated_mlp_graph_matches_the_oracle_composition(dev, dtype, odt):
    batch, seq, h, inter = 2, 3, 40, 24
    rows = batch * seq
    rng = np.random.default_rng(3)
    f = lambda *shape: rng.standard_normal(shape).astype(np.float32)  # noqa: E731
    x, wg, wu, wd = f(rows, h) * 2.0, f(inter, h) * 0.3, f(inter, h) * 0.3, f(h, inter) * 0.3
    wn = (1.0 + 0.1 * f(h)).astype(np.float32)
    if dtype == ffi.DT_BF16:
        x, wg, wu, wd, wn = (oracle.f32_to_bf16_bits(a) for a in (x, wg, wu, wd, wn))
    sess = api.GraphSession(api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(batch, seq, h, inter, dtype, norm_eps=1e-5)), dev)
    try:
        sess.set_constant("post_attention_layernorm.weight", wn)
        sess.set_constant("mlp.gate_proj.weight", wg)
        sess.set_constant("mlp.up_proj.weight", wu)
        sess.set_constant("mlp.down_proj.weight", wd)
        for _ in range(2):  # a session runs again and again over the same constants
            got = sess.run({"residual": x})["mlp.block_output"]
        normed = oracle.rms_norm(x, wn, rows, h, 1e-5, dtype=odt)
        gate = oracle.linear_rows(normed, wg, None, rows, h, inter, dtype=odt, weight_out_in=True)
        up = oracle.linear_rows(normed, wu, None, rows, h, inter, dtype=odt, weight_out_in=True)
        act = oracle.swiglu(gate, up, dtype=odt)
        down = oracle.linear_rows(act, wd, None, rows, inter, h, dtype=odt, weight_out_in=True)
        want = oracle.residual_add(x, down, dtype=odt)
        if dtype == ffi.DT_F32:
            # the projections are byte-exact against the oracle; SwiGLU's exp sits in the reference's 128-ULP window
            np.testing.assert_allclose(np.frombuffer(got, np.float32), want, rtol=2e-5, atol=1e-6)
        else:
            a, b = oracle.bf16_bits_to_f32(np.frombuffer(got, np.uint16)), oracle.bf16_bits_to_f32(want)
            assert np.abs(a - b).max() <= 2 ** -7 * max(1.0, np.abs(b).max())  # one bf16 ulp of the activation, propagated
        with pytest.raises(vb.BackendError, match="bind the graph input"):
            sess.run({})
        with pytest.raises(vb.BackendError, match="needs .* bytes by its contract"):
            sess.run({"residual": x[:1]})
    finally:
        sess.close()


def test_quantized_gated_mlp_graph_with_constants_from_a_safetensors_shard(dev, tmp_path):
    rows, h, inter = 3, 2048, 4096  # both projections take the decode GEMV
    x, wg, sg = synth.int4_linear_inputs(rows, inter, h, seed=5)
    _, wu, su = synth.int4_linear_inputs(rows, inter, h, seed=6)
    _, wd, sd = synth.int4_linear_inputs(rows, h, inter, seed=7)
    x = oracle.f32_to_bf16_bits(oracle.bf16_bits_to_f32(x) * 0.25)
    tensors = {"mlp.gate_proj.qweight": wg, "mlp.gate_proj.scales": sg, "mlp.up_proj.qweight": wu, "mlp.up_proj.scales": su,
               "mlp.down_proj.qweight": wd, "mlp.down_proj.scales": sd}
    header, blob = {}, b""
    for name, a in tensors.items():
        raw = a.tobytes()
        header[name] = {"dtype": "U8" if a.dtype == np.uint8 else "BF16", "shape": list(a.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hdr = json.dumps(header).encode()
    path = tmp_path / "mlp.safetensors"
    path.write_bytes(struct.pack("<Q", len(hdr)) + hdr + blob)

    graph = api.quantized_gated_mlp_graph(api.QuantizedGatedMlpSpec(rows, h, inter))
    sess = api.GraphSession(graph, dev)
    try:
        idx = api.SafetensorIndex.open(str(path))
        for name in tensors:
            sess.set_constant(name, handle=idx.load_resident(dev, name))
        got = oracle.bf16_bits_to_f32(np.frombuffer(sess.run({"mlp.normalized": x})["mlp.down"], np.uint16)).reshape(rows, h)
        gate = oracle.int4_rowmajor_linear(x, wg, sg, rows, inter, h)
        up = oracle.int4_rowmajor_linear(x, wu, su, rows, inter, h)
        act = oracle.swiglu(gate.reshape(-1), up.reshape(-1), dtype=oracle.DT_BF16)
        want = oracle.bf16_bits_to_f32(oracle.int4_rowmajor_linear(act, wd, sd, rows, h, inter)).reshape(rows, h)
        scale = np.sqrt((want ** 2).mean())
        assert np.abs(got - want).max() <= 2e-2 * max(scale, np.abs(want).max() * 0.1), (np.abs(got - want).max(), scale)
        # and byte for byte against the same three operators submitted one by one
        def op(prog, arrays):
            return vb.ArtifactSession.compile(prog, dev).run_host(arrays)[0]
        g1 = np.frombuffer(op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, h, inter, 128, ffi.DT_BF16), [x, wg.view(np.uint32), sg]), np.uint16)
        u1 = np.frombuffer(op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, h, inter, 128, ffi.DT_BF16), [x, wu.view(np.uint32), su]), np.uint16)
        a1 = np.frombuffer(op(vb.swiglu_typed("g", "u", "o", rows * inter, ffi.DT_BF16), [g1, u1]), np.uint16)
        d1 = op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, inter, h, 128, ffi.DT_BF16), [a1, wd.view(np.uint32), sd])
        assert sess.run({"mlp.normalized": x})["mlp.down"] == d1
    finally:
        sess.close()
    # the whole residual block over the same weights: RMSNorm in front, residual add behind, byte for byte against the
    # five operators submitted one by one
    whole = api.GraphSession(api.quantized_gated_mlp_graph(api.QuantizedGatedMlpSpec(rows, h, inter, norm_eps=1e-5)), dev)
    try:
        idx = api.SafetensorIndex.open(str(path))
        for name in tensors:
            whole.set_constant(name, handle=idx.load_resident(dev, name))
        wn = oracle.f32_to_bf16_bits((1.0 + 0.1 * np.random.default_rng(8).standard_normal(h)).astype(np.float32))
        whole.set_constant("post_attention_layernorm.weight", wn)
        got = whole.run({"residual": x})["mlp.block_output"]
        n1 = np.frombuffer(op(vb.learned_rms_norm("i", "w", "o", rows, h, 1e-5, ffi.DT_BF16), [x, wn]), np.uint16)
        # rows of 2048 elements take the tree form of the sum of squares: equal to the oracle's chain except for rare flips
        nd = np.abs(n1.astype(np.int32) - oracle.rms_norm(x, wn, rows, h, 1e-5, dtype=oracle.DT_BF16).astype(np.int32))
        assert nd.max() <= 2 and np.mean(nd != 0) < 0.01
        g1 = np.frombuffer(op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, h, inter, 128, ffi.DT_BF16), [n1, wg.view(np.uint32), sg]), np.uint16)
        u1 = np.frombuffer(op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, h, inter, 128, ffi.DT_BF16), [n1, wu.view(np.uint32), su]), np.uint16)
        a1 = np.frombuffer(op(vb.swiglu_typed("g", "u", "o", rows * inter, ffi.DT_BF16), [g1, u1]), np.uint16)
        d1 = np.frombuffer(op(vb.linear_int4_grouped_rowmajor("x", "w", "s", "o", rows, inter, h, 128, ffi.DT_BF16), [a1, wd.view(np.uint32), sd]), np.uint16)
        assert got == op(vb.residual_add_typed("r", "b", "o", rows * h, ffi.DT_BF16), [x.reshape(-1), d1])
        names = [n["name"] for n in whole.graph.nodes()] if hasattr(whole, "graph") else None
        assert names is None or names == ["mlp.norm", "mlp.gate_proj", "mlp.up_proj", "mlp.swiglu", "mlp.down_proj", "mlp.residual"]
    finally:
        whole.close()
