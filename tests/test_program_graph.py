"""ProgramGraph construction rules (vyre-foundation/src/ir_inner/model/program_graph.rs:217-470, 541-634) and the gated-MLP
templates. CPU only: graphs are host metadata."""
import pytest

import vyre_b200 as vb
from vyre_b200 import api, ffi

F32, INV, CONST, RET, OUT = ffi.DT_F32, ffi.LIFETIME_INVOCATION, ffi.LIFETIME_CONSTANT, ffi.LIFETIME_RETAINED, ffi.LIFETIME_OUTPUT
RO, RW = ffi.ACCESS_READ_ONLY, ffi.ACCESS_READ_WRITE
C = api.value_contract


def refuses(fn, fragment):
    with pytest.raises(vb.BackendError) as e:
        fn()
    assert e.value.code == ffi.ERR_INVALID_PROGRAM and "Fix:" in str(e.value) and fragment in str(e.value), str(e.value)


def test_from_program_lifts_every_host_visible_buffer():
    prog = vb.softmax_top_k("scores", "idx", "w", 8, 2)  # read-only, output, read-write and two read-write scratch buffers
    g = api.ProgramGraph.from_program("topk", prog)
    vals = {v["name"]: v for v in g.values()}
    assert vals["scores"]["contract"] == {"dtype": F32, "access": RO, "lifetime": INV, "shape": [8]} and vals["scores"]["producer"] is None
    assert vals["w"]["contract"]["lifetime"] == RET and vals["w"]["producer"] is None  # read-write: retained, external
    assert vals["idx"]["contract"]["lifetime"] == OUT and vals["idx"]["producer"] == 0
    (node,) = g.nodes()
    assert node["name"] == "topk" and node["program"].op_id == "vyre-libs::nn::softmax_top_k"
    # workgroup scratch stays inside the node
    gate = api.ProgramGraph.from_program("gate", vb.moe_gate("s", "i", "w", 8, 2))
    assert sorted(v["name"] for v in gate.values()) == ["i", "s", "w"]
    # launch-padded outputs carry their logical element count
    aff = api.ProgramGraph.from_program("aff", vb.linear_4bit_affine_grouped("x", "w", "s", "z", "b", "out", 8, 2, 4))
    assert {v["name"]: v["contract"]["shape"] for v in aff.values()}["out"] == [2]


def test_node_rules():
    sw = vb.swiglu("gate", "up", "out", 16)
    g = api.ProgramGraph()
    a = g.add_external_value("a", C(F32, [16], INV))
    b = g.add_external_value("b", C(F32, [4, 4], INV))
    refuses(lambda: g.add_external_value("a", C(F32, [16], INV)), "duplicate graph name `a`")
    ok_out = [("out", "y", C(F32, [16], OUT, RW))]
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("up", 99, C(F32, [16], INV))], ok_out), "graph value 99 does not exist")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("nope", b, C(F32, [4, 4], INV))], ok_out), "has no buffer `nope`")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("gate", b, C(F32, [4, 4], INV))], ok_out), "binds buffer `gate` more than once")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("up", a, C(F32, [16], INV))], ok_out), "binds graph value 0 more than once")
    # the consumer's contract must equal the value's dtype, shape and lifetime
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], CONST)), ("up", b, C(F32, [4, 4], INV))], ok_out), "expects another dtype, shape or lifetime")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [4, 4], INV)), ("up", b, C(F32, [4, 4], INV))], ok_out), "expects another dtype, shape or lifetime")
    # the Program's buffer must agree with the contract: element type, element count, access, role
    h = g.add_external_value("h", C(ffi.DT_BF16, [16], INV))
    refuses(lambda: g.add_node("n", sw, [("gate", h, C(ffi.DT_BF16, [16], INV)), ("up", b, C(F32, [4, 4], INV))], ok_out), "Program uses dtype tag")
    c = g.add_external_value("c", C(F32, [15], INV))
    refuses(lambda: g.add_node("n", sw, [("gate", c, C(F32, [15], INV)), ("up", b, C(F32, [4, 4], INV))], ok_out),
            "Program declares 16 elements, graph shape requires 15")
    w = g.add_external_value("w", C(F32, [16], RET, RW))
    refuses(lambda: g.add_node("n", sw, [("gate", w, C(F32, [16], RET, RW)), ("up", b, C(F32, [4, 4], INV))], ok_out), "does not satisfy graph access")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("up", b, C(F32, [4, 4], INV))], [("gate", "y", C(F32, [16], OUT, RW))]),
            "binds buffer `gate` more than once")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV))], [("up", "y", C(F32, [16], OUT, RO))]), "Output port cannot use ReadOnly access")
    refuses(lambda: g.add_node("a", sw, [("gate", a, C(F32, [16], INV)), ("up", b, C(F32, [4, 4], INV))], ok_out), "duplicate graph name `a`")
    refuses(lambda: g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("up", b, C(F32, [4, 4], INV))], [("out", "b", C(F32, [16], OUT, RW))]),
            "duplicate graph name `b`")
    refuses(lambda: g.add_node("n", vb.swiglu("g", "u", "o", 0), [], []), "trap program")
    # nothing above changed the graph; a valid node commits, and a second one consumes its output
    assert len(g.nodes()) == 0 and len(g.values()) == 5
    nid, (y,) = g.add_node("n", sw, [("gate", a, C(F32, [16], INV)), ("up", b, C(F32, [4, 4], INV))], [("out", "y", C(F32, [16], INV, RW))])
    nid2, (z,) = g.add_node("n2", sw, [("gate", y, C(F32, [16], INV)), ("up", a, C(F32, [16], INV))], [("out", "z", C(F32, [16], OUT, RW))])
    vals = g.values()
    assert (nid, nid2, g.schedule()) == (0, 1, [0, 1]) and vals[y]["producer"] == 0 and vals[y]["live"] == (0, 1) and vals[a]["live"] == (0, 1)
    assert vals[z]["live"] == (1, 1) and vals[b]["consumers"] == 1 and vals[a]["consumers"] == 2


def test_retained_successors():
    tk = vb.softmax_top_k("scores", "idx", "w", 8, 2)  # w, best_vals, best_idxs are read-write
    g = api.ProgramGraph()
    s = g.add_external_value("s", C(F32, [8], INV))
    w0 = g.add_external_value("w0", C(F32, [2], RET, RW))
    other = g.add_external_value("other", C(F32, [2], RET, RW))
    ins = [("scores", s, C(F32, [8], INV)), ("w", w0, C(F32, [2], RET, RW))]
    idx_out = ("idx", "idx0", C(ffi.DT_U32, [2], OUT, RW))
    refuses(lambda: g.add_node("n", tk, ins, [idx_out, ("w", "w1", C(F32, [2], RET, RW), other)]), "without consuming that prior value")
    refuses(lambda: g.add_node("n", tk, ins, [idx_out, ("w", "w1", C(F32, [2], OUT, RW), w0)]), "not a type-preserving successor")
    refuses(lambda: g.add_node("n", tk, ins, [idx_out, ("w", "w1", C(F32, [2], RET, RW))]), "binds buffer `w` more than once")
    _, (i0, w1) = g.add_node("n", tk, ins, [idx_out, ("w", "w1", C(F32, [2], RET, RW), w0)])  # the same buffer, rebound to its successor
    assert g.values()[w1]["retained_successor_of"] == w0 and g.values()[i0]["producer"] == 0


def test_gated_mlp_templates():
    g = api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(batch=2, sequence=3, hidden_dim=8, intermediate_dim=12, dtype=ffi.DT_BF16))
    names = [n["name"] for n in g.nodes()]
    assert names == ["mlp.norm", "mlp.gate_proj", "mlp.up_proj", "mlp.swiglu", "mlp.down_proj", "mlp.residual"]
    vals = {v["name"]: v for v in g.values()}
    assert vals["mlp.gate_proj.weight"]["contract"] == {"dtype": ffi.DT_BF16, "access": RO, "lifetime": CONST, "shape": [12, 8]}
    assert vals["mlp.down_proj.weight"]["contract"]["shape"] == [8, 12] and vals["mlp.block_output"]["contract"]["lifetime"] == OUT
    assert vals["post_attention_layernorm.weight"]["contract"] == {"dtype": ffi.DT_BF16, "access": RO, "lifetime": CONST, "shape": [8]}
    assert vals["residual"]["consumers"] == 2  # the norm and the residual add (dense_gated_mlp.rs:171-200, 331-346)
    assert vals["mlp.normalized"]["consumers"] == 2 and vals["mlp.activated"]["contract"]["shape"] == [2, 3, 12]
    assert [n["program"].op_id for n in g.nodes()] == ["vyre-libs::nn::learned_rms_norm", "vyre-libs::nn::linear_rows", "vyre-libs::nn::linear_rows",
                                                       "vyre-libs::nn::swiglu", "vyre-libs::nn::linear_rows", "vyre-libs::nn::residual_add"]
    assert g.digest() != api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(2, 3, 8, 12, ffi.DT_BF16, norm_eps=1e-5)).digest()
    same = api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(2, 3, 8, 12, ffi.DT_BF16))
    other = api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(2, 3, 8, 16, ffi.DT_BF16))
    assert g.digest() == same.digest() != other.digest()
    refuses(lambda: api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(0, 3, 8, 12)), "must be nonzero")
    refuses(lambda: api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(1, 3, 8, 12, ffi.DT_U32)), "dtype must be F16, BF16, or F32")
    # vyre-libs/tests/dense_gated_mlp_graph_contract.rs:207-235 graph_stage_order_is_canonical
    canon = api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(1, 1, 2, 3, ffi.DT_F32, norm_eps=1e-6))
    assert [n["name"] for n in canon.nodes()] == names
    # :237-262 production_qwen35_dimensions_build_exact_weight_contracts
    big = {n["name"]: n for n in api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(1, 1, 5120, 17408, ffi.DT_BF16, norm_eps=1e-6)).nodes()}
    assert big["mlp.gate_proj"]["program"].buffers()[1]["count"] == 17408 * 5120
    assert big["mlp.down_proj"]["program"].buffers()[1]["count"] == 5120 * 17408
    # :264-291 invalid_dense_mlp_contracts_are_rejected (the empty batch and the integer dtype are refused above)
    with pytest.raises(api.BackendError):
        api.dense_gated_mlp_graph(api.DenseGatedMlpSpec(0xFFFFFFFF, 2, 2, 2, ffi.DT_F32))
    q = api.quantized_gated_mlp_graph(api.QuantizedGatedMlpSpec(rows=4, hidden_dim=256, intermediate_dim=512))
    qv = {v["name"]: v for v in q.values()}
    assert qv["mlp.gate_proj.qweight"]["contract"] == {"dtype": ffi.DT_U32, "access": RO, "lifetime": CONST, "shape": [512, 32]}
    assert qv["mlp.down_proj.scales"]["contract"]["shape"] == [256, 4] and [n["name"] for n in q.nodes()] == names[1:5]
    qw = api.quantized_gated_mlp_graph(api.QuantizedGatedMlpSpec(rows=4, hidden_dim=256, intermediate_dim=512, norm_eps=1e-6))
    assert [n["name"] for n in qw.nodes()] == names
    qwv = {v["name"]: v for v in qw.values()}
    assert qwv["residual"]["consumers"] == 2 and qwv["mlp.block_output"]["contract"]["lifetime"] == OUT
    assert qwv["mlp.down"]["contract"]["lifetime"] != OUT and qw.digest() != q.digest()
