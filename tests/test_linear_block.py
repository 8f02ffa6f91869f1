"""The int4 projection with its neighbours of the residual block in one node (`linear_int4_block`) and the graph pass that
forms such nodes: builder rules, slot order, the target compiler's choice of kernel, and the rewritten graph's wiring.
Host logic only; the device checks are in test_gpu_linear_block.py."""
import pytest

import vyre_b200 as vb
from vyre_b200 import ffi


def variant(program) -> int:
    return vb.target_compile(vb.compile(program)).kernel_variant()


def test_builder_slots_and_errors():
    p = vb.linear_int4_block("x", "nw", "w", "s", "res", "out", 2, 4096, 1024, 128, 1e-6)
    assert p.op_id == "vyre-b200::nn::linear_int4_block" and p.op_id in vb.supported_ops()
    assert [(b["name"], b["binding"], b["count"]) for b in p.buffers()] == [
        ("x", 0, 2 * 4096), ("nw", 1, 4096), ("w", 2, 1024 * 512), ("s", 3, 1024 * 32), ("res", 4, 2 * 1024), ("out", 5, 2 * 1024)]
    assert [b["name"] for b in vb.linear_int4_block("x", None, "w", "s", "res", "out", 1, 4096, 64, 128).buffers()] == \
        ["x", "w", "s", "res", "out"]
    assert [b["name"] for b in vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 4096, 64, 128, 1e-5).buffers()] == \
        ["x", "nw", "w", "s", "out"]
    assert [(b["name"], b["binding"], b["count"]) for b in
            vb.linear_int4_block("x", "nw", "w", "s", None, "out", 2, 4096, 64, 128, 1e-6, gate="g").buffers()] == \
        [("x", 0, 8192), ("nw", 1, 4096), ("w", 2, 64 * 512), ("s", 3, 64 * 32), ("g", 4, 128), ("out", 5, 128)]
    with pytest.raises(vb.BackendError, match="needs a norm weight, a gate, a residual, or a norm weight with one of the two"):
        vb.linear_int4_block("x", None, "w", "s", None, "out", 1, 4096, 64, 128)
    with pytest.raises(vb.BackendError, match="a gate or a residual behind the projection, not both"):
        vb.linear_int4_block("x", "nw", "w", "s", "res", "out", 1, 4096, 64, 128, 1e-6, gate="g")
    with pytest.raises(vb.BackendError, match="requires nonzero batch, in_dim, out_dim and group_size; got batch=0"):
        vb.linear_int4_block("x", "nw", "w", "s", None, "out", 0, 4096, 64, 128)
    with pytest.raises(vb.BackendError, match="in_dim=100 is not divisible by 8"):
        vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 100, 64, 4)
    with pytest.raises(vb.BackendError, match="is not a multiple of group_size=128"):
        vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 192, 64, 128)
    with pytest.raises(vb.BackendError, match="non-negative"):
        vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 4096, 64, 128, -1.0)
    with pytest.raises(vb.BackendError, match="overflow u32"):
        vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1 << 20, 1 << 13, 64, 128)
    # different epsilons, different programs
    a = vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 4096, 64, 128, 1e-5).fingerprint()
    assert a != vb.linear_int4_block("x", "nw", "w", "s", None, "out", 1, 4096, 64, 128, 1e-6).fingerprint()


@pytest.mark.parametrize("batch,k,norm,resid,want", [
    (1, 4096, True, True, 9), (2, 2048, True, False, 9), (2, 4096, False, True, 9), (2, 4096, "swiglu", False, 9),
    (4, 14336, "swiglu", False, 9), (1, 4096, "norm+swiglu", False, 9), (1, 14336, "norm+swiglu", False, 9),
    (5, 14336, "swiglu", False, 1), (3, 4096, "swiglu", False, 1),
    (3, 4096, True, True, 1),       # three rows take the f16 tensor path: the parts run as their own kernels
    (1, 14336, False, True, 9),     # long rows: the residual add joins the k-block launch ...
    (4, 8192, False, True, 9),
    (1, 14336, True, False, 1),     # ... the norm of a long row does not
    (1, 14336, True, True, 9),
    (5, 8192, False, True, 1),
    (1, 3072, True, True, 1),       # other k: the bulk-copy GEMV
    (256, 4096, True, True, 2),     # prefill
    (1, 96, True, True, 0),
])
def test_target_compiler_names_the_fused_kernel_only_where_it_exists(batch, k, norm, resid, want):
    group = 128 if k % 128 == 0 else 32
    p = vb.linear_int4_block("x", "nw" if norm in (True, "norm+swiglu") else None, "w", "s", "res" if resid else None, "out", batch,
                             k, 256, group, 1e-6, gate="g" if str(norm).endswith("swiglu") else None)
    assert variant(p) == want
    bare = vb.linear_int4_grouped_rowmajor("x", "w", "s", "out", batch, k, 256, group)
    if want != 9:
        assert variant(bare) == want


def names(graph):
    vals = graph.values()
    return [(n["name"], n["program"].op_id.split("::")[-1], {i["buffer"]: vals[i["value"]]["name"] for i in n["inputs"]},
             [o["name"] for o in n["outputs"]]) for n in graph.nodes()]


def test_graph_pass_takes_norm_and_residual_into_the_projections():
    g = vb.quantized_gated_mlp_graph(vb.QuantizedGatedMlpSpec(1, 4096, 14336, 128, norm_eps=1e-6))
    f, taken = g.fuse_linear_blocks()
    assert taken == 3 and len(f.nodes()) == 3
    got = names(f)
    assert got[0] == ("mlp.gate_proj", "linear_int4_block",
                      {"input": "residual", "weight": "mlp.gate_proj.qweight", "scale": "mlp.gate_proj.scales",
                       "norm_weight": "post_attention_layernorm.weight"}, ["mlp.gate"])
    assert got[1] == ("mlp.up_proj", "linear_int4_block",
                      {"input": "residual", "weight": "mlp.up_proj.qweight", "scale": "mlp.up_proj.scales",
                       "norm_weight": "post_attention_layernorm.weight", "gate": "mlp.gate"}, ["mlp.activated"])
    assert got[2] == ("mlp.down_proj", "linear_int4_block",
                      {"input": "mlp.activated", "weight": "mlp.down_proj.qweight", "scale": "mlp.down_proj.scales",
                       "residual": "residual"}, ["mlp.block_output"])
    vals = {v["name"]: v for v in f.values()}
    assert not {"mlp.normalized", "mlp.up", "mlp.down"} & set(vals)
    assert vals["mlp.block_output"]["contract"]["lifetime"] == ffi.LIFETIME_OUTPUT
    assert vals["residual"]["consumers"] == 3
    assert f.digest() != g.digest()
    # nothing left to take in; the original graph is untouched
    again, taken = f.fuse_linear_blocks()
    assert taken == 0 and again.digest() == f.digest()
    assert len(g.nodes()) == 6


def test_graph_pass_leaves_what_the_kernel_does_not_take():
    # four rows: the gate / up projections run on the f16 tensor path (norm and SwiGLU stay nodes), the long-row down
    # projection still takes the residual add
    f, taken = vb.quantized_gated_mlp_graph(vb.QuantizedGatedMlpSpec(4, 4096, 14336, 128, norm_eps=1e-6)).fuse_linear_blocks()
    assert taken == 1
    assert [n[1] for n in names(f)] == ["learned_rms_norm", "linear_int4_grouped_rowmajor", "linear_int4_grouped_rowmajor",
                                        "swiglu", "linear_int4_block"]
    # without the norm and the residual add around them, the up projection still takes SwiGLU
    f, taken = vb.quantized_gated_mlp_graph(vb.QuantizedGatedMlpSpec(1, 4096, 14336, 128)).fuse_linear_blocks()
    assert taken == 1 and names(f)[1][2]["gate"] == "mlp.gate" and names(f)[1][3] == ["mlp.activated"]
    # prefill rows, and a graph without the two neighbours: unchanged
    for spec in (vb.QuantizedGatedMlpSpec(64, 4096, 8192, 128, norm_eps=1e-6), vb.QuantizedGatedMlpSpec(8, 4096, 14336, 128)):
        g = vb.quantized_gated_mlp_graph(spec)
        f, taken = g.fuse_linear_blocks()
        assert taken == 0 and f.digest() == g.digest()
    # the reference's dense block (f32 / bf16 dense projections) has no int4 linear: unchanged
    g = vb.dense_gated_mlp_graph(vb.DenseGatedMlpSpec(1, 1, 64, 32, ffi.DT_BF16))
    f, taken = g.fuse_linear_blocks()
    assert taken == 0 and f.digest() == g.digest()


def test_graph_pass_keeps_a_norm_that_something_else_reads():
    bf16, r, h, n = ffi.DT_BF16, 1, 4096, 256
    inv, const, outl = ffi.LIFETIME_INVOCATION, ffi.LIFETIME_CONSTANT, ffi.LIFETIME_OUTPUT
    rd = vb.value_contract(bf16, [r, h], inv)
    g = vb.ProgramGraph()
    x = g.add_external_value("x", rd)
    nw = g.add_external_value("nw", vb.value_contract(bf16, [h], const))
    w = g.add_external_value("w", vb.value_contract(ffi.DT_U32, [n, h // 8], const))
    s = g.add_external_value("s", vb.value_contract(bf16, [n, h // 128], const))
    _, (normed,) = g.add_node("norm", vb.learned_rms_norm("input", "weight", "output", r, h, 1e-6, bf16),
                              [("input", x, rd), ("weight", nw, vb.value_contract(bf16, [h], const))],
                              [("output", "normed", vb.value_contract(bf16, [r, h], inv, ffi.ACCESS_READ_WRITE))])
    g.add_node("proj", vb.linear_int4_grouped_rowmajor("input", "weight", "scale", "output", r, h, n, 128),
               [("input", normed, rd), ("weight", w, vb.value_contract(ffi.DT_U32, [n, h // 8], const)),
                ("scale", s, vb.value_contract(bf16, [n, h // 128], const))],
               [("output", "y", vb.value_contract(bf16, [r, n], outl, ffi.ACCESS_READ_WRITE))])
    g.add_node("other", vb.residual_add_typed("residual", "branch", "output", r * h, bf16),
               [("residual", x, rd), ("branch", normed, rd)],
               [("output", "z", vb.value_contract(bf16, [r, h], outl, ffi.ACCESS_READ_WRITE))])
    f, taken = g.fuse_linear_blocks()
    assert taken == 0 and f.digest() == g.digest()
