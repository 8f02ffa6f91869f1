// ProgramGraph: executable Programs connected by typed values (vyre-foundation/src/ir_inner/model/program_graph.rs:20-648).
// Construction order is the topological schedule; every port is checked against the Program's buffer declaration
// (element type, element count, access) and against the value it connects to (dtype, shape, lifetime), names are unique
// over nodes and values, a buffer or a value is bound once per node, retained successors must consume and preserve the
// value they replace. Only statically known dimensions exist here (the reference's ShapeDim::Symbol is not rebuilt).
// The graph is host metadata: the runtime walks its schedule and submits one materialised Program per node.
#include <algorithm>
#include <cstring>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "blake3.hpp"
#include "model.hpp"

namespace vyb {
namespace {

struct Contract {
    uint32_t dtype = 0, access = 0, lifetime = 0;
    std::vector<uint64_t> shape;
    bool operator==(const Contract& o) const { return dtype == o.dtype && access == o.access && lifetime == o.lifetime && shape == o.shape; }
};

struct Input {
    std::string buffer;
    uint32_t value = 0;
    Contract contract;
};
struct Output {
    std::string buffer, name;
    Contract contract;
    int64_t retained_successor_of = -1;
    uint32_t value = 0;
};
struct Node {
    std::string name;
    vyb_program program;
    std::vector<Input> inputs;
    std::vector<Output> outputs;
};
struct Value {
    std::string name;
    Contract contract;
    int64_t producer = -1;
    std::vector<uint32_t> consumers;
    int64_t retained_successor_of = -1;
};

Contract from_c(const vyb_value_contract& c) {
    Contract r;
    r.dtype = c.dtype;
    r.access = c.access;
    r.lifetime = c.lifetime;
    r.shape.assign(c.shape, c.shape + std::min<uint32_t>(c.rank, 6));
    return r;
}
void to_c(const Contract& c, vyb_value_contract* out) {
    *out = vyb_value_contract{};
    out->dtype = c.dtype;
    out->access = c.access;
    out->lifetime = c.lifetime;
    out->rank = uint32_t(c.shape.size());
    std::copy(c.shape.begin(), c.shape.end(), out->shape);
}

const char* access_name(uint32_t a) {
    switch (a) {
        case VYB_ACCESS_READ_ONLY: return "ReadOnly";
        case VYB_ACCESS_READ_WRITE: return "ReadWrite";
        case VYB_ACCESS_OUTPUT: return "ReadWrite (output)";
        case VYB_ACCESS_WORKGROUP: return "Workgroup";
        default: return "?";
    }
}

int32_t graph_error(const std::string& what) { return fail_invalid_program("Fix: " + what); }

// program_graph.rs:541-634. A declared output buffer is a ReadWrite buffer with the output flag; the reference's WriteOnly
// and Uniform accesses do not occur in this operator set.
int32_t validate_buffer(const std::string& node, const Program& program, const std::string& buffer_name, const Contract& contract,
                        bool output_role) {
    const BufferDecl* buffer = nullptr;
    for (const BufferDecl& b : program.buffers)
        if (b.name == buffer_name) buffer = &b;
    if (!buffer) return graph_error("program node `" + node + "` has no buffer `" + buffer_name + "`");
    auto disagree = [&](const std::string& reason) {
        return graph_error("program node `" + node + "` buffer `" + buffer_name + "` disagrees with its value contract: " + reason);
    };
    if (buffer->dtype != contract.dtype)
        return disagree("Program uses dtype tag " + std::to_string(buffer->dtype) + ", graph uses " + std::to_string(contract.dtype));
    uint64_t elements = 1;
    for (uint64_t extent : contract.shape) {
        if (extent && elements > UINT64_MAX / extent) return disagree("graph shape element count overflows u64; reduce or shard dimensions");
        elements *= extent;
    }
    // a padded output (launch-shape padding with a logical readback range) carries its logical element count
    uint64_t declared = buffer->count;
    if (buffer->has_output_byte_range) declared = (buffer->output_byte_end - buffer->output_byte_begin) / std::max(1u, dtype_size_bytes(buffer->dtype));
    if (declared != 0 && elements != declared)
        return disagree("Program declares " + std::to_string(declared) + " elements, graph shape requires " + std::to_string(elements));
    const bool program_rw = buffer->access == VYB_ACCESS_READ_WRITE || buffer->access == VYB_ACCESS_OUTPUT;
    bool satisfies = false;
    if (contract.access == VYB_ACCESS_READ_ONLY) satisfies = buffer->access == VYB_ACCESS_READ_ONLY || program_rw;
    if (contract.access == VYB_ACCESS_READ_WRITE) satisfies = program_rw;
    if (!satisfies)
        return disagree(std::string("Program access ") + access_name(buffer->access) + " does not satisfy graph access " + access_name(contract.access));
    const bool compatible = output_role ? program_rw : (buffer->access == VYB_ACCESS_READ_ONLY || program_rw);
    if (!compatible) return disagree(std::string(output_role ? "Output" : "Input") + " port cannot use " + access_name(buffer->access) + " access");
    return VYB_OK;
}

}  // namespace
}  // namespace vyb

using namespace vyb;

struct vyb_graph {
    std::vector<Node> nodes;
    std::vector<Value> values;
    std::set<std::string> names;
};

extern "C" {

int32_t vyb_graph_new(vyb_graph** graph) {
    if (!graph) return fail_invalid_program("Fix: pass an out-pointer for the graph.");
    *graph = new vyb_graph();
    return VYB_OK;
}
void vyb_graph_free(vyb_graph* g) { delete g; }

int32_t vyb_graph_add_external_value(vyb_graph* g, const char* name, const vyb_value_contract* contract, uint32_t* value_id) {
    if (!g || !name || !contract || !value_id) return fail_invalid_program("Fix: pass a graph, a value name, a contract and an out-pointer.");
    if (contract->rank > 6) return graph_error("a value contract holds at most six dimensions");
    if (g->names.count(name)) return graph_error(std::string("duplicate graph name `") + name + "`; use one stable identity per node or value");
    Value v;
    v.name = name;
    v.contract = from_c(*contract);
    g->names.insert(name);
    g->values.push_back(std::move(v));
    *value_id = uint32_t(g->values.size() - 1);
    return VYB_OK;
}

int32_t vyb_graph_add_node(vyb_graph* g, const char* name, const vyb_program* program, const vyb_graph_input* inputs, uint32_t n_inputs,
                           const vyb_graph_output* outputs, uint32_t n_outputs, uint32_t* node_id, uint32_t* output_value_ids) {
    if (!g || !name || !program || (n_inputs && !inputs) || (n_outputs && !outputs))
        return fail_invalid_program("Fix: pass a graph, a node name, a program and its port arrays.");
    if (program->p.trap) return graph_error(std::string("program node `") + name + "` is a trap program: " + program->p.trap_message);
    const std::string node = name;
    if (g->names.count(node)) return graph_error("duplicate graph name `" + node + "`; use one stable identity per node or value");
    std::set<std::string> new_names{node};
    for (uint32_t i = 0; i < n_outputs; ++i) {
        if (!outputs[i].name || !outputs[i].buffer) return fail_invalid_program("Fix: every output port needs a buffer and a value name.");
        if (outputs[i].contract.rank > 6) return graph_error("a value contract holds at most six dimensions");
        if (g->names.count(outputs[i].name) || !new_names.insert(outputs[i].name).second)
            return graph_error(std::string("duplicate graph name `") + outputs[i].name + "`; use one stable identity per node or value");
    }
    Node n;
    n.name = node;
    n.program.p = program->p;
    std::set<std::string> bound;
    std::set<uint32_t> bound_values;
    for (uint32_t i = 0; i < n_inputs; ++i) {
        if (!inputs[i].buffer) return fail_invalid_program("Fix: every input port needs a buffer name.");
        if (inputs[i].contract.rank > 6) return graph_error("a value contract holds at most six dimensions");
        Input in;
        in.buffer = inputs[i].buffer;
        in.value = inputs[i].value;
        in.contract = from_c(inputs[i].contract);
        if (!bound.insert(in.buffer).second) return graph_error("program node `" + node + "` binds buffer `" + in.buffer + "` more than once");
        if (!bound_values.insert(in.value).second)
            return graph_error("program node `" + node + "` binds graph value " + std::to_string(in.value) + " more than once");
        if (in.value >= g->values.size()) return graph_error("graph value " + std::to_string(in.value) + " does not exist");
        const Contract& actual = g->values[in.value].contract;
        if (actual.dtype != in.contract.dtype || actual.shape != in.contract.shape || actual.lifetime != in.contract.lifetime)
            return graph_error("program node `" + node + "` buffer `" + in.buffer + "` expects another dtype, shape or lifetime than graph value " +
                               std::to_string(in.value) + " (`" + g->values[in.value].name + "`) provides");
        if (int32_t rc = validate_buffer(node, n.program.p, in.buffer, in.contract, false)) return rc;
        n.inputs.push_back(std::move(in));
    }
    for (uint32_t i = 0; i < n_outputs; ++i) {
        Output o;
        o.buffer = outputs[i].buffer;
        o.name = outputs[i].name;
        o.contract = from_c(outputs[i].contract);
        o.retained_successor_of = outputs[i].retained_successor_of;
        bool retained_rebind = false;
        if (o.retained_successor_of >= 0) {
            const uint32_t prior = uint32_t(o.retained_successor_of);
            if (prior >= g->values.size()) return graph_error("graph value " + std::to_string(prior) + " does not exist");
            bool consumed = false;
            for (const Input& in : n.inputs) {
                consumed |= in.value == prior;
                retained_rebind |= in.value == prior && in.buffer == o.buffer;
            }
            if (!consumed)
                return graph_error("retained output `" + o.name + "` names value " + std::to_string(prior) + " without consuming that prior value");
            const Contract& pc = g->values[prior].contract;
            if (pc.lifetime != VYB_LIFETIME_RETAINED || o.contract.lifetime != VYB_LIFETIME_RETAINED || !(pc == o.contract))
                return graph_error("retained output `" + o.name + "` is not a type-preserving successor of value " + std::to_string(prior));
        }
        if (!bound.insert(o.buffer).second && !retained_rebind)
            return graph_error("program node `" + node + "` binds buffer `" + o.buffer + "` more than once");
        if (int32_t rc = validate_buffer(node, n.program.p, o.buffer, o.contract, true)) return rc;
        n.outputs.push_back(std::move(o));
    }
    // commit
    const uint32_t id = uint32_t(g->nodes.size());
    g->names.insert(node);
    for (const Input& in : n.inputs) g->values[in.value].consumers.push_back(id);
    for (uint32_t i = 0; i < n.outputs.size(); ++i) {
        Output& o = n.outputs[i];
        Value v;
        v.name = o.name;
        v.contract = o.contract;
        v.producer = id;
        v.retained_successor_of = o.retained_successor_of;
        g->names.insert(o.name);
        g->values.push_back(std::move(v));
        o.value = uint32_t(g->values.size() - 1);
        if (output_value_ids) output_value_ids[i] = o.value;
    }
    g->nodes.push_back(std::move(n));
    if (node_id) *node_id = id;
    clear_error();
    return VYB_OK;
}

// ProgramGraph::from_program (program_graph.rs:225-270): every host-visible buffer becomes an external value (read-only:
// Invocation, read-write: Retained) or, for outputs, a produced Output value; workgroup scratch stays inside the node.
int32_t vyb_graph_from_program(const char* node_name, const vyb_program* program, vyb_graph** graph) {
    if (!node_name || !program || !graph) return fail_invalid_program("Fix: pass a node name, a program and an out-pointer.");
    std::unique_ptr<vyb_graph> g(new vyb_graph());
    std::vector<vyb_graph_input> ins;
    std::vector<vyb_graph_output> outs;
    for (const BufferDecl& b : program->p.buffers) {
        if (b.access == VYB_ACCESS_WORKGROUP) continue;
        vyb_value_contract c{};
        c.dtype = b.dtype;
        c.rank = 1;
        c.shape[0] = b.has_output_byte_range ? (b.output_byte_end - b.output_byte_begin) / std::max(1u, dtype_size_bytes(b.dtype)) : b.count;
        if (b.access == VYB_ACCESS_OUTPUT) {
            c.access = VYB_ACCESS_READ_WRITE;
            c.lifetime = VYB_LIFETIME_OUTPUT;
            vyb_graph_output o{};
            o.buffer = b.name.c_str();
            o.name = b.name.c_str();
            o.contract = c;
            o.retained_successor_of = -1;
            outs.push_back(o);
        } else {
            c.access = b.access;
            c.lifetime = b.access == VYB_ACCESS_READ_WRITE ? VYB_LIFETIME_RETAINED : VYB_LIFETIME_INVOCATION;
            uint32_t id = 0;
            if (int32_t rc = vyb_graph_add_external_value(g.get(), b.name.c_str(), &c, &id)) return rc;
            vyb_graph_input in{};
            in.buffer = b.name.c_str();
            in.value = id;
            in.contract = c;
            ins.push_back(in);
        }
    }
    if (int32_t rc = vyb_graph_add_node(g.get(), node_name, program, ins.data(), uint32_t(ins.size()), outs.data(), uint32_t(outs.size()),
                                        nullptr, nullptr))
        return rc;
    *graph = g.release();
    return VYB_OK;
}

uint32_t vyb_graph_node_count(const vyb_graph* g) { return g ? uint32_t(g->nodes.size()) : 0; }
uint32_t vyb_graph_value_count(const vyb_graph* g) { return g ? uint32_t(g->values.size()) : 0; }

int32_t vyb_graph_value(const vyb_graph* g, uint32_t id, vyb_graph_value_info* out) {
    if (!g || !out || id >= g->values.size()) return graph_error("graph value " + std::to_string(id) + " does not exist");
    const Value& v = g->values[id];
    out->name = v.name.c_str();
    to_c(v.contract, &out->contract);
    out->producer = v.producer;
    out->n_consumers = uint32_t(v.consumers.size());
    out->retained_successor_of = v.retained_successor_of;
    // liveness_intervals (program_graph.rs:486-503): producer's schedule index (0 for external values) to the last consumer's
    out->live_start = v.producer < 0 ? 0u : uint32_t(v.producer);
    out->live_end = out->live_start;
    for (uint32_t c : v.consumers) out->live_end = std::max(out->live_end, c);
    return VYB_OK;
}

int32_t vyb_graph_node(const vyb_graph* g, uint32_t id, vyb_graph_node_info* out) {
    if (!g || !out || id >= g->nodes.size()) return graph_error("graph node " + std::to_string(id) + " does not exist");
    const Node& n = g->nodes[id];
    out->name = n.name.c_str();
    out->program = &n.program;
    out->n_inputs = uint32_t(n.inputs.size());
    out->n_outputs = uint32_t(n.outputs.size());
    return VYB_OK;
}

int32_t vyb_graph_node_input(const vyb_graph* g, uint32_t node, uint32_t index, vyb_graph_input* out) {
    if (!g || !out || node >= g->nodes.size() || index >= g->nodes[node].inputs.size()) return graph_error("no such input port");
    const Input& in = g->nodes[node].inputs[index];
    out->buffer = in.buffer.c_str();
    out->value = in.value;
    to_c(in.contract, &out->contract);
    return VYB_OK;
}

int32_t vyb_graph_node_output(const vyb_graph* g, uint32_t node, uint32_t index, vyb_graph_output* out, uint32_t* value_id) {
    if (!g || !out || node >= g->nodes.size() || index >= g->nodes[node].outputs.size()) return graph_error("no such output port");
    const Output& o = g->nodes[node].outputs[index];
    out->buffer = o.buffer.c_str();
    out->name = o.name.c_str();
    to_c(o.contract, &out->contract);
    out->retained_successor_of = o.retained_successor_of;
    if (value_id) *value_id = o.value;
    return VYB_OK;
}

// The residual block's projections with their neighbours taken in (dense_gated_mlp.rs:168-200: `mlp.norm` feeds gate_proj
// and up_proj, `mlp.residual` follows down_proj): a copy of the graph in which
//   * a bf16 learned RMSNorm node whose output is read only as the activation of int4 row-major linears (bf16 outputs) is
//     dropped, and each of those linears becomes a linear_int4_block node that reads the norm's input and weight itself;
//   * a bf16 SwiGLU node whose `up` is produced by such a linear, and read by nothing else, is dropped, and the linear becomes
//     (or stays) a linear_int4_block node that reads the gate and produces the SwiGLU's output value;
//   * a bf16 residual add whose `branch` is produced by such a linear, and read by nothing else, is dropped, and the linear
//     becomes (or stays) a linear_int4_block node that reads the residual and produces the add's output value.
// Every other node and value is carried over with its name, contract and order. Values of the fused graph equal those of
// the original (the block node rounds where the stand-alone operators round). `n_fused` counts the dropped nodes.
int32_t vyb_graph_fuse_linear_blocks(const vyb_graph* g, vyb_graph** fused, uint32_t* n_fused) {
    if (!g || !fused) return fail_invalid_program("Fix: pass a graph and an out-pointer for the fused graph.");
    const size_t nn = g->nodes.size();
    auto is_linear = [&](const Node& n) {
        if (n.program.p.kind != OpKind::LinearInt4GroupedRowmajor || n.program.p.params.u[4] != VYB_DT_BF16 || n.inputs.size() != 3 ||
            n.outputs.size() != 1)
            return false;
        for (const BufferDecl& b : n.program.p.buffers)
            if (b.name == "norm_weight" || b.name == "residual" || b.name == "gate") return false;  // the block node's added ports
        return true;
    };
    // only where the decode kernel takes the part into its own launch (the target compiler's rule for the block node)
    auto kernel_takes = [&](const Node& lin, uint32_t part) {
        Program probe = lin.program.p;
        probe.kind = OpKind::LinearInt4Block;
        probe.params.u[5] = part;
        return select_kernel_variant(probe) == KV_INT4_BLOCK_GEMV;
    };
    auto port_value = [](const Node& n, const std::string& buffer) -> int64_t {
        for (const Input& in : n.inputs)
            if (in.buffer == buffer) return in.value;
        return -1;
    };
    struct Plan {
        int64_t norm = -1;   // linear: the norm node taken into its prologue
        int64_t gate = -1;   // linear: the SwiGLU node taken into its stores
        int64_t resid = -1;  // linear: the residual-add node taken into its stores
        bool dropped = false;
    };
    std::vector<Plan> plan(nn);
    for (size_t i = 0; i < nn; ++i) {
        const Node& n = g->nodes[i];
        const Program& np = n.program.p;
        if (np.kind == OpKind::RmsNorm && np.params.u[5] == 0 && np.params.u[3] == VYB_DT_BF16 && np.params.u[4] == VYB_DT_BF16 &&
            n.inputs.size() == 2 && n.outputs.size() == 1) {
            const Value& out = g->values[n.outputs[0].value];
            bool ok = !out.consumers.empty() && out.contract.lifetime == VYB_LIFETIME_INVOCATION && out.retained_successor_of < 0;
            for (uint32_t c : out.consumers) {
                const Node& lin = g->nodes[c];
                ok = ok && is_linear(lin) && kernel_takes(lin, 1u) &&
                     port_value(lin, lin.program.p.buffers[0].name) == int64_t(n.outputs[0].value) &&
                     lin.program.p.params.u[0] == np.params.u[0] && lin.program.p.params.u[1] == np.params.u[1];
            }
            if (ok) {
                plan[i].dropped = true;
                for (uint32_t c : out.consumers) plan[c].norm = int64_t(i);
            }
        }
        if (np.kind == OpKind::Swiglu && np.params.u[1] == VYB_DT_BF16 && n.inputs.size() == 2 && n.outputs.size() == 1) {
            // buffers: gate, up, output (swiglu.rs:51-79)
            const int64_t gate = port_value(n, np.buffers[0].name), up = port_value(n, np.buffers[1].name);
            if (gate >= 0 && up >= 0) {
                const Value& uv = g->values[size_t(up)];
                const Value& gv = g->values[size_t(gate)];
                if (uv.producer >= 0 && uv.consumers.size() == 1 && uv.contract.lifetime == VYB_LIFETIME_INVOCATION &&
                    gv.producer < uv.producer) {  // the gate exists when the up projection runs
                    const size_t li = size_t(uv.producer);
                    const Node& lin = g->nodes[li];
                    if (is_linear(lin) && kernel_takes(lin, 4u) && plan[li].gate < 0 && plan[li].resid < 0 &&
                        uint64_t(lin.program.p.params.u[0]) * lin.program.p.params.u[2] == np.params.u[0]) {
                        plan[i].dropped = true;
                        plan[li].gate = int64_t(i);
                    }
                }
            }
        }
        if (np.kind == OpKind::ResidualAdd && np.params.u[1] == VYB_DT_BF16 && n.inputs.size() == 2 && n.outputs.size() == 1) {
            // buffers: residual, branch, output (residual_add.rs:8-52)
            const int64_t branch = port_value(n, np.buffers[1].name), residual = port_value(n, np.buffers[0].name);
            if (branch < 0 || residual < 0) continue;
            const Value& bv = g->values[size_t(branch)];
            if (bv.producer < 0 || bv.consumers.size() != 1 || bv.contract.lifetime != VYB_LIFETIME_INVOCATION) continue;
            const Node& lin = g->nodes[size_t(bv.producer)];
            if (!is_linear(lin) || !kernel_takes(lin, 2u) || plan[size_t(bv.producer)].resid >= 0 || plan[size_t(bv.producer)].gate >= 0)
                continue;
            if (uint64_t(lin.program.p.params.u[0]) * lin.program.p.params.u[2] != np.params.u[0]) continue;
            // the residual must exist when the linear runs
            const Value& rv = g->values[size_t(residual)];
            if (rv.producer >= bv.producer) continue;
            plan[i].dropped = true;
            plan[size_t(bv.producer)].resid = int64_t(i);
        }
    }
    std::unique_ptr<vyb_graph> out(new vyb_graph());
    // values and nodes are re-created in the order of the original (value ids are creation order: an external value when it
    // was declared, a node's outputs when the node was added), so that a graph with nothing to take in comes out identical
    std::vector<int64_t> remap(g->values.size(), -1);
    std::vector<bool> emitted(nn, false);
    uint32_t dropped = 0;
    auto emit_node = [&](size_t i) -> int32_t {
        emitted[i] = true;
        const Node& n = g->nodes[i];
        if (plan[i].dropped) {
            ++dropped;
            return VYB_OK;
        }
        std::vector<Input> ins = n.inputs;
        std::vector<Output> outs = n.outputs;
        vyb_program* built = nullptr;
        const vyb_program* program = &n.program;
        if (plan[i].norm >= 0 || plan[i].resid >= 0 || plan[i].gate >= 0) {
            const Program& lp = n.program.p;
            const Node* swi = plan[i].gate >= 0 ? &g->nodes[size_t(plan[i].gate)] : nullptr;
            const Node* norm = plan[i].norm >= 0 ? &g->nodes[size_t(plan[i].norm)] : nullptr;
            const Node* add = plan[i].resid >= 0 ? &g->nodes[size_t(plan[i].resid)] : nullptr;
            float eps = 0.0f;
            if (norm) std::memcpy(&eps, &norm->program.p.params.u[2], 4);
            if (int32_t rc = vyb_nn_linear_int4_block(lp.buffers[0].name.c_str(), norm ? "norm_weight" : nullptr, lp.buffers[1].name.c_str(),
                                                      lp.buffers[2].name.c_str(), swi ? "gate" : nullptr, add ? "residual" : nullptr,
                                                      lp.buffers[3].name.c_str(),
                                                      lp.params.u[0], lp.params.u[1], lp.params.u[2], lp.params.u[3], eps, &built))
                return rc;
            program = built;
            if (norm) {
                // the activation port now reads what the norm read; the norm's weight becomes a port of this node
                const Program& np = norm->program.p;
                for (Input& in : ins)
                    if (in.buffer == lp.buffers[0].name)
                        for (const Input& ni : norm->inputs)
                            if (ni.buffer == np.buffers[0].name) {
                                in.value = ni.value;
                                in.contract = ni.contract;
                            }
                for (const Input& ni : norm->inputs)
                    if (ni.buffer == np.buffers[1].name) {
                        Input w = ni;
                        w.buffer = "norm_weight";
                        ins.push_back(w);
                    }
            }
            if (swi) {
                // the gate becomes a port of this node, which now produces the SwiGLU's output value
                const Program& sp = swi->program.p;
                for (const Input& si : swi->inputs)
                    if (si.buffer == sp.buffers[0].name) {
                        Input gi = si;
                        gi.buffer = "gate";
                        ins.push_back(gi);
                    }
                outs[0].name = swi->outputs[0].name;
                outs[0].contract = swi->outputs[0].contract;
                outs[0].retained_successor_of = -1;
            }
            if (add) {
                const Program& ap = add->program.p;
                for (const Input& ai : add->inputs)
                    if (ai.buffer == ap.buffers[0].name) {
                        Input r = ai;
                        r.buffer = "residual";
                        ins.push_back(r);
                    }
                outs[0].name = add->outputs[0].name;
                outs[0].contract = add->outputs[0].contract;
                outs[0].retained_successor_of = -1;
            }
        }
        std::vector<vyb_graph_input> cin(ins.size());
        std::vector<vyb_graph_output> cout(outs.size());
        for (size_t k = 0; k < ins.size(); ++k) {
            cin[k].buffer = ins[k].buffer.c_str();
            cin[k].value = uint32_t(remap[ins[k].value]);
            to_c(ins[k].contract, &cin[k].contract);
        }
        for (size_t k = 0; k < outs.size(); ++k) {
            cout[k].buffer = outs[k].buffer.c_str();
            cout[k].name = outs[k].name.c_str();
            to_c(outs[k].contract, &cout[k].contract);
            cout[k].retained_successor_of = outs[k].retained_successor_of < 0 ? -1 : remap[size_t(outs[k].retained_successor_of)];
        }
        std::vector<uint32_t> ids(std::max<size_t>(1, outs.size()));
        const int32_t rc = vyb_graph_add_node(out.get(), n.name.c_str(), program, cin.data(), uint32_t(cin.size()), cout.data(),
                                              uint32_t(cout.size()), nullptr, ids.data());
        if (built) vyb_program_free(built);
        if (rc) return rc;
        // the values this node produced in the original graph (and, with the add taken in, the add's output) map to the new ones
        for (size_t k = 0; k < n.outputs.size(); ++k) remap[n.outputs[k].value] = ids[k];
        if (plan[i].resid >= 0) remap[g->nodes[size_t(plan[i].resid)].outputs[0].value] = ids[0];
        if (plan[i].gate >= 0) remap[g->nodes[size_t(plan[i].gate)].outputs[0].value] = ids[0];
        return VYB_OK;
    };
    for (size_t v = 0; v < g->values.size(); ++v) {
        const Value& val = g->values[v];
        if (val.producer >= 0) {
            if (!emitted[size_t(val.producer)])
                if (int32_t rc = emit_node(size_t(val.producer))) return rc;
            continue;
        }
        vyb_value_contract c;
        to_c(val.contract, &c);
        uint32_t id = 0;
        if (int32_t rc = vyb_graph_add_external_value(out.get(), val.name.c_str(), &c, &id)) return rc;
        remap[v] = id;
    }
    for (size_t i = 0; i < nn; ++i)  // nodes without outputs
        if (!emitted[i])
            if (int32_t rc = emit_node(i)) return rc;
    if (n_fused) *n_fused = dropped;
    *fused = out.release();
    clear_error();
    return VYB_OK;
}

// identity of the whole graph: blake3 over names, contracts, wiring and every node's program fingerprint, in schedule order
void vyb_graph_digest(const vyb_graph* g, uint8_t out[32]) {
    std::vector<uint8_t> v = {'V', 'Y', 'B', 'G'};
    auto put_u64 = [&](uint64_t x) {
        for (int i = 0; i < 8; ++i) v.push_back(uint8_t(x >> (8 * i)));
    };
    auto put_str = [&](const std::string& s) {
        put_u64(s.size());
        v.insert(v.end(), s.begin(), s.end());
    };
    auto put_contract = [&](const Contract& c) {
        put_u64(c.dtype);
        put_u64(c.access);
        put_u64(c.lifetime);
        put_u64(c.shape.size());
        for (uint64_t d : c.shape) put_u64(d);
    };
    if (g) {
        put_u64(g->values.size());
        for (const Value& val : g->values) {
            put_str(val.name);
            put_contract(val.contract);
            put_u64(uint64_t(val.producer));
            put_u64(uint64_t(val.retained_successor_of));
        }
        put_u64(g->nodes.size());
        for (const Node& n : g->nodes) {
            put_str(n.name);
            Digest fp = n.program.p.fingerprint();
            v.insert(v.end(), fp.begin(), fp.end());
            put_u64(n.inputs.size());
            for (const Input& in : n.inputs) {
                put_str(in.buffer);
                put_u64(in.value);
                put_contract(in.contract);
            }
            put_u64(n.outputs.size());
            for (const Output& o : n.outputs) {
                put_str(o.buffer);
                put_u64(o.value);
            }
        }
    }
    blake3(v.data(), v.size(), out);
}

}  // extern "C"
