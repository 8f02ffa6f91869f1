// Operator surface: one builder per reference builder, same argument order, same validation and the same
// "Fix: ..." texts. A Program here is the reference Program's observable shape (buffers, workgroup size,
// op region id) plus the op parameters the native facet dispatches on.
#include <limits>
#include <mutex>

#include "blake3.hpp"
#include "model.hpp"

namespace vyb {

namespace {
thread_local std::string g_last_error;
}

int32_t fail(int32_t code, const std::string& message) {
    g_last_error = message;
    return code;
}
void clear_error() { g_last_error.clear(); }
int32_t fail_invalid_program(const std::string& fix) { return fail(VYB_ERR_INVALID_PROGRAM, fix); }
int32_t fail_unsupported(const std::string& name) {
    return fail(VYB_ERR_UNSUPPORTED_FEATURE,
                "unsupported feature `" + name + "` on backend `" + BACKEND_ID +
                    "`. Fix: check backend capability before using this feature, or select a backend that supports it.");
}
int32_t fail_dispatch(int32_t cuda_code, const std::string& message) {
    return fail(VYB_ERR_DISPATCH_FAILED,
                "dispatch failed (code Some(" + std::to_string(cuda_code) + ")): " + message +
                    ". Fix: inspect the backend error code and queue state, reduce dispatch pressure, or reacquire the "
                    "backend before retrying.");
}
int32_t fail_oom(uint64_t requested, uint64_t available) {
    return fail(VYB_ERR_DEVICE_OUT_OF_MEMORY,
                "device out of memory: requested " + std::to_string(requested) + " bytes, " +
                    std::to_string(available) +
                    " available. Fix: reduce buffer sizes or split the dispatch into smaller chunks.");
}
int32_t fail_device_lost(const std::string& device, uint64_t generation, const std::string& message) {
    return fail(VYB_ERR_DEVICE_LOST,
                "device generation " + std::to_string(generation) + " was lost on backend `" + BACKEND_ID +
                    "` device `" + device + "`: " + message +
                    ". Fix: reacquire the registered materializer and rematerialize the authenticated artifact before "
                    "retrying.");
}

uint32_t dtype_size_bytes(uint32_t dtype) {
    switch (dtype) {
        case VYB_DT_U32:
        case VYB_DT_I32:
        case VYB_DT_F32: return 4;
        case VYB_DT_F16:
        case VYB_DT_BF16: return 2;
        case VYB_DT_U8:
        case VYB_DT_I8: return 1;
        default: return 4;
    }
}

// ---- wire -------------------------------------------------------------------------------------------
namespace {
void put_u32(std::vector<uint8_t>& v, uint32_t x) {
    for (int i = 0; i < 4; ++i) v.push_back(uint8_t(x >> (8 * i)));
}
void put_u64(std::vector<uint8_t>& v, uint64_t x) {
    for (int i = 0; i < 8; ++i) v.push_back(uint8_t(x >> (8 * i)));
}
void put_str(std::vector<uint8_t>& v, const std::string& s) {
    put_u32(v, uint32_t(s.size()));
    v.insert(v.end(), s.begin(), s.end());
}
struct Reader {
    const uint8_t* p;
    size_t n, off = 0;
    bool ok = true;
    uint32_t u32() {
        if (off + 4 > n) { ok = false; return 0; }
        uint32_t x = 0;
        for (int i = 0; i < 4; ++i) x |= uint32_t(p[off + i]) << (8 * i);
        off += 4;
        return x;
    }
    uint64_t u64() {
        uint64_t lo = u32();
        uint64_t hi = u32();
        return lo | (hi << 32);
    }
    std::string str() {
        uint32_t len = u32();
        if (!ok || off + len > n) { ok = false; return {}; }
        std::string s(reinterpret_cast<const char*>(p + off), len);
        off += len;
        return s;
    }
};
}  // namespace

std::vector<uint8_t> Program::to_wire() const {
    std::vector<uint8_t> v = {'V', 'Y', 'B', 'P'};
    put_u32(v, 1);
    put_str(v, op_id);
    put_u32(v, uint32_t(kind));
    for (uint32_t w : workgroup) put_u32(v, w);
    put_u32(v, trap ? 1 : 0);
    put_str(v, trap_message);
    for (uint32_t x : params.u) put_u32(v, x);
    put_u32(v, uint32_t(buffers.size()));
    for (const BufferDecl& b : buffers) {
        put_str(v, b.name);
        put_u32(v, b.binding);
        put_u32(v, b.access);
        put_u32(v, b.dtype);
        put_u32(v, b.count);
        put_u32(v, b.has_output_byte_range ? 1 : 0);
        put_u64(v, b.output_byte_begin);
        put_u64(v, b.output_byte_end);
    }
    return v;
}

bool Program::from_wire(const uint8_t* bytes, size_t len, Program* out, std::string* error) {
    if (len < 8 || std::memcmp(bytes, "VYBP", 4) != 0) {
        *error = "program wire does not start with the VYBP magic";
        return false;
    }
    Reader r{bytes, len, 4};
    if (r.u32() != 1) {
        *error = "unknown program wire version";
        return false;
    }
    Program p;
    p.op_id = r.str();
    p.kind = OpKind(r.u32());
    for (auto& w : p.workgroup) w = r.u32();
    p.trap = r.u32() != 0;
    p.trap_message = r.str();
    for (auto& x : p.params.u) x = r.u32();
    uint32_t nb = r.u32();
    if (!r.ok || nb > 64) {
        *error = "program wire is truncated";
        return false;
    }
    for (uint32_t i = 0; i < nb; ++i) {
        BufferDecl b;
        b.name = r.str();
        b.binding = r.u32();
        b.access = r.u32();
        b.dtype = r.u32();
        b.count = r.u32();
        b.has_output_byte_range = r.u32() != 0;
        b.output_byte_begin = r.u64();
        b.output_byte_end = r.u64();
        p.buffers.push_back(std::move(b));
    }
    if (!r.ok || r.off != len) {
        *error = "program wire is truncated or has trailing bytes";
        return false;
    }
    *out = std::move(p);
    return true;
}

Digest Program::fingerprint() const {
    std::vector<uint8_t> w = to_wire();
    Digest d;
    blake3(w.data(), w.size(), d.data());
    return d;
}

const BufferDecl* Program::buffer_by_binding(uint32_t binding) const {
    for (const BufferDecl& b : buffers)
        if (b.access != VYB_ACCESS_WORKGROUP && b.binding == binding) return &b;
    return nullptr;
}

namespace {

BufferDecl storage(const char* name, uint32_t binding, uint32_t access, uint32_t dtype, uint32_t count) {
    BufferDecl b;
    b.name = name ? name : "";
    b.binding = binding;
    b.access = access;
    b.dtype = dtype;
    b.count = count;
    return b;
}
BufferDecl output(const char* name, uint32_t binding, uint32_t dtype, uint32_t count) {
    return storage(name, binding, VYB_ACCESS_OUTPUT, dtype, count);
}
BufferDecl workgroup(const char* name, uint32_t count, uint32_t dtype) {
    BufferDecl b = storage(name, 0, VYB_ACCESS_WORKGROUP, dtype, count);
    return b;
}

bool checked_mul(uint32_t a, uint32_t b, uint32_t* out) {
    uint64_t r = uint64_t(a) * uint64_t(b);
    if (r > std::numeric_limits<uint32_t>::max()) return false;
    *out = uint32_t(r);
    return true;
}
uint32_t div_ceil(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

int32_t emit(vyb_program** out, Program&& p) {
    if (!out) return fail_invalid_program("Fix: pass a non-null program out-pointer.");
    auto* h = new vyb_program();
    h->p = std::move(p);
    *out = h;
    clear_error();
    return VYB_OK;
}

// vyre-primitives/src/lib.rs:83-98 invalid_output_program: one output word, body = trap.
Program trap_program(const char* op_id, const char* out_name, uint32_t dtype, const std::string& message) {
    Program p;
    p.op_id = op_id;
    p.kind = OpKind::I4Unpack;
    p.workgroup = {1, 1, 1};
    p.buffers.push_back(output(out_name, 0, dtype, 1));
    p.trap = true;
    p.trap_message = message;
    return p;
}

bool names_ok(std::initializer_list<const char*> names) {
    for (const char* n : names)
        if (!n) return false;
    return true;
}
#define VYB_REQUIRE_NAMES(...) \
    if (!names_ok({__VA_ARGS__})) return fail_invalid_program("Fix: every buffer name must be a non-null string.")

}  // namespace
}  // namespace vyb

using namespace vyb;

extern "C" {

uint32_t vyb_abi_version(void) { return VYB_ABI_VERSION; }
const char* vyb_last_error_message(void) { return g_last_error.c_str(); }
uint32_t vyb_i4_packed_words(uint32_t lane_count) { return (lane_count + 7) / 8; }
void vyb_blake3(const void* data, size_t len, uint8_t out[32]) { blake3(data, len, out); }

// ---- linear_4bit (linear_4bit.rs:255-335) ---------------------------------------------------------------
int32_t vyb_nn_linear_4bit(const char* x, const char* w_packed, const char* b, const char* out, uint32_t in_dim,
                           uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, b, out);
    if (in_dim == 0) return fail_invalid_program("Fix: linear_4bit in_dim=0 is invalid: empty reduction");
    if (out_dim == 0) return fail_invalid_program("Fix: linear_4bit out_dim=0 is invalid: empty output");
    if (in_dim % 8 != 0)
        return fail_invalid_program("Fix: linear_4bit in_dim=" + std::to_string(in_dim) +
                                    " is not divisible by 8; pad weights to a multiple of 8.");
    uint32_t total;
    if (!checked_mul(in_dim / 8, out_dim, &total))
        return fail_invalid_program("Fix: linear_4bit in_dim/8 * out_dim overflows u32; reduce dimensions.");
    Program p;
    p.op_id = "vyre-libs::nn::linear_4bit";
    p.kind = OpKind::Linear4Bit;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = in_dim;
    p.params.u[1] = out_dim;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, in_dim),
                 storage(w_packed, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, total),
                 storage(b, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, out_dim), output(out, 3, VYB_DT_F32, out_dim)};
    return emit(program, std::move(p));
}

// ---- linear_4bit_affine_grouped[_batched] (linear_4bit.rs:399-775, weight-reuse variant :778-997) --------
int32_t vyb_nn_linear_4bit_affine_grouped_batched(const char* x, const char* w_packed, const char* scale,
                                                  const char* zero_point, const char* b, const char* out,
                                                  uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                                  uint32_t batch_size, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, scale, zero_point, b, out);
    if (in_dim == 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped in_dim=0 is invalid: empty reduction");
    if (out_dim == 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped out_dim=0 is invalid: empty output");
    if (group_size == 0)
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped group_size=0 is invalid: group size must be > 0");
    if (batch_size == 0)
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped batch_size=0 is invalid: batch size must be > 0");
    uint32_t input_count, logical_out, total, sidecar;
    if (!checked_mul(in_dim, batch_size, &input_count))
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped in_dim*batch_size overflows u32; reduce dimensions.");
    if (!checked_mul(out_dim, batch_size, &logical_out))
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped out_dim*batch_size overflows u32; reduce dimensions.");
    if (in_dim % 8 != 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped in_dim=" + std::to_string(in_dim) +
                                    " is not divisible by 8; pad weights to a multiple of 8.");
    if (!checked_mul(in_dim / 8, out_dim, &total))
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped in_dim/8 * out_dim overflows u32; reduce dimensions.");
    uint32_t group_count = div_ceil(in_dim, group_size);
    if (!checked_mul(group_count, out_dim, &sidecar))
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped group_count*out_dim overflows u32; reduce dimensions.");
    // launch-shape padding of the output: 8 outputs (warps) per 256-thread workgroup (linear_4bit.rs:743-771);
    // the weight-reuse variant uses (batch/8)*out_dim workgroups (linear_4bit.rs:456-479,793-811).
    bool shadows_tile = false;
    for (const char* name : {x, w_packed, scale, zero_point, b, out})
        if (std::strcmp(name, "linear_4bit_weight_tile") == 0) shadows_tile = true;
    const bool reuse = batch_size >= 8 && batch_size % 8 == 0 && in_dim == 256 && group_size >= 32 &&
                       group_size % 32 == 0 && !shadows_tile;
    uint32_t workgroups, padded;
    if (reuse) {
        if (!checked_mul(batch_size / 8, out_dim, &workgroups))
            return fail_invalid_program(
                "Fix: linear_4bit_affine_grouped batched output workgroups overflow u32; reduce dimensions.");
        if (!checked_mul(workgroups, 256, &padded))
            return fail_invalid_program(
                "Fix: linear_4bit_affine_grouped batched padded output count overflows u32; reduce dimensions.");
    } else {
        workgroups = div_ceil(logical_out, 8);
        if (!checked_mul(workgroups, 256, &padded))
            return fail_invalid_program(
                "Fix: linear_4bit_affine_grouped output workgroups overflow u32; reduce dimensions.");
    }
    Program p;
    p.op_id = "vyre-libs::nn::linear_4bit_affine_grouped";
    p.kind = OpKind::Linear4BitAffineGrouped;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = in_dim;
    p.params.u[1] = out_dim;
    p.params.u[2] = group_size;
    p.params.u[3] = batch_size;
    p.params.u[4] = reuse ? 1 : 0;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, input_count),
                 storage(w_packed, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, total),
                 storage(scale, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, sidecar),
                 storage(zero_point, 3, VYB_ACCESS_READ_ONLY, VYB_DT_U32, sidecar),
                 storage(b, 4, VYB_ACCESS_READ_ONLY, VYB_DT_F32, out_dim)};
    if (reuse) p.buffers.push_back(workgroup("linear_4bit_weight_tile", in_dim, VYB_DT_F32));
    BufferDecl o = output(out, 5, VYB_DT_F32, padded);
    o.has_output_byte_range = true;
    o.output_byte_begin = 0;
    o.output_byte_end = uint64_t(logical_out) * 4;
    p.buffers.push_back(o);
    return emit(program, std::move(p));
}

int32_t vyb_nn_linear_4bit_affine_grouped(const char* x, const char* w_packed, const char* scale,
                                          const char* zero_point, const char* b, const char* out, uint32_t in_dim,
                                          uint32_t out_dim, uint32_t group_size, vyb_program** program) {
    return vyb_nn_linear_4bit_affine_grouped_batched(x, w_packed, scale, zero_point, b, out, in_dim, out_dim,
                                                     group_size, 1, program);
}

void vyb_quantized_linear_4bit_spec_affine_grouped(uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                                   vyb_quantized_linear_4bit_spec* spec) {
    if (!spec) return;
    spec->in_dim = in_dim;
    spec->out_dim = out_dim;
    spec->storage_dtype = VYB_DT_I4;
    spec->scale_group_size = group_size;
    spec->zero_point_group_size = group_size;
}

// QuantizedLinear4BitSpec::affine_group_size (linear_4bit.rs:104-134)
static int32_t spec_group_size(const vyb_quantized_linear_4bit_spec* spec, uint32_t* group) {
    if (!spec) return fail_invalid_program("Fix: pass a non-null QuantizedLinear4BitSpec.");
    if (spec->storage_dtype != VYB_DT_I4)
        return fail_invalid_program("Fix: grouped INT4 linear requires DataType::Quantized storage I4, got tag " +
                                    std::to_string(spec->storage_dtype) + ".");
    if (spec->scale_group_size != spec->zero_point_group_size)
        return fail_invalid_program(
            "Fix: grouped INT4 linear requires scale and zero-point group sizes to match, got scale=" +
            std::to_string(spec->scale_group_size) + ", zero_point=" + std::to_string(spec->zero_point_group_size) +
            ".");
    if (spec->scale_group_size == 0)
        return fail_invalid_program("Fix: grouped INT4 linear requires quantized group_size > 0.");
    *group = spec->scale_group_size;
    return VYB_OK;
}

int32_t vyb_nn_linear_4bit_affine_grouped_typed(const vyb_quantized_linear_4bit_spec* spec, const char* x,
                                                const char* w_packed, const char* scale, const char* zero_point,
                                                const char* b, const char* out, vyb_program** program) {
    uint32_t g = 0;
    if (int32_t rc = spec_group_size(spec, &g)) return rc;
    return vyb_nn_linear_4bit_affine_grouped(x, w_packed, scale, zero_point, b, out, spec->in_dim, spec->out_dim, g,
                                             program);
}

int32_t vyb_nn_linear_4bit_affine_grouped_batched_typed(const vyb_quantized_linear_4bit_spec* spec,
                                                        uint32_t batch_size, const char* x, const char* w_packed,
                                                        const char* scale, const char* zero_point, const char* b,
                                                        const char* out, vyb_program** program) {
    uint32_t g = 0;
    if (int32_t rc = spec_group_size(spec, &g)) return rc;
    return vyb_nn_linear_4bit_affine_grouped_batched(x, w_packed, scale, zero_point, b, out, spec->in_dim,
                                                     spec->out_dim, g, batch_size, program);
}

// linear_4bit.rs:147-223
int32_t vyb_nn_linear_4bit_affine_grouped_planner_evidence(const vyb_quantized_linear_4bit_spec* spec,
                                                           vyb_planner_evidence* out) {
    uint32_t g = 0;
    if (int32_t rc = spec_group_size(spec, &g)) return rc;
    if (!out) return fail_invalid_program("Fix: pass a non-null planner evidence out-pointer.");
    const uint32_t in_dim = spec->in_dim, out_dim = spec->out_dim;
    if (in_dim == 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped planner evidence requires in_dim > 0.");
    if (out_dim == 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped planner evidence requires out_dim > 0.");
    if (in_dim % 8 != 0)
        return fail_invalid_program("Fix: linear_4bit_affine_grouped planner evidence in_dim=" +
                                    std::to_string(in_dim) + " is not divisible by 8.");
    uint32_t packed_words, sidecars;
    if (!checked_mul(in_dim / 8, out_dim, &packed_words))
        return fail_invalid_program(
            "Fix: linear_4bit_affine_grouped planner evidence packed weights overflow u32.");
    uint32_t group_count = div_ceil(in_dim, g);
    if (!checked_mul(group_count, out_dim, &sidecars))
        return fail_invalid_program("Fix: linear_4bit_affine_grouped planner evidence sidecars overflow u32.");
    *out = vyb_planner_evidence{};
    out->in_dim = in_dim;
    out->out_dim = out_dim;
    out->group_size = g;
    out->group_count = group_count;
    out->packed_weight_bytes = uint64_t(packed_words) * 4;
    out->dequantized_weight_bytes = uint64_t(in_dim) * out_dim * 4;
    out->sidecar_bytes = uint64_t(sidecars) * 8;
    out->bias_bytes = uint64_t(out_dim) * 4;
    out->output_bytes = uint64_t(out_dim) * 4;
    out->dequant_bytes_elided = out->dequantized_weight_bytes;
    out->matmul_m = out_dim;
    out->matmul_k = in_dim;
    out->matmul_n = 1;
    out->matmul_tile = 32;
    // The reference plans this op as strict f32 (F32MatmulMode::StrictF32), hence "cooperative".
    out->matmul_selected_path = "cooperative";
    out->matmul_candidate_path = nullptr;
    out->matmul_fallback_reason = "strict_f32_requested";
    out->tensor_core_eligible = 0;
    out->output_drift_abs_tolerance = 1.0e-4f;
    clear_error();
    return VYB_OK;
}

// ---- packed INT4 primitives (programs.rs) -----------------------------------------------------------------
int32_t vyb_math_unpack_i4x8(const char* packed_words, const char* out_lanes, uint32_t lane_count,
                             vyb_program** program) {
    VYB_REQUIRE_NAMES(packed_words, out_lanes);
    const char* id = "vyre-primitives::math::quantized::unpack_i4x8";
    if (lane_count == 0)
        return emit(program, trap_program(id, out_lanes, VYB_DT_I32, "Fix: unpack_i4x8 requires lane_count > 0."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::I4Unpack;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = lane_count;
    p.buffers = {storage(packed_words, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, vyb_i4_packed_words(lane_count)),
                 storage(out_lanes, 1, VYB_ACCESS_READ_WRITE, VYB_DT_I32, lane_count)};
    return emit(program, std::move(p));
}

int32_t vyb_math_i4x8_dot_i32(const char* lhs, const char* rhs, const char* out, uint32_t lane_count,
                              uint32_t lib_op_id, vyb_program** program) {
    VYB_REQUIRE_NAMES(lhs, rhs, out);
    const char* id = lib_op_id ? "vyre-libs::quant::int4_dot_i32" : "vyre-primitives::math::quantized::i4x8_dot_i32";
    if (lane_count == 0)
        return emit(program, trap_program(id, out, VYB_DT_I32, "Fix: i4x8_dot_i32 requires lane_count > 0."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::I4DotI32;
    p.params.u[0] = lane_count;
    uint32_t words = vyb_i4_packed_words(lane_count);
    p.buffers = {storage(lhs, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, words),
                 storage(rhs, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, words), output(out, 2, VYB_DT_I32, 1)};
    return emit(program, std::move(p));
}

int32_t vyb_math_i4x8_dot_f32_scaled(const char* lhs, const char* rhs, const char* lhs_scale, const char* rhs_scale,
                                     const char* out, uint32_t lane_count, uint32_t lib_op_id,
                                     vyb_program** program) {
    VYB_REQUIRE_NAMES(lhs, rhs, lhs_scale, rhs_scale, out);
    const char* id = lib_op_id ? "vyre-libs::quant::int4_dot_f32_scaled"
                               : "vyre-primitives::math::quantized::i4x8_dot_f32_scaled";
    if (lane_count == 0)
        return emit(program, trap_program(id, out, VYB_DT_F32, "Fix: i4x8_dot_f32_scaled requires lane_count > 0."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::I4DotF32Scaled;
    p.params.u[0] = lane_count;
    uint32_t words = vyb_i4_packed_words(lane_count);
    p.buffers = {storage(lhs, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, words),
                 storage(rhs, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, words),
                 storage(lhs_scale, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, 1),
                 storage(rhs_scale, 3, VYB_ACCESS_READ_ONLY, VYB_DT_F32, 1), output(out, 4, VYB_DT_F32, 1)};
    return emit(program, std::move(p));
}

int32_t vyb_math_i4x8_batched_matvec_f32_scaled(const char* weights, const char* x, const char* row_scales,
                                                const char* out, uint32_t batch, uint32_t rows, uint32_t cols,
                                                uint32_t lib_op_id, vyb_program** program) {
    VYB_REQUIRE_NAMES(weights, x, row_scales, out);
    const char* id = lib_op_id ? "vyre-libs::quant::int4_batched_matvec_f32_scaled"
                               : "vyre-primitives::math::quantized::i4x8_batched_matvec_f32_scaled";
    if (batch == 0 || rows == 0 || cols == 0)
        return emit(program,
                    trap_program(id, out, VYB_DT_F32,
                                 "Fix: i4x8_batched_matvec_f32_scaled requires batch > 0, rows > 0, and cols > 0."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::I4BatchedMatvec;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = batch;
    p.params.u[1] = rows;
    p.params.u[2] = cols;
    uint32_t wpr = vyb_i4_packed_words(cols);
    p.buffers = {storage(weights, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, rows * wpr),
                 storage(x, 1, VYB_ACCESS_READ_ONLY, VYB_DT_F32, batch * cols),
                 storage(row_scales, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, rows),
                 output(out, 3, VYB_DT_F32, batch * rows)};
    return emit(program, std::move(p));
}

int32_t vyb_math_i4x8_matvec_f32_scaled(const char* weights, const char* x, const char* row_scales, const char* out,
                                        uint32_t rows, uint32_t cols, uint32_t lib_op_id, vyb_program** program) {
    VYB_REQUIRE_NAMES(weights, x, row_scales, out);
    const char* id = lib_op_id ? "vyre-libs::quant::int4_matvec_f32_scaled"
                               : "vyre-primitives::math::quantized::i4x8_matvec_f32_scaled";
    if (rows == 0 || cols == 0)
        return emit(program, trap_program(id, out, VYB_DT_F32,
                                          "Fix: i4x8_matvec_f32_scaled requires rows > 0 and cols > 0."));
    int32_t rc = vyb_math_i4x8_batched_matvec_f32_scaled(weights, x, row_scales, out, 1, rows, cols, lib_op_id,
                                                         program);
    if (rc == VYB_OK) (*program)->p.op_id = id;
    return rc;
}

static int32_t matmul_common(const char* id, OpKind kind, const char* trap_msg, uint32_t out_count_mul,
                             const char* weights, const char* activations, const char* row_scales,
                             const char* batch_scales, const char* out, uint32_t batch, uint32_t rows,
                             uint32_t cols, vyb_program** program) {
    if (batch == 0 || rows == 0 || cols == 0) return emit(program, trap_program(id, out, VYB_DT_F32, trap_msg));
    Program p;
    p.op_id = id;
    p.kind = kind;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = batch;
    p.params.u[1] = rows;
    p.params.u[2] = cols;
    uint32_t wpr = vyb_i4_packed_words(cols);
    p.buffers = {storage(weights, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, rows * wpr),
                 storage(activations, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, batch * wpr),
                 storage(row_scales, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, rows),
                 storage(batch_scales, 3, VYB_ACCESS_READ_ONLY, VYB_DT_F32, batch),
                 output(out, 4, VYB_DT_F32, out_count_mul == 0 ? batch * rows : batch * out_count_mul)};
    return emit(program, std::move(p));
}

int32_t vyb_math_i4x8_batched_matmul_f32_scaled(const char* weights, const char* activations,
                                                const char* row_scales, const char* batch_scales, const char* out,
                                                uint32_t batch, uint32_t rows, uint32_t cols, uint32_t lib_op_id,
                                                vyb_program** program) {
    VYB_REQUIRE_NAMES(weights, activations, row_scales, batch_scales, out);
    return matmul_common(lib_op_id ? "vyre-libs::quant::int4_batched_matmul_f32_scaled"
                                   : "vyre-primitives::math::quantized::i4x8_batched_matmul_f32_scaled",
                         OpKind::I4BatchedMatmul,
                         "Fix: i4x8_batched_matmul_f32_scaled requires batch > 0, rows > 0, and cols > 0.", 0, weights,
                         activations, row_scales, batch_scales, out, batch, rows, cols, program);
}

int32_t vyb_math_i4x8_batched_matmul_top1_f32_scaled(const char* weights, const char* activations,
                                                     const char* row_scales, const char* batch_scales,
                                                     const char* out_scores, uint32_t batch, uint32_t rows,
                                                     uint32_t cols, uint32_t lib_op_id, vyb_program** program) {
    VYB_REQUIRE_NAMES(weights, activations, row_scales, batch_scales, out_scores);
    return matmul_common(lib_op_id ? "vyre-libs::quant::int4_batched_matmul_top1_f32_scaled"
                                   : "vyre-primitives::math::quantized::i4x8_batched_matmul_top1_f32_scaled",
                         OpKind::I4BatchedMatmulTop1,
                         "Fix: i4x8_batched_matmul_top1_f32_scaled requires batch > 0, rows > 0, and cols > 0.", 2,
                         weights, activations, row_scales, batch_scales, out_scores, batch, rows, cols, program);
}

// ---- int8 (int8.rs:15-78) -----------------------------------------------------------------------------------
int32_t vyb_quant_int8_unpack(const char* packed, const char* scales, const char* output_name, uint32_t n,
                              uint32_t cols, vyb_program** program) {
    VYB_REQUIRE_NAMES(packed, scales, output_name);
    if (cols == 0)
        return fail_invalid_program(
            "Fix: int8_unpack cols=0 divides by zero in the reference builder; pass cols > 0.");
    Program p;
    p.op_id = "vyre-libs::quant::int8_unpack";
    p.kind = OpKind::Int8Unpack;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = n;
    p.params.u[1] = cols;
    p.buffers = {storage(packed, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, n),
                 storage(scales, 1, VYB_ACCESS_READ_ONLY, VYB_DT_F32, div_ceil(n, cols)),
                 output(output_name, 2, VYB_DT_F32, n)};
    return emit(program, std::move(p));
}

int32_t vyb_quant_int8_pack(const char* input, const char* output_name, uint32_t n, vyb_program** program) {
    VYB_REQUIRE_NAMES(input, output_name);
    Program p;
    p.op_id = "vyre-libs::quant::int8_pack";
    p.kind = OpKind::Int8Pack;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = n;
    p.buffers = {storage(input, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, n), output(output_name, 1, VYB_DT_U32, n)};
    return emit(program, std::move(p));
}

// ---- linear_rows (builder.rs:253-361) -------------------------------------------------------------------------
static int32_t linear_rows_impl(const char* x, const char* w, const char* bias, const char* out, uint32_t rows,
                                uint32_t in_dim, uint32_t out_dim, uint32_t dtype, bool out_in,
                                vyb_program** program) {
    if (rows == 0 || in_dim == 0 || out_dim == 0)
        return fail_invalid_program(
            "Fix: linear_rows requires nonzero rows, input dimension, and output dimension");
    if (dtype != VYB_DT_F16 && dtype != VYB_DT_BF16 && dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: linear_rows supports F16, BF16, or F32 tensors; got tag " +
                                    std::to_string(dtype));
    uint32_t ic, oc, wc;
    if (!checked_mul(rows, in_dim, &ic))
        return fail_invalid_program("Fix: linear_rows rows*in_dim overflows u32; split the row batch");
    if (!checked_mul(rows, out_dim, &oc))
        return fail_invalid_program("Fix: linear_rows rows*out_dim overflows u32; split the row batch");
    if (!checked_mul(in_dim, out_dim, &wc))
        return fail_invalid_program("Fix: linear_rows in_dim*out_dim overflows u32; shard the projection");
    Program p;
    p.op_id = "vyre-libs::nn::linear_rows";
    p.kind = OpKind::LinearRows;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = rows;
    p.params.u[1] = in_dim;
    p.params.u[2] = out_dim;
    p.params.u[3] = dtype;
    p.params.u[4] = out_in ? 1 : 0;
    p.params.u[5] = bias ? 1 : 0;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, dtype, ic), storage(w, 1, VYB_ACCESS_READ_ONLY, dtype, wc)};
    if (bias) p.buffers.push_back(storage(bias, 2, VYB_ACCESS_READ_ONLY, dtype, out_dim));
    p.buffers.push_back(output(out, bias ? 3 : 2, dtype, oc));
    return emit(program, std::move(p));
}

int32_t vyb_nn_linear_rows(const char* x, const char* w, const char* b, const char* out, uint32_t rows,
                           uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, b, out);
    return linear_rows_impl(x, w, b, out, rows, in_dim, out_dim, VYB_DT_F32, false, program);
}
int32_t vyb_nn_linear_rows_no_bias(const char* x, const char* w, const char* out, uint32_t rows, uint32_t in_dim,
                                   uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, out);
    return linear_rows_impl(x, w, nullptr, out, rows, in_dim, out_dim, VYB_DT_F32, false, program);
}
int32_t vyb_nn_linear_rows_no_bias_typed(const char* x, const char* w, const char* out, uint32_t rows,
                                         uint32_t in_dim, uint32_t out_dim, uint32_t dtype, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, out);
    return linear_rows_impl(x, w, nullptr, out, rows, in_dim, out_dim, dtype, false, program);
}
int32_t vyb_nn_linear_rows_no_bias_out_in_typed(const char* x, const char* w, const char* out, uint32_t rows,
                                                uint32_t in_dim, uint32_t out_dim, uint32_t dtype,
                                                vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, out);
    return linear_rows_impl(x, w, nullptr, out, rows, in_dim, out_dim, dtype, true, program);
}

// ---- Matmul / MatmulBias (matmul.rs:17-136, 138-271) and nn::linear over them: u32 wrapping ----------------------
namespace {
// matmul_tiled/program.rs:105-200 for the cooperative (non-MMA) path, which is the one a U32 product takes: the
// default [16, 16, 1] workgroup gives 16 x 16 output tiles on 256 flat lanes, two workgroup tiles of tile x 16 values,
// and an output padded to whole tiles with the logical bytes as its readback range.
int32_t tiled_matmul_program(const char* op_id, const char* a, const char* b, const char* bias, const char* out,
                             uint32_t m, uint32_t k, uint32_t n, uint32_t tile, vyb_program** program) {
    uint32_t ac, bc, oc, a_tile, b_tile, tiles, padded;
    if (!checked_mul(m, k, &ac) || !checked_mul(k, n, &bc) || !checked_mul(m, n, &oc) || !checked_mul(16, tile, &a_tile) ||
        !checked_mul(tile, 16, &b_tile) || !checked_mul(div_ceil(m, 16), div_ceil(n, 16), &tiles) ||
        !checked_mul(tiles, 256, &padded))
        return fail_invalid_program(std::string("Fix: ") + op_id + " element counts overflow u32; shard the product.");
    Program p;
    p.op_id = op_id;
    p.kind = OpKind::MatmulU32;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = m;
    p.params.u[1] = k;
    p.params.u[2] = n;
    p.params.u[3] = bias ? 1 : 0;
    p.params.u[4] = tile;
    p.buffers = {storage(a, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, ac), storage(b, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, bc)};
    if (bias) p.buffers.push_back(storage(bias, 2, VYB_ACCESS_READ_ONLY, VYB_DT_U32, n));
    p.buffers.push_back(workgroup("matmul_a_tile", a_tile, VYB_DT_U32));
    p.buffers.push_back(workgroup("matmul_b_tile", b_tile, VYB_DT_U32));
    BufferDecl o = output(out, bias ? 3 : 2, VYB_DT_U32, padded);
    o.has_output_byte_range = true;
    o.output_byte_begin = 0;
    o.output_byte_end = uint64_t(oc) * 4;
    p.buffers.push_back(o);
    return emit(program, std::move(p));
}

int32_t flat_matmul_program(const char* op_id, const char* a, const char* b, const char* bias, const char* out, uint32_t m,
                            uint32_t k, uint32_t n, vyb_program** program) {
    uint32_t ac, bc, oc;
    if (!checked_mul(m, k, &ac) || !checked_mul(k, n, &bc) || !checked_mul(m, n, &oc))
        return fail_invalid_program(std::string("Fix: ") + op_id + " element counts overflow u32; shard the product.");
    Program p;
    p.op_id = op_id;
    p.kind = OpKind::MatmulU32;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = m;
    p.params.u[1] = k;
    p.params.u[2] = n;
    p.params.u[3] = bias ? 1 : 0;
    p.buffers = {storage(a, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, ac), storage(b, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, bc)};
    if (bias) p.buffers.push_back(storage(bias, 2, VYB_ACCESS_READ_ONLY, VYB_DT_U32, n));
    p.buffers.push_back(output(out, bias ? 3 : 2, VYB_DT_U32, oc));
    return emit(program, std::move(p));
}
}  // namespace

int32_t vyb_math_matmul(const char* a, const char* b, const char* out, uint32_t m, uint32_t k, uint32_t n,
                        vyb_program** program) {
    VYB_REQUIRE_NAMES(a, b, out);
    if (m == 0 || k == 0 || n == 0)
        return fail_invalid_program("Fix: matmul requires nonzero m, k and n.");
    return flat_matmul_program("vyre-libs::math::matmul", a, b, nullptr, out, m, k, n, program);
}

int32_t vyb_math_matmul_bias(const char* a, const char* b, const char* bias, const char* out, uint32_t m, uint32_t k,
                             uint32_t n, vyb_program** program) {
    VYB_REQUIRE_NAMES(a, b, bias, out);
    if (m == 0 || k == 0 || n == 0)
        return fail_invalid_program("Fix: matmul_bias requires nonzero m, k and n.");
    return flat_matmul_program("vyre-libs::math::matmul_bias", a, b, bias, out, m, k, n, program);
}

int32_t vyb_math_matmul_bias_tiled(const char* a, const char* b, const char* bias, const char* out, uint32_t m, uint32_t k,
                                   uint32_t n, uint32_t tile, vyb_program** program) {
    VYB_REQUIRE_NAMES(a, b, bias, out);
    if (m == 0 || k == 0 || n == 0 || tile == 0)
        return fail_invalid_program("Fix: matmul_bias_tiled requires nonzero m, k, n and tile.");
    return tiled_matmul_program("vyre-libs::math::matmul_bias_tiled", a, b, bias, out, m, k, n, tile, program);
}

// nn::linear (vyre-libs/src/nn/linear/inner/builder.rs:139-162): out[i] = sum_k x[k] * w[k, i] + b[i]; from
// in_dim * out_dim >= 1024 on the builder hands over to linear_tiled with tile 32 (tiled.rs:13-50)
int32_t vyb_nn_linear_tiled(const char* x, const char* w, const char* b, const char* out, uint32_t in_dim, uint32_t out_dim,
                            uint32_t tile, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, b, out);
    if (in_dim == 0) return fail_invalid_program("Fix: linear_tiled in_dim=0 is invalid: empty reduction");
    if (out_dim == 0) return fail_invalid_program("Fix: linear_tiled out_dim=0 is invalid: empty output");
    if (tile == 0) return fail_invalid_program("Fix: linear_tiled tile=0 is invalid: tile width must be > 0");
    uint32_t work;
    if (!checked_mul(in_dim, out_dim, &work))
        return fail_invalid_program("Fix: linear_tiled in_dim*out_dim overflows u32; reduce dimensions.");
    return tiled_matmul_program("vyre-libs::nn::linear_tiled", x, w, b, out, 1, in_dim, out_dim, tile, program);
}

int32_t vyb_nn_linear(const char* x, const char* w, const char* b, const char* out, uint32_t in_dim, uint32_t out_dim,
                      vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, b, out);
    uint32_t work;
    if (checked_mul(in_dim, out_dim, &work) && work >= 1024)
        return vyb_nn_linear_tiled(x, w, b, out, in_dim, out_dim, 32, program);
    if (in_dim == 0 || out_dim == 0)
        return fail_invalid_program("Fix: vyre-libs::nn::linear build failed: x and out need at least one element each.");
    if (!checked_mul(in_dim, out_dim, &work))
        return fail_invalid_program("Fix: linear in_dim*out_dim overflows u32; reduce dimensions.");
    return flat_matmul_program("vyre-libs::nn::linear", x, w, b, out, 1, in_dim, out_dim, program);
}

// ---- MoE (gating.rs:19-69, softmax_top_k.rs:25-101, top_k.rs:18-60) -----------------------------------------------
int32_t vyb_nn_moe_gate(const char* input_scores, const char* output_indices, const char* output_weights,
                        uint32_t num_experts, uint32_t k, vyb_program** program) {
    VYB_REQUIRE_NAMES(input_scores, output_indices, output_weights);
    Program p;
    p.op_id = "vyre-libs::nn::moe_gate";
    p.kind = OpKind::MoeGate;
    p.workgroup = {1, 1, 1};
    p.params.u[0] = num_experts;
    p.params.u[1] = k;
    p.params.u[2] = 1;  // tokens
    p.buffers = {storage(input_scores, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, num_experts),
                 storage(output_indices, 1, VYB_ACCESS_READ_WRITE, VYB_DT_U32, k),
                 output(output_weights, 2, VYB_DT_F32, k),
                 workgroup("__moe_gate_scores_scratch", num_experts, VYB_DT_F32),
                 workgroup("__moe_gate_stats", 2, VYB_DT_F32)};
    return emit(program, std::move(p));
}

int32_t vyb_nn_softmax_top_k(const char* scores, const char* out_indices, const char* out_weights, uint32_t n,
                             uint32_t k, vyb_program** program) {
    VYB_REQUIRE_NAMES(scores, out_indices, out_weights);
    const char* id = "vyre-libs::nn::softmax_top_k";
    if (k == 0)
        return emit(program,
                    trap_program(id, out_indices, VYB_DT_U32,
                                 "Fix: softmax_top_k requires k > 0 so the selection scratch has at least one slot."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::SoftmaxTopK;
    p.params.u[0] = n;
    p.params.u[1] = k;
    p.buffers = {storage(scores, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, n), output(out_indices, 1, VYB_DT_U32, k),
                 storage(out_weights, 2, VYB_ACCESS_READ_WRITE, VYB_DT_F32, k),
                 storage("best_vals", 3, VYB_ACCESS_READ_WRITE, VYB_DT_F32, k),
                 storage("best_idxs", 4, VYB_ACCESS_READ_WRITE, VYB_DT_U32, k)};
    return emit(program, std::move(p));
}

int32_t vyb_nn_top_k(const char* input, const char* output_indices, uint32_t n, uint32_t k, vyb_program** program) {
    VYB_REQUIRE_NAMES(input, output_indices);
    const char* id = "vyre-libs::nn::top_k";
    if (k == 0)
        return emit(program, trap_program(id, output_indices, VYB_DT_U32,
                                          "Fix: top_k requires k > 0 so the selection scratch has at least one slot."));
    Program p;
    p.op_id = id;
    p.kind = OpKind::TopK;
    p.params.u[0] = n;
    p.params.u[1] = k;
    p.buffers = {storage(input, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, n), output(output_indices, 1, VYB_DT_U32, k),
                 storage("best_vals", 2, VYB_ACCESS_READ_WRITE, VYB_DT_F32, k),
                 storage("best_idxs", 3, VYB_ACCESS_READ_WRITE, VYB_DT_U32, k)};
    return emit(program, std::move(p));
}

// ---- swiglu (swiglu.rs:17-48) ----------------------------------------------------------------------------------------
static int32_t swiglu_impl(const char* gate, const char* up, const char* out, uint32_t n, uint32_t dtype,
                           vyb_program** program) {
    const char* id = "vyre-libs::nn::swiglu";
    if (n == 0) return emit(program, trap_program(id, out, dtype, "Fix: swiglu requires n > 0"));
    Program p;
    p.op_id = id;
    p.kind = OpKind::Swiglu;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = n;
    p.params.u[1] = dtype;
    p.buffers = {storage(gate, 0, VYB_ACCESS_READ_ONLY, dtype, n), storage(up, 1, VYB_ACCESS_READ_ONLY, dtype, n),
                 output(out, 2, dtype, n)};
    return emit(program, std::move(p));
}
int32_t vyb_nn_swiglu(const char* gate, const char* up, const char* output_name, uint32_t n, vyb_program** program) {
    VYB_REQUIRE_NAMES(gate, up, output_name);
    return swiglu_impl(gate, up, output_name, n, VYB_DT_F32, program);
}
int32_t vyb_nn_swiglu_typed(const char* gate, const char* up, const char* output_name, uint32_t n, uint32_t dtype,
                            vyb_program** program) {
    VYB_REQUIRE_NAMES(gate, up, output_name);
    if (n == 0) return fail_invalid_program("Fix: swiglu_typed requires n > 0");
    if (dtype != VYB_DT_F16 && dtype != VYB_DT_BF16 && dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: swiglu_typed supports F16, BF16, or F32 tensors; got tag " +
                                    std::to_string(dtype));
    return swiglu_impl(gate, up, output_name, n, dtype, program);
}

// ---- residual_add (residual_add.rs:8-52 over unary.rs:44-76) ----------------------------------------------------------
static int32_t residual_add_impl(const char* residual, const char* branch, const char* out, uint32_t n, uint32_t dtype,
                                 vyb_program** program) {
    const char* id = "vyre-libs::nn::residual_add";
    if (n == 0) return emit(program, trap_program(id, out, dtype, "Fix: residual_add requires n > 0"));
    Program p;
    p.op_id = id;
    p.kind = OpKind::ResidualAdd;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = n;
    p.params.u[1] = dtype;
    p.buffers = {storage(residual, 0, VYB_ACCESS_READ_ONLY, dtype, n), storage(branch, 1, VYB_ACCESS_READ_ONLY, dtype, n),
                 output(out, 2, dtype, n)};
    return emit(program, std::move(p));
}
int32_t vyb_nn_residual_add(const char* residual, const char* branch, const char* output_name, uint32_t n,
                            vyb_program** program) {
    VYB_REQUIRE_NAMES(residual, branch, output_name);
    return residual_add_impl(residual, branch, output_name, n, VYB_DT_F32, program);
}
int32_t vyb_nn_residual_add_typed(const char* residual, const char* branch, const char* output_name, uint32_t n,
                                  uint32_t dtype, vyb_program** program) {
    VYB_REQUIRE_NAMES(residual, branch, output_name);
    if (n == 0) return fail_invalid_program("Fix: residual_add_typed requires n > 0");
    if (dtype != VYB_DT_F16 && dtype != VYB_DT_BF16 && dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: residual_add_typed supports F16, BF16, or F32 tensors; got tag " +
                                    std::to_string(dtype));
    return residual_add_impl(residual, branch, output_name, n, dtype, program);
}

// ---- learned_rms_norm / gated_rms_norm (gated_rms_norm.rs:35-247) -------------------------------------------------------
static int32_t rms_norm_impl(const char* input, const char* weight, const char* gate, const char* out, uint32_t rows,
                             uint32_t hidden, float eps, uint32_t dtype, uint32_t weight_dtype, vyb_program** program) {
    auto floating = [](uint32_t t) { return t == VYB_DT_F16 || t == VYB_DT_BF16 || t == VYB_DT_F32; };
    if (rows == 0 || hidden == 0)
        return fail_invalid_program("Fix: gated RMSNorm requires nonzero rows and hidden size; got rows=" + std::to_string(rows) +
                                    ", hidden=" + std::to_string(hidden));
    if (!floating(dtype) || !floating(weight_dtype))
        return fail_invalid_program("Fix: gated RMSNorm supports F16, BF16, or F32 source tensors; got tag " +
                                    std::to_string(floating(dtype) ? weight_dtype : dtype));
    if (uint64_t(rows) * hidden > 0xFFFFFFFFull)
        return fail_invalid_program("Fix: gated RMSNorm rows*hidden overflows u32; split the tensor");
    const uint32_t total = rows * hidden;
    Program p;
    p.op_id = gate ? "vyre-libs::nn::gated_rms_norm" : "vyre-libs::nn::learned_rms_norm";
    p.kind = OpKind::RmsNorm;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = rows;
    p.params.u[1] = hidden;
    std::memcpy(&p.params.u[2], &eps, 4);
    p.params.u[3] = dtype;
    p.params.u[4] = weight_dtype;
    p.params.u[5] = gate ? 1u : 0u;
    p.buffers = {storage(input, 0, VYB_ACCESS_READ_ONLY, dtype, total), storage(weight, 1, VYB_ACCESS_READ_ONLY, weight_dtype, hidden)};
    if (gate) p.buffers.push_back(storage(gate, 2, VYB_ACCESS_READ_ONLY, dtype, total));
    p.buffers.push_back(output(out, gate ? 3 : 2, dtype, total));
    return emit(program, std::move(p));
}
int32_t vyb_nn_learned_rms_norm(const char* input, const char* weight, const char* output_name, uint32_t rows,
                                uint32_t hidden, float eps, uint32_t dtype, vyb_program** program) {
    VYB_REQUIRE_NAMES(input, weight, output_name);
    return rms_norm_impl(input, weight, nullptr, output_name, rows, hidden, eps, dtype, dtype, program);
}
int32_t vyb_nn_gated_rms_norm(const char* input, const char* weight, const char* gate, const char* output_name,
                              uint32_t rows, uint32_t hidden, float eps, uint32_t dtype, vyb_program** program) {
    VYB_REQUIRE_NAMES(input, weight, gate, output_name);
    return rms_norm_impl(input, weight, gate, output_name, rows, hidden, eps, dtype, dtype, program);
}
int32_t vyb_nn_gated_rms_norm_with_weight_dtype(const char* input, const char* weight, const char* gate, const char* output_name,
                                                uint32_t rows, uint32_t hidden, float eps, uint32_t dtype, uint32_t weight_dtype,
                                                vyb_program** program) {
    VYB_REQUIRE_NAMES(input, weight, gate, output_name);
    return rms_norm_impl(input, weight, gate, output_name, rows, hidden, eps, dtype, weight_dtype, program);
}

// ---- GGML K-quants (ggml.rs:28-400): Q4_K blocks of 32 weights in 4 words, Q2_K blocks of 16 weights in 1 word ----------
static int32_t k_quant_unpack_impl(uint32_t bits, const char* packed, const char* scales, const char* mins, const char* out,
                                   uint32_t n, vyb_program** program) {
    const std::string id = bits == 4 ? "vyre-libs::quant::q4_k_unpack" : "vyre-libs::quant::q2_k_unpack";
    if (n == 0) return fail_invalid_program("Fix: " + id + " n=0 is invalid");
    const uint32_t block_size = bits == 4 ? 32u : 16u, words_per_block = bits == 4 ? 4u : 1u;
    const uint64_t blocks = (uint64_t(n) + block_size - 1) / block_size;
    if (blocks * words_per_block > 0xFFFFFFFFull) return fail_invalid_program("Fix: " + id + " packed word count overflows u32");
    Program p;
    p.op_id = id;
    p.kind = OpKind::KQuantUnpack;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = n;
    p.params.u[1] = bits;
    p.buffers = {storage(packed, 0, VYB_ACCESS_READ_ONLY, VYB_DT_U32, uint32_t(blocks * words_per_block)),
                 storage(scales, 1, VYB_ACCESS_READ_ONLY, VYB_DT_F32, uint32_t(blocks)),
                 storage(mins, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, uint32_t(blocks)), output(out, 3, VYB_DT_F32, n)};
    return emit(program, std::move(p));
}
int32_t vyb_quant_q4_k_unpack(const char* packed, const char* scales, const char* mins, const char* output_name, uint32_t n,
                              vyb_program** program) {
    VYB_REQUIRE_NAMES(packed, scales, mins, output_name);
    return k_quant_unpack_impl(4, packed, scales, mins, output_name, n, program);
}
int32_t vyb_quant_q2_k_unpack(const char* packed, const char* scales, const char* mins, const char* output_name, uint32_t n,
                              vyb_program** program) {
    VYB_REQUIRE_NAMES(packed, scales, mins, output_name);
    return k_quant_unpack_impl(2, packed, scales, mins, output_name, n, program);
}
static int32_t k_quant_linear_impl(uint32_t bits, const char* x, const char* w_packed, const char* w_scales, const char* w_mins,
                                   const char* b, const char* out, uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    const std::string id = bits == 4 ? "vyre-libs::quant::q4_k_linear" : "vyre-libs::quant::q2_k_linear";
    if (in_dim == 0 || out_dim == 0) return fail_invalid_program("Fix: " + id + " all dims must be > 0");
    if (uint64_t(in_dim) * out_dim > 0xFFFFFFFFull) return fail_invalid_program("Fix: " + id + " dimensions overflow u32");
    const uint32_t block_size = bits == 4 ? 32u : 16u, words_per_block = bits == 4 ? 4u : 1u;
    const uint64_t blocks = (uint64_t(in_dim) * out_dim + block_size - 1) / block_size;
    if (blocks * words_per_block > 0xFFFFFFFFull) return fail_invalid_program("Fix: " + id + " packed word count overflows u32");
    Program p;
    p.op_id = id;
    p.kind = OpKind::KQuantLinear;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = in_dim;
    p.params.u[1] = out_dim;
    p.params.u[2] = bits;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, in_dim),
                 storage(w_packed, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, uint32_t(blocks * words_per_block)),
                 storage(w_scales, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, uint32_t(blocks)),
                 storage(w_mins, 3, VYB_ACCESS_READ_ONLY, VYB_DT_F32, uint32_t(blocks)),
                 storage(b, 4, VYB_ACCESS_READ_ONLY, VYB_DT_F32, out_dim), output(out, 5, VYB_DT_F32, out_dim)};
    return emit(program, std::move(p));
}
int32_t vyb_quant_q4_k_linear(const char* x, const char* w_packed, const char* w_scales, const char* w_mins, const char* b,
                              const char* out, uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, w_scales, w_mins, b, out);
    return k_quant_linear_impl(4, x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim, program);
}
int32_t vyb_quant_q2_k_linear(const char* x, const char* w_packed, const char* w_scales, const char* w_mins, const char* b,
                              const char* out, uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, w_scales, w_mins, b, out);
    return k_quant_linear_impl(2, x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim, program);
}

// ---- expert_mlp (expert_mlp.rs:18-150) ---------------------------------------------------------------------------------
int32_t vyb_nn_expert_mlp(const char* x, const char* w_gate, const char* b_gate, const char* w_up, const char* b_up,
                          const char* w_down, const char* b_down, const char* out, uint32_t in_dim,
                          uint32_t hidden_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_gate, b_gate, w_up, b_up, w_down, b_down, out);
    if (in_dim == 0 || hidden_dim == 0 || out_dim == 0)
        return fail_invalid_program("Fix: expert_mlp all dims must be > 0");
    uint32_t ih, ho;
    if (!checked_mul(in_dim, hidden_dim, &ih))
        return fail_invalid_program("Fix: expert_mlp in_dim*hidden_dim overflows u32; reduce dimensions.");
    if (!checked_mul(hidden_dim, out_dim, &ho))
        return fail_invalid_program("Fix: expert_mlp hidden_dim*out_dim overflows u32; reduce dimensions.");
    Program p;
    p.op_id = "vyre-libs::nn::moe::expert_mlp";
    p.kind = OpKind::ExpertMlp;
    p.workgroup = {64, 1, 1};
    p.params.u[0] = in_dim;
    p.params.u[1] = hidden_dim;
    p.params.u[2] = out_dim;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, in_dim),
                 storage(w_gate, 1, VYB_ACCESS_READ_ONLY, VYB_DT_F32, ih),
                 storage(b_gate, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, hidden_dim),
                 storage(w_up, 3, VYB_ACCESS_READ_ONLY, VYB_DT_F32, ih),
                 storage(b_up, 4, VYB_ACCESS_READ_ONLY, VYB_DT_F32, hidden_dim),
                 storage(w_down, 5, VYB_ACCESS_READ_ONLY, VYB_DT_F32, ho),
                 storage(b_down, 6, VYB_ACCESS_READ_ONLY, VYB_DT_F32, out_dim),
                 output(out, 7, VYB_DT_F32, out_dim)};
    return emit(program, std::move(p));
}

// ---- moe_layer_route_and_accumulate (moe_layer.rs:33-121) -----------------------------------------------------------------
int32_t vyb_nn_moe_layer_route_and_accumulate(const char* x, const char* w_router, const char* b_router,
                                              const char* expert_indices, const char* expert_weights,
                                              const char* expert_outputs, const char* out, uint32_t in_dim,
                                              uint32_t num_experts, uint32_t out_dim, uint32_t k,
                                              vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_router, b_router, expert_indices, expert_weights, expert_outputs, out);
    if (in_dim == 0 || num_experts == 0 || out_dim == 0 || k == 0)
        return fail_invalid_program("Fix: moe_layer all dims must be > 0");
    if (k > num_experts) return fail_invalid_program("Fix: moe_layer k cannot exceed num_experts");
    uint32_t wr, eo;
    if (!checked_mul(in_dim, num_experts, &wr)) return fail_invalid_program("Fix: moe_layer w_router count overflow");
    if (!checked_mul(k, out_dim, &eo)) return fail_invalid_program("Fix: moe_layer expert_outputs count overflow");
    Program p;
    p.op_id = "vyre-libs::nn::moe_layer_accumulate";
    p.kind = OpKind::MoeLayerAccumulate;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = in_dim;
    p.params.u[1] = num_experts;
    p.params.u[2] = out_dim;
    p.params.u[3] = k;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, in_dim),
                 storage(w_router, 1, VYB_ACCESS_READ_ONLY, VYB_DT_F32, wr),
                 storage(b_router, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, num_experts),
                 storage(expert_indices, 3, VYB_ACCESS_READ_ONLY, VYB_DT_U32, k),
                 storage(expert_weights, 4, VYB_ACCESS_READ_ONLY, VYB_DT_F32, k),
                 storage(expert_outputs, 5, VYB_ACCESS_READ_ONLY, VYB_DT_F32, eo),
                 output(out, 6, VYB_DT_F32, out_dim)};
    return emit(program, std::move(p));
}

// ---- serving-layout operators -------------------------------------------------------------------------------------------------
int32_t vyb_nn_linear_int4_grouped_rowmajor(const char* x, const char* w_packed, const char* scale, const char* out,
                                            uint32_t batch, uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                            uint32_t out_dtype, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, scale, out);
    if (in_dim == 0)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor in_dim=0 is invalid: empty reduction");
    if (out_dim == 0)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor out_dim=0 is invalid: empty output");
    if (batch == 0)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor batch=0 is invalid: batch size must be > 0");
    if (group_size == 0)
        return fail_invalid_program(
            "Fix: linear_int4_grouped_rowmajor group_size=0 is invalid: group size must be > 0");
    if (in_dim % 8 != 0)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor in_dim=" + std::to_string(in_dim) +
                                    " is not divisible by 8; pad weights to a multiple of 8.");
    if (in_dim % group_size != 0)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor in_dim=" + std::to_string(in_dim) +
                                    " is not a multiple of group_size=" + std::to_string(group_size) +
                                    "; pad the last group.");
    if (out_dtype != VYB_DT_BF16 && out_dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: linear_int4_grouped_rowmajor output dtype must be BF16 or F32.");
    uint32_t xc, wc, sc, oc;
    if (!checked_mul(batch, in_dim, &xc) || !checked_mul(out_dim, in_dim / 8, &wc) ||
        !checked_mul(out_dim, in_dim / group_size, &sc) || !checked_mul(batch, out_dim, &oc))
        return fail_invalid_program(
            "Fix: linear_int4_grouped_rowmajor element counts overflow u32; shard the projection.");
    Program p;
    p.op_id = "vyre-b200::nn::linear_int4_grouped_rowmajor";
    p.kind = OpKind::LinearInt4GroupedRowmajor;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = batch;
    p.params.u[1] = in_dim;
    p.params.u[2] = out_dim;
    p.params.u[3] = group_size;
    p.params.u[4] = out_dtype;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, xc),
                 storage(w_packed, 1, VYB_ACCESS_READ_ONLY, VYB_DT_U32, wc),
                 storage(scale, 2, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, sc), output(out, 3, out_dtype, oc)};
    return emit(program, std::move(p));
}

// The projection of a residual block as ONE node: learned RMSNorm (dense_gated_mlp.rs:168-200 `mlp.norm`, bf16) in front
// when `norm_weight` is named, residual add (`mlp.residual`) behind when `residual` is named. Values are those of the three
// operators run one after the other (every intermediate rounded to bf16 as the stand-alone operators round it). With `gate`
// named instead of `residual`, the output is SwiGLU(gate, projection) (`mlp.swiglu` behind up_proj, gate = gate_proj's output).
int32_t vyb_nn_linear_int4_block(const char* x, const char* norm_weight, const char* w_packed, const char* scale, const char* gate,
                                 const char* residual, const char* out, uint32_t batch, uint32_t in_dim, uint32_t out_dim,
                                 uint32_t group_size, float norm_eps, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_packed, scale, out);
    if (!norm_weight && !residual && !gate)
        return fail_invalid_program(
            "Fix: linear_int4_block needs a norm weight, a gate, a residual, or a norm weight with one of the two; use "
            "linear_int4_grouped_rowmajor for the bare projection.");
    if (gate && residual)
        return fail_invalid_program("Fix: linear_int4_block takes a gate or a residual behind the projection, not both.");
    if (batch == 0 || in_dim == 0 || out_dim == 0 || group_size == 0)
        return fail_invalid_program("Fix: linear_int4_block requires nonzero batch, in_dim, out_dim and group_size; got batch=" +
                                    std::to_string(batch) + ", in_dim=" + std::to_string(in_dim) + ", out_dim=" +
                                    std::to_string(out_dim) + ", group_size=" + std::to_string(group_size) + ".");
    if (in_dim % 8 != 0)
        return fail_invalid_program("Fix: linear_int4_block in_dim=" + std::to_string(in_dim) +
                                    " is not divisible by 8; pad weights to a multiple of 8.");
    if (in_dim % group_size != 0)
        return fail_invalid_program("Fix: linear_int4_block in_dim=" + std::to_string(in_dim) + " is not a multiple of group_size=" +
                                    std::to_string(group_size) + "; pad the last group.");
    if (norm_weight && !(norm_eps >= 0.0f))
        return fail_invalid_program("Fix: linear_int4_block needs a non-negative, finite-or-zero norm epsilon.");
    uint32_t xc, wc, sc, oc;
    if (!checked_mul(batch, in_dim, &xc) || !checked_mul(out_dim, in_dim / 8, &wc) ||
        !checked_mul(out_dim, in_dim / group_size, &sc) || !checked_mul(batch, out_dim, &oc))
        return fail_invalid_program("Fix: linear_int4_block element counts overflow u32; shard the projection.");
    Program p;
    p.op_id = "vyre-b200::nn::linear_int4_block";
    p.kind = OpKind::LinearInt4Block;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = batch;
    p.params.u[1] = in_dim;
    p.params.u[2] = out_dim;
    p.params.u[3] = group_size;
    p.params.u[4] = VYB_DT_BF16;
    p.params.u[5] = (norm_weight ? 1u : 0u) | (residual ? 2u : 0u) | (gate ? 4u : 0u);
    std::memcpy(&p.params.u[6], &norm_eps, 4);
    uint32_t slot = 0;
    p.buffers.push_back(storage(x, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, xc));
    if (norm_weight) p.buffers.push_back(storage(norm_weight, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, in_dim));
    p.buffers.push_back(storage(w_packed, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_U32, wc));
    p.buffers.push_back(storage(scale, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, sc));
    if (gate) p.buffers.push_back(storage(gate, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, oc));
    if (residual) p.buffers.push_back(storage(residual, slot++, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, oc));
    p.buffers.push_back(output(out, slot++, VYB_DT_BF16, oc));
    return emit(program, std::move(p));
}

int32_t vyb_nn_linear_int8_weight_only(const char* x, const char* w, const char* scale, const char* out,
                                       uint32_t batch, uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, scale, out);
    if (batch == 0 || in_dim == 0 || out_dim == 0)
        return fail_invalid_program(
            "Fix: linear_int8_weight_only requires nonzero batch, input dimension, and output dimension");
    uint32_t xc, wc, oc;
    if (!checked_mul(batch, in_dim, &xc) || !checked_mul(out_dim, in_dim, &wc) || !checked_mul(batch, out_dim, &oc))
        return fail_invalid_program(
            "Fix: linear_int8_weight_only element counts overflow u32; shard the projection.");
    Program p;
    p.op_id = "vyre-b200::nn::linear_int8_weight_only";
    p.kind = OpKind::LinearInt8WeightOnly;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = batch;
    p.params.u[1] = in_dim;
    p.params.u[2] = out_dim;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_F32, xc),
                 storage(w, 1, VYB_ACCESS_READ_ONLY, VYB_DT_I8, wc),
                 storage(scale, 2, VYB_ACCESS_READ_ONLY, VYB_DT_F32, out_dim), output(out, 3, VYB_DT_F32, oc)};
    return emit(program, std::move(p));
}

int32_t vyb_nn_linear_int8_dynamic(const char* x, const char* w, const char* x_scale, const char* out, uint32_t rows,
                                   uint32_t in_dim, uint32_t out_dim, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w, x_scale, out);
    if (rows == 0 || in_dim == 0 || out_dim == 0)
        return fail_invalid_program(
            "Fix: linear_int8_dynamic requires nonzero rows, input dimension, and output dimension");
    if (in_dim % 16 != 0)
        return fail_invalid_program("Fix: linear_int8_dynamic in_dim=" + std::to_string(in_dim) +
                                    " is not divisible by 16; pad the reduction dimension.");
    uint32_t xc, wc, oc;
    if (!checked_mul(rows, in_dim, &xc) || !checked_mul(out_dim, in_dim, &wc) || !checked_mul(rows, out_dim, &oc))
        return fail_invalid_program("Fix: linear_int8_dynamic element counts overflow u32; shard the projection.");
    Program p;
    p.op_id = "vyre-b200::nn::linear_int8_dynamic";
    p.kind = OpKind::LinearInt8Dynamic;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = rows;
    p.params.u[1] = in_dim;
    p.params.u[2] = out_dim;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, xc),
                 storage(w, 1, VYB_ACCESS_READ_ONLY, VYB_DT_I8, wc),
                 storage(x_scale, 2, VYB_ACCESS_READ_WRITE, VYB_DT_F32, rows), output(out, 3, VYB_DT_I32, oc)};
    return emit(program, std::move(p));
}

int32_t vyb_nn_moe_ffn_int4(const char* x, const char* w_router, const char* w13, const char* s13, const char* w2,
                            const char* s2, const char* out, const char* routing_idx, const char* routing_w,
                            uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk,
                            uint32_t group_size, vyb_program** program) {
    VYB_REQUIRE_NAMES(x, w_router, w13, s13, w2, s2, out, routing_idx, routing_w);
    if (tokens == 0 || hidden == 0 || inter == 0 || experts == 0 || topk == 0)
        return fail_invalid_program("Fix: moe_ffn_int4 all dims must be > 0");
    if (topk > experts) return fail_invalid_program("Fix: moe_ffn_int4 topk cannot exceed experts");
    if (group_size == 0 || hidden % group_size != 0 || inter % group_size != 0)
        return fail_invalid_program(
            "Fix: moe_ffn_int4 hidden and inter must be multiples of a non-zero group_size; pad the projections.");
    if (hidden % 8 != 0 || inter % 8 != 0)
        return fail_invalid_program("Fix: moe_ffn_int4 hidden and inter must be divisible by 8.");
    uint64_t w13_words = uint64_t(experts) * 2 * inter * (hidden / 8);
    uint64_t s13_count = uint64_t(experts) * 2 * inter * (hidden / group_size);
    uint64_t w2_words = uint64_t(experts) * hidden * (inter / 8);
    uint64_t s2_count = uint64_t(experts) * hidden * (inter / group_size);
    uint64_t xo = uint64_t(tokens) * hidden;
    const uint64_t lim = std::numeric_limits<uint32_t>::max();
    if (w13_words > lim || s13_count > lim || w2_words > lim || s2_count > lim || xo > lim)
        return fail_invalid_program("Fix: moe_ffn_int4 element counts overflow u32; shard experts or tokens.");
    Program p;
    p.op_id = "vyre-b200::nn::moe_ffn_int4";
    p.kind = OpKind::MoeFfnInt4;
    p.workgroup = {256, 1, 1};
    p.params.u[0] = tokens;
    p.params.u[1] = hidden;
    p.params.u[2] = inter;
    p.params.u[3] = experts;
    p.params.u[4] = topk;
    p.params.u[5] = group_size;
    p.buffers = {storage(x, 0, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, uint32_t(xo)),
                 storage(w_router, 1, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, experts * hidden),
                 storage(w13, 2, VYB_ACCESS_READ_ONLY, VYB_DT_U32, uint32_t(w13_words)),
                 storage(s13, 3, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, uint32_t(s13_count)),
                 storage(w2, 4, VYB_ACCESS_READ_ONLY, VYB_DT_U32, uint32_t(w2_words)),
                 storage(s2, 5, VYB_ACCESS_READ_ONLY, VYB_DT_BF16, uint32_t(s2_count)),
                 output(out, 6, VYB_DT_BF16, uint32_t(xo)),
                 storage(routing_idx, 7, VYB_ACCESS_READ_WRITE, VYB_DT_U32, tokens * topk),
                 storage(routing_w, 8, VYB_ACCESS_READ_WRITE, VYB_DT_F32, tokens * topk)};
    return emit(program, std::move(p));
}

// ---- accessors ----------------------------------------------------------------------------------------------------------------------
// ---- Program from an op id plus the BufferDecls of a vyre Program -----------------------------------------------------
// What TargetCompiler::compile(&Artifact) (vyre-megakernel/src/target.rs:180-189, helper :253-322) can call: it is
// handed an Artifact, i.e. a Program whose dimensions are IR literals, not builder arguments. The op id (the outermost
// Region generator) picks the builder; the dimensions come from the op spec when the caller attached one to the
// Program's metadata map (docs/wire-format.md:104-111), else from the buffer counts; the rebuilt program's buffers are
// then cross-checked against the declarations one by one.
static const vyb_buffer_decl* decl_at(const vyb_buffer_decl* d, uint32_t n, uint32_t binding) {
    for (uint32_t i = 0; i < n; ++i)
        if (d[i].binding == binding && d[i].access != VYB_ACCESS_WORKGROUP) return &d[i];
    return nullptr;
}

int32_t vyb_program_from_op(const char* op_id, const vyb_buffer_decl* decls, uint32_t n_decls, const uint32_t* op_spec,
                            uint32_t n_spec, vyb_program** program) {
    if (!op_id || !decls || !program) return fail_invalid_program("Fix: pass a non-null op id, buffer declarations and program out-pointer.");
    const std::string id = op_id;
    auto need = [&](uint32_t slots) -> bool {
        for (uint32_t b = 0; b < slots; ++b)
            if (!decl_at(decls, n_decls, b) || !decl_at(decls, n_decls, b)->name) return false;
        return true;
    };
    auto count = [&](uint32_t b) -> uint64_t { return decl_at(decls, n_decls, b)->count; };
    auto name = [&](uint32_t b) -> const char* { return decl_at(decls, n_decls, b)->name; };
    auto bad_shape = [&](const std::string& what) {
        return fail_invalid_program("Fix: the buffer counts of `" + id + "` do not describe a valid shape (" + what +
                                    "); attach the op spec to the Program metadata or correct the declarations.");
    };
    vyb_program* out = nullptr;
    int32_t rc = VYB_OK;
    if (id == "vyre-libs::nn::linear_4bit_affine_grouped") {
        // x=0, w=1, scale=2, zp=3, b=4, out=5 (linear_4bit.rs:757-771); spec = [in_dim, out_dim, group_size, batch]
        if (!need(6)) return bad_shape("six buffers x, w, scale, zero_point, b, out expected");
        uint64_t in_dim, out_dim, group, batch;
        if (op_spec && n_spec >= 4) {
            in_dim = op_spec[0]; out_dim = op_spec[1]; group = op_spec[2]; batch = op_spec[3];
        } else {
            out_dim = count(4);
            if (!out_dim || (count(1) * 8) % out_dim) return bad_shape("packed words are not a multiple of out_dim");
            in_dim = count(1) * 8 / out_dim;
            if (!in_dim || count(0) % in_dim) return bad_shape("x is not a multiple of in_dim");
            batch = count(0) / in_dim;
            const uint64_t groups = count(2) / out_dim;
            if (!groups || count(2) % out_dim || in_dim % groups) return bad_shape("scale sidecar is not groups x out_dim");
            group = in_dim / groups;
        }
        rc = vyb_nn_linear_4bit_affine_grouped_batched(name(0), name(1), name(2), name(3), name(4), name(5), uint32_t(in_dim),
                                                       uint32_t(out_dim), uint32_t(group), uint32_t(batch), &out);
    } else if (id == "vyre-libs::nn::linear_4bit") {
        if (!need(4)) return bad_shape("four buffers x, w, b, out expected");
        const uint64_t in_dim = op_spec && n_spec >= 2 ? op_spec[0] : count(0);
        const uint64_t out_dim = op_spec && n_spec >= 2 ? op_spec[1] : count(2);
        rc = vyb_nn_linear_4bit(name(0), name(1), name(2), name(3), uint32_t(in_dim), uint32_t(out_dim), &out);
    } else if (id == "vyre-libs::quant::int4_batched_matvec_f32_scaled" || id == "vyre-libs::quant::int4_matvec_f32_scaled" ||
               id == "vyre-primitives::math::quantized::i4x8_batched_matvec_f32_scaled" ||
               id == "vyre-primitives::math::quantized::i4x8_matvec_f32_scaled") {
        // weights=0, x=1, scales=2, out=3 (programs.rs:217-225); spec = [batch, rows, cols]
        if (!need(4)) return bad_shape("four buffers weights, x, scales, out expected");
        uint64_t batch, rows, cols;
        if (op_spec && n_spec >= 3) {
            batch = op_spec[0]; rows = op_spec[1]; cols = op_spec[2];
        } else {
            rows = count(2);
            if (!rows || count(3) % rows) return bad_shape("out is not batch x rows");
            batch = count(3) / rows;
            if (!batch || count(1) % batch) return bad_shape("x is not batch x cols");
            cols = count(1) / batch;
        }
        const uint32_t lib = id.rfind("vyre-libs", 0) == 0 ? 1u : 0u;
        if (id.find("batched") != std::string::npos)
            rc = vyb_math_i4x8_batched_matvec_f32_scaled(name(0), name(1), name(2), name(3), uint32_t(batch), uint32_t(rows),
                                                         uint32_t(cols), lib, &out);
        else
            rc = vyb_math_i4x8_matvec_f32_scaled(name(0), name(1), name(2), name(3), uint32_t(rows), uint32_t(cols), lib, &out);
    } else if (id == "vyre-libs::nn::moe_gate") {
        // scores=0, indices=1, weights=2 (gating.rs:56-68); spec = [num_experts, k]
        if (!need(3)) return bad_shape("three buffers scores, indices, weights expected");
        const uint64_t experts = op_spec && n_spec >= 2 ? op_spec[0] : count(0);
        const uint64_t k = op_spec && n_spec >= 2 ? op_spec[1] : count(1);
        rc = vyb_nn_moe_gate(name(0), name(1), name(2), uint32_t(experts), uint32_t(k), &out);
    } else if (id == "vyre-libs::nn::swiglu") {
        if (!need(3)) return bad_shape("three buffers gate, up, out expected");
        rc = vyb_nn_swiglu_typed(name(0), name(1), name(2), uint32_t(op_spec && n_spec >= 1 ? op_spec[0] : count(0)),
                                 decl_at(decls, n_decls, 0)->dtype, &out);
    } else if (id == "vyre-libs::nn::residual_add") {
        if (!need(3)) return bad_shape("three buffers residual, branch, out expected");
        rc = vyb_nn_residual_add_typed(name(0), name(1), name(2), uint32_t(count(0)), decl_at(decls, n_decls, 0)->dtype, &out);
    } else if (id == "vyre-libs::nn::learned_rms_norm" || id == "vyre-libs::nn::gated_rms_norm") {
        // input=0, weight=1, [gate=2,] out; hidden = count(weight), rows = count(input) / hidden; spec = [eps bits]
        const bool gated = id == "vyre-libs::nn::gated_rms_norm";
        if (!need(gated ? 4 : 3)) return bad_shape(gated ? "four buffers input, weight, gate, out expected" : "three buffers input, weight, out expected");
        const uint64_t hidden = count(1);
        if (!hidden || count(0) % hidden) return bad_shape("input elements are not rows x hidden");
        if (!op_spec || n_spec < 1) return bad_shape("the op spec must carry eps as f32 bits");
        float eps;
        std::memcpy(&eps, &op_spec[0], 4);
        if (gated)
            rc = vyb_nn_gated_rms_norm(name(0), name(1), name(2), name(3), uint32_t(count(0) / hidden), uint32_t(hidden), eps,
                                       decl_at(decls, n_decls, 0)->dtype, &out);
        else
            rc = vyb_nn_learned_rms_norm(name(0), name(1), name(2), uint32_t(count(0) / hidden), uint32_t(hidden), eps,
                                         decl_at(decls, n_decls, 0)->dtype, &out);
    } else if (id == "vyre-libs::quant::q4_k_unpack" || id == "vyre-libs::quant::q2_k_unpack") {
        if (!need(4)) return bad_shape("four buffers packed, scales, mins, out expected");
        rc = id == "vyre-libs::quant::q4_k_unpack" ? vyb_quant_q4_k_unpack(name(0), name(1), name(2), name(3), uint32_t(count(3)), &out)
                                                   : vyb_quant_q2_k_unpack(name(0), name(1), name(2), name(3), uint32_t(count(3)), &out);
    } else if (id == "vyre-libs::quant::q4_k_linear" || id == "vyre-libs::quant::q2_k_linear") {
        if (!need(6)) return bad_shape("six buffers x, w_packed, w_scales, w_mins, b, out expected");
        rc = id == "vyre-libs::quant::q4_k_linear"
                 ? vyb_quant_q4_k_linear(name(0), name(1), name(2), name(3), name(4), name(5), uint32_t(count(0)), uint32_t(count(5)), &out)
                 : vyb_quant_q2_k_linear(name(0), name(1), name(2), name(3), name(4), name(5), uint32_t(count(0)), uint32_t(count(5)), &out);
    } else if (id == "vyre-libs::quant::int8_unpack") {
        if (!need(3)) return bad_shape("three buffers packed, scales, out expected");
        const uint64_t n = op_spec && n_spec >= 2 ? op_spec[0] : count(0);
        const uint64_t rows = count(1);
        if (!rows || n % rows) return bad_shape("packed values are not rows x cols");
        rc = vyb_quant_int8_unpack(name(0), name(1), name(2), uint32_t(n), uint32_t(op_spec && n_spec >= 2 ? op_spec[1] : n / rows), &out);
    } else if (id == "vyre-libs::math::matmul" || id == "vyre-libs::math::matmul_bias") {
        // a=0, b=1, [bias=2,] out=last (matmul.rs:120-131, 252-268); spec = [m, k, n] (m cannot be recovered from the
        // counts alone unless bias gives n)
        const bool bias = id.back() == 's';
        if (!need(bias ? 4 : 3)) return bad_shape(bias ? "four buffers a, b, bias, out expected" : "three buffers a, b, out expected");
        uint64_t m, k, n;
        if (op_spec && n_spec >= 3) {
            m = op_spec[0]; k = op_spec[1]; n = op_spec[2];
        } else if (bias) {
            n = count(2);
            if (!n || count(1) % n || count(3) % n) return bad_shape("b and out are not multiples of the bias length");
            k = count(1) / n;
            m = count(3) / n;
        } else {
            return bad_shape("matmul needs the op spec [m, k, n]: three counts m*k, k*n, m*n do not fix it uniquely");
        }
        rc = bias ? vyb_math_matmul_bias(name(0), name(1), name(2), name(3), uint32_t(m), uint32_t(k), uint32_t(n), &out)
                  : vyb_math_matmul(name(0), name(1), name(2), uint32_t(m), uint32_t(k), uint32_t(n), &out);
    } else if (id == "vyre-libs::nn::linear" || id == "vyre-libs::nn::linear_tiled") {
        // x=0, w=1, b=2, out=3 (builder.rs:139-162, tiled.rs:20-50); spec = [in_dim, out_dim, tile]
        if (!need(4)) return bad_shape("four buffers x, w, b, out expected");
        const uint64_t in_dim = op_spec && n_spec >= 2 ? op_spec[0] : count(0);
        const uint64_t out_dim = op_spec && n_spec >= 2 ? op_spec[1] : count(2);
        if (id == "vyre-libs::nn::linear")
            rc = flat_matmul_program("vyre-libs::nn::linear", name(0), name(1), name(2), name(3), 1, uint32_t(in_dim),
                                     uint32_t(out_dim), &out);
        else
            rc = vyb_nn_linear_tiled(name(0), name(1), name(2), name(3), uint32_t(in_dim), uint32_t(out_dim),
                                     op_spec && n_spec >= 3 ? op_spec[2] : 32u, &out);
    } else {
        return fail_unsupported("rebuilding a program for operator `" + id + "` from buffer declarations");
    }
    if (rc != VYB_OK) return rc;
    // cross-check: every declared storage buffer must match the rebuilt program's buffer of the same slot
    for (const BufferDecl& b : out->p.buffers) {
        if (b.access == VYB_ACCESS_WORKGROUP) continue;
        const vyb_buffer_decl* d = decl_at(decls, n_decls, b.binding);
        if (!d || d->count != b.count || d->dtype != b.dtype || d->access != b.access) {
            const std::string which = b.name;
            delete out;
            return fail_invalid_program("Fix: buffer `" + which + "` (slot " + std::to_string(b.binding) + ") of `" + id +
                                        "` disagrees with the shape recovered from the op spec or the other buffers "
                                        "(count, dtype or access differ); the artifact is not the program this op id names.");
        }
    }
    *program = out;
    return VYB_OK;
}

const char* vyb_program_op_id(const vyb_program* p) { return p ? p->p.op_id.c_str() : ""; }
uint32_t vyb_program_buffer_count(const vyb_program* p) { return p ? uint32_t(p->p.buffers.size()) : 0; }
int32_t vyb_program_buffer(const vyb_program* p, uint32_t index, vyb_buffer_decl* out) {
    if (!p || !out || index >= p->p.buffers.size())
        return fail_invalid_program("Fix: buffer index is out of range for this program.");
    const BufferDecl& b = p->p.buffers[index];
    out->name = b.name.c_str();
    out->binding = b.binding;
    out->access = b.access;
    out->dtype = b.dtype;
    out->count = b.count;
    out->has_output_byte_range = b.has_output_byte_range ? 1 : 0;
    out->output_byte_begin = b.output_byte_begin;
    out->output_byte_end = b.output_byte_end;
    return VYB_OK;
}
void vyb_program_workgroup_size(const vyb_program* p, uint32_t out[3]) {
    for (int i = 0; i < 3; ++i) out[i] = p ? p->p.workgroup[i] : 0;
}
uint32_t vyb_program_is_trap(const vyb_program* p) { return p && p->p.trap ? 1 : 0; }
const char* vyb_program_trap_message(const vyb_program* p) { return p ? p->p.trap_message.c_str() : ""; }
void vyb_program_fingerprint(const vyb_program* p, uint8_t out[32]) {
    Digest d = p->p.fingerprint();
    std::memcpy(out, d.data(), 32);
}
void vyb_program_free(vyb_program* p) { delete p; }

}  // extern "C"
