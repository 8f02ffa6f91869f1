// Artifact / TargetPayload mirrors and the pure target-compiler facet.
//   compile        = ProgramGraph::from_program + vyre_megakernel::compile (vyre-megakernel/src/lib.rs:832)
//   target_compile = TargetCompiler::compile via compile_selected_modules (vyre-megakernel/src/target.rs:180-322)
// The payload module carries the selected kernel variant and launch geometry instead of PTX text; it stays
// digest-bound to the neutral artifact exactly as TargetPayload::new does (envelope.rs:246-300).
#include <algorithm>
#include <cstdio>

#include "blake3.hpp"
#include "model.hpp"

namespace vyb {

namespace {
void put_u32(std::vector<uint8_t>& v, uint32_t x) {
    for (int i = 0; i < 4; ++i) v.push_back(uint8_t(x >> (8 * i)));
}
void put_str(std::vector<uint8_t>& v, const std::string& s) {
    put_u32(v, uint32_t(s.size()));
    v.insert(v.end(), s.begin(), s.end());
}
void put_bytes(std::vector<uint8_t>& v, const std::vector<uint8_t>& b) {
    put_u32(v, uint32_t(b.size()));
    v.insert(v.end(), b.begin(), b.end());
}
struct Rd {
    const uint8_t* p;
    size_t n, off;
    bool ok = true;
    uint32_t u32() {
        if (off + 4 > n) { ok = false; return 0; }
        uint32_t x = 0;
        for (int i = 0; i < 4; ++i) x |= uint32_t(p[off + i]) << (8 * i);
        off += 4;
        return x;
    }
    bool raw(void* dst, size_t len) {
        if (off + len > n) { ok = false; return false; }
        std::memcpy(dst, p + off, len);
        off += len;
        return true;
    }
    std::vector<uint8_t> bytes() {
        uint32_t len = u32();
        if (!ok || off + len > n) { ok = false; return {}; }
        std::vector<uint8_t> v(p + off, p + off + len);
        off += len;
        return v;
    }
    std::string str() {
        auto b = bytes();
        return std::string(b.begin(), b.end());
    }
};
}  // namespace

vyb_target_profile native_profile() {
    vyb_target_profile pr{};
    std::snprintf(pr.identity, sizeof(pr.identity), "%s", "nvidia-sm100a-b200");
    pr.generation = 100;
    pr.max_workgroup_size[0] = 1024;
    pr.max_workgroup_size[1] = 1024;
    pr.max_workgroup_size[2] = 64;
    pr.max_invocations = 1024;
    pr.max_dynamic_shared_bytes = 232448;
    pr.subgroup_size = 32;
    return pr;
}

bool profile_equal(const vyb_target_profile& a, const vyb_target_profile& b) {
    return std::strncmp(a.identity, b.identity, sizeof(a.identity)) == 0 && a.generation == b.generation &&
           std::memcmp(a.max_workgroup_size, b.max_workgroup_size, sizeof(a.max_workgroup_size)) == 0 &&
           a.max_invocations == b.max_invocations && a.max_dynamic_shared_bytes == b.max_dynamic_shared_bytes &&
           a.subgroup_size == b.subgroup_size;
}

// Which hand-written kernel serves a program. Decided at target-compile time from the op spec alone (pure:
// no device is consulted), recorded in the payload and re-derived at materialisation as a cross-check.
uint32_t select_kernel_variant(const Program& p) {
    switch (p.kind) {
        case OpKind::LinearInt4GroupedRowmajor: {
            const uint32_t batch = p.params.u[0], in_dim = p.params.u[1], group = p.params.u[3];
            // decode batches stream the weights once per 8 rows; from 65 rows on the contraction is dense enough
            // for the tensor-core path with in-kernel dequantisation
            const bool gemv_ok = group == 128 && in_dim % 1024 == 0;
            const bool prefill_ok = in_dim % 64 == 0 && group % 64 == 0 && in_dim % group == 0;
            if (gemv_ok && (batch <= 64 || !prefill_ok)) return KV_INT4_GEMV_TMA;
            if (prefill_ok && batch > 8) return KV_INT4_PREFILL_TCGEN05;
            return KV_GENERIC;
        }
        case OpKind::LinearInt4Block: {
            // decode shapes whose GEMV takes the norm and / or the residual add into its own launch; everything else runs
            // the stand-alone kernels one after the other inside the node
            const uint32_t batch = p.params.u[0], in_dim = p.params.u[1], group = p.params.u[3], parts = p.params.u[5];
            const bool whole_rows = in_dim == 2048 || in_dim == 4096;
            const bool k_blocks = in_dim > 4096 && in_dim % 2048 == 0 && (parts & 6u);  // the residual add or SwiGLU joins that form, a norm does not
            if (group == 128 && ((whole_rows && batch <= 2) || (k_blocks && batch <= 4))) return KV_INT4_BLOCK_GEMV;
            Program bare = p;
            bare.kind = OpKind::LinearInt4GroupedRowmajor;
            return select_kernel_variant(bare);
        }
        case OpKind::LinearInt8Dynamic: return KV_INT8_GEMM_TCGEN05;
        case OpKind::MoeFfnInt4: return KV_MOE_FUSED;
        // the reference's own operators: small shapes keep the kernels that follow the reference's evaluation order
        // (bit-exact against its interpreter), large ones get kernels shaped for the layout (same dequantisation,
        // different summation order)
        case OpKind::Linear4BitAffineGrouped: {
            const uint64_t in_dim = p.params.u[0], out_dim = p.params.u[1], group = p.params.u[2], batch = p.params.u[3];
            const bool big = in_dim * out_dim * batch >= (1ull << 24);
            return big && in_dim % 8 == 0 && group % 8 == 0 && in_dim % group == 0 ? KV_AFFINE_GROUPED_OUTPUT_MAJOR : KV_GENERIC;
        }
        case OpKind::I4BatchedMatvec: {
            const uint64_t batch = p.params.u[0], rows = p.params.u[1], cols = p.params.u[2];
            return batch * rows * cols >= (1ull << 22) ? KV_I4_MATVEC_WARP_ROWS : KV_GENERIC;
        }
        // long rows: the chain of `hidden` dependent additions becomes a tree (f32 rounding of the sum differs, about 1e-7)
        case OpKind::RmsNorm: return p.params.u[1] >= 2048 ? KV_RMS_NORM_TREE : KV_GENERIC;
        case OpKind::KQuantLinear: {
            const uint64_t in_dim = p.params.u[0], out_dim = p.params.u[1], bits = p.params.u[2];
            return in_dim * out_dim >= (1ull << 20) && out_dim % (4 * (32 / bits)) == 0 ? KV_K_QUANT_WORD_COLUMNS : KV_GENERIC;
        }
        default: return KV_GENERIC;
    }
}

void Payload::seal() {
    std::vector<uint8_t> v = {'V', 'Y', 'B', 'T'};
    put_u32(v, 1);
    v.insert(v.end(), neutral_artifact.begin(), neutral_artifact.end());
    put_str(v, format);
    put_u32(v, format_version);
    v.insert(v.end(), reinterpret_cast<const uint8_t*>(&profile),
             reinterpret_cast<const uint8_t*>(&profile) + sizeof(profile));
    put_u32(v, uint32_t(modules.size()));
    for (const TargetModule& m : modules) {
        put_str(v, m.entry_point);
        put_u32(v, m.node);
        for (uint32_t w : m.workgroup) put_u32(v, w);
        for (uint32_t g : m.grid) put_u32(v, g);
        put_u32(v, m.dynamic_shared_bytes);
        put_u32(v, m.kernel_variant);
        put_bytes(v, m.program_wire);
    }
    blake3(v.data(), v.size(), digest.data());
    v.insert(v.end(), digest.begin(), digest.end());
    bytes = std::move(v);
}

bool Payload::from_bytes(const uint8_t* b, size_t len, Payload* out, std::string* error) {
    if (len < 8 + 32 + 32 || std::memcmp(b, "VYBT", 4) != 0) {
        *error = "target payload does not start with the VYBT magic";
        return false;
    }
    // authenticate first: trailing 32 bytes = blake3 of everything before them
    Digest want;
    blake3(b, len - 32, want.data());
    if (std::memcmp(want.data(), b + len - 32, 32) != 0) {
        *error = "target payload digest does not match its bytes";
        return false;
    }
    Rd r{b, len - 32, 4};
    if (r.u32() != 1) {
        *error = "unknown target payload frame version";
        return false;
    }
    Payload p;
    r.raw(p.neutral_artifact.data(), 32);
    p.format = r.str();
    p.format_version = r.u32();
    r.raw(&p.profile, sizeof(p.profile));
    uint32_t nm = r.u32();
    if (!r.ok || nm > 1024) {
        *error = "target payload is truncated";
        return false;
    }
    for (uint32_t i = 0; i < nm; ++i) {
        TargetModule m;
        m.entry_point = r.str();
        m.node = r.u32();
        for (auto& w : m.workgroup) w = r.u32();
        for (auto& g : m.grid) g = r.u32();
        m.dynamic_shared_bytes = r.u32();
        m.kernel_variant = r.u32();
        m.program_wire = r.bytes();
        p.modules.push_back(std::move(m));
    }
    if (!r.ok || r.off != len - 32) {
        *error = "target payload is truncated or has trailing bytes";
        return false;
    }
    p.digest = want;
    p.bytes.assign(b, b + len);
    *out = std::move(p);
    return true;
}

}  // namespace vyb

using namespace vyb;

namespace {
const char* const SUPPORTED_OPS[] = {
    "vyre-libs::nn::linear_4bit",
    "vyre-libs::nn::linear_4bit_affine_grouped",
    "vyre-libs::nn::linear_rows",
    "vyre-libs::math::matmul",
    "vyre-libs::quant::int4_dot_i32",
    "vyre-libs::quant::int4_dot_f32_scaled",
    "vyre-libs::quant::int4_matvec_f32_scaled",
    "vyre-libs::quant::int4_batched_matvec_f32_scaled",
    "vyre-libs::quant::int4_batched_matmul_f32_scaled",
    "vyre-libs::quant::int4_batched_matmul_top1_f32_scaled",
    "vyre-primitives::math::quantized::unpack_i4x8",
    "vyre-primitives::math::quantized::i4x8_dot_i32",
    "vyre-primitives::math::quantized::i4x8_dot_f32_scaled",
    "vyre-primitives::math::quantized::i4x8_matvec_f32_scaled",
    "vyre-primitives::math::quantized::i4x8_batched_matvec_f32_scaled",
    "vyre-primitives::math::quantized::i4x8_batched_matmul_f32_scaled",
    "vyre-primitives::math::quantized::i4x8_batched_matmul_top1_f32_scaled",
    "vyre-libs::quant::int8_pack",
    "vyre-libs::quant::int8_unpack",
    "vyre-libs::nn::moe_gate",
    "vyre-libs::nn::softmax_top_k",
    "vyre-libs::nn::top_k",
    "vyre-libs::nn::moe::expert_mlp",
    "vyre-libs::nn::moe_layer_accumulate",
    "vyre-libs::nn::swiglu",
    "vyre-libs::nn::residual_add",
    "vyre-libs::nn::learned_rms_norm",
    "vyre-libs::nn::gated_rms_norm",
    "vyre-libs::quant::q4_k_unpack",
    "vyre-libs::quant::q2_k_unpack",
    "vyre-libs::quant::q4_k_linear",
    "vyre-libs::quant::q2_k_linear",
    "vyre-b200::nn::linear_int4_grouped_rowmajor",
    "vyre-b200::nn::linear_int4_block",
    "vyre-b200::nn::linear_int8_weight_only",
    "vyre-b200::nn::linear_int8_dynamic",
    "vyre-b200::nn::moe_ffn_int4",
};
}

extern "C" {

int32_t vyb_registration(vyb_registration_info* out) {
    if (!out) return fail_invalid_program("Fix: pass a non-null registration out-pointer.");
    out->id = BACKEND_ID;
    out->target_id = TARGET_ID;
    out->payload_format = PAYLOAD_FORMAT;
    out->format_version = PAYLOAD_FORMAT_VERSION;
    out->precedence = 4;  // ahead of the generic CUDA backend (rank 5) for the ops it supports
    out->profile = native_profile();
    return VYB_OK;
}
uint32_t vyb_supported_op_count(void) { return uint32_t(sizeof(SUPPORTED_OPS) / sizeof(SUPPORTED_OPS[0])); }
const char* vyb_supported_op(uint32_t index) { return index < vyb_supported_op_count() ? SUPPORTED_OPS[index] : nullptr; }

int32_t vyb_compile(const vyb_program* program, vyb_artifact** artifact) {
    if (!program || !artifact) return fail_invalid_program("Fix: pass a non-null program and artifact out-pointer.");
    if (program->p.trap)
        return fail_invalid_program(program->p.trap_message.empty()
                                        ? std::string("Fix: the builder rejected its arguments and produced a trap program.")
                                        : program->p.trap_message);
    auto* a = new vyb_artifact();
    a->a.program = program->p;
    std::vector<uint8_t> wire = program->p.to_wire();
    std::vector<uint8_t> v = {'V', 'Y', 'B', 'A'};
    put_u32(v, 1);
    put_u32(v, 1);  // one fusion group, one node
    put_bytes(v, wire);
    blake3(v.data(), v.size(), a->a.digest.data());
    a->a.bytes = std::move(v);
    *artifact = a;
    clear_error();
    return VYB_OK;
}
void vyb_artifact_digest(const vyb_artifact* a, uint8_t out[32]) { std::memcpy(out, a->a.digest.data(), 32); }
void vyb_artifact_free(vyb_artifact* a) { delete a; }

int32_t vyb_target_compile(const vyb_artifact* artifact, vyb_payload** payload) {
    if (!artifact || !payload) return fail_invalid_program("Fix: pass a non-null artifact and payload out-pointer.");
    const Program& prog = artifact->a.program;
    auto* h = new vyb_payload();
    Payload& p = h->p;
    p.neutral_artifact = artifact->a.digest;
    p.format = PAYLOAD_FORMAT;
    p.format_version = PAYLOAD_FORMAT_VERSION;
    p.profile = native_profile();
    TargetModule m;
    m.entry_point = "main";
    m.node = 0;
    m.workgroup = prog.workgroup;
    m.kernel_variant = select_kernel_variant(prog);
    // grid as the reference derives it: ceil(max output elements / workgroup invocations)
    // (vyre-reference/src/execution/hashmap/mod.rs:294-313); the native kernels size their own launch.
    uint64_t max_out = 1;
    for (const BufferDecl& b : prog.buffers)
        if (b.access == VYB_ACCESS_OUTPUT || b.access == VYB_ACCESS_READ_WRITE) max_out = std::max<uint64_t>(max_out, b.count);
    uint64_t inv = uint64_t(prog.workgroup[0]) * prog.workgroup[1] * prog.workgroup[2];
    m.grid = {uint32_t((max_out + inv - 1) / inv), 1, 1};
    m.program_wire = prog.to_wire();
    p.modules.push_back(std::move(m));
    p.seal();
    *payload = h;
    clear_error();
    return VYB_OK;
}
void vyb_payload_digest(const vyb_payload* p, uint8_t out[32]) { std::memcpy(out, p->p.digest.data(), 32); }
void vyb_payload_neutral_artifact(const vyb_payload* p, uint8_t out[32]) {
    std::memcpy(out, p->p.neutral_artifact.data(), 32);
}
const char* vyb_payload_format(const vyb_payload* p) { return p->p.format.c_str(); }
uint32_t vyb_payload_kernel_variant(const vyb_payload* p) {
    return p && !p->p.modules.empty() ? p->p.modules.front().kernel_variant : 0u;
}
int32_t vyb_payload_bytes(const vyb_payload* p, const uint8_t** bytes, size_t* len) {
    if (!p || !bytes || !len) return fail_invalid_program("Fix: pass non-null payload, bytes and len pointers.");
    *bytes = p->p.bytes.data();
    *len = p->p.bytes.size();
    return VYB_OK;
}
int32_t vyb_payload_from_bytes(const uint8_t* bytes, size_t len, vyb_payload** payload) {
    if (!bytes || !payload) return fail_invalid_program("Fix: pass non-null payload bytes and out-pointer.");
    auto* h = new vyb_payload();
    std::string err;
    if (!Payload::from_bytes(bytes, len, &h->p, &err)) {
        delete h;
        return fail_invalid_program("Fix: " + err + "; re-run the target compiler instead of editing payload bytes.");
    }
    *payload = h;
    clear_error();
    return VYB_OK;
}
void vyb_payload_free(vyb_payload* p) { delete p; }

}  // extern "C"
