// Host-side data model of the native backend: Program / Artifact / TargetPayload mirrors and the error
// channel. Mirrors the shapes of vyre_foundation::ir::Program (buffers + workgroup size + op region),
// vyre_megakernel::{Artifact, TargetPayload} and vyre_driver::BackendError; see include/vyre_b200.h for the
// per-item reference citations.
#pragma once

#include <array>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/vyre_b200.h"

namespace vyb {

using Digest = std::array<uint8_t, 32>;

// ---- error channel -----------------------------------------------------------------------------------
// Thread-local last error; every message carries "Fix: " (vyre-driver/src/backend/error.rs:61-75).
int32_t fail(int32_t code, const std::string& message);
int32_t fail_invalid_program(const std::string& fix);                             // BackendError::InvalidProgram
int32_t fail_unsupported(const std::string& name);                                // BackendError::UnsupportedFeature
int32_t fail_dispatch(int32_t cuda_code, const std::string& message);             // BackendError::DispatchFailed
int32_t fail_oom(uint64_t requested, uint64_t available);                         // BackendError::DeviceOutOfMemory
int32_t fail_device_lost(const std::string& device, uint64_t generation, const std::string& message);
void clear_error();

constexpr const char* BACKEND_ID = "cuda-b200";
constexpr const char* TARGET_ID = "nvidia-sm100a";
constexpr const char* PAYLOAD_FORMAT = "b200-native";
constexpr uint32_t PAYLOAD_FORMAT_VERSION = 1;

// ---- operator kinds (dispatch keys of the native facet; op ids are the reference's, verbatim) ----------
enum class OpKind : uint32_t {
    Linear4Bit = 1,
    Linear4BitAffineGrouped = 2,
    I4Unpack = 3,
    I4DotI32 = 4,
    I4DotF32Scaled = 5,
    I4BatchedMatvec = 6,  // also the unbatched matvec (batch == 1)
    I4BatchedMatmul = 7,
    I4BatchedMatmulTop1 = 8,
    Int8Unpack = 9,
    Int8Pack = 10,
    LinearRows = 11,
    MatmulU32 = 12,
    MoeGate = 13,
    SoftmaxTopK = 14,
    TopK = 15,
    Swiglu = 16,
    ExpertMlp = 17,
    MoeLayerAccumulate = 18,
    ResidualAdd = 19,
    RmsNorm = 20,      // learned_rms_norm and gated_rms_norm
    KQuantUnpack = 21, // q4_k_unpack, q2_k_unpack
    KQuantLinear = 22, // q4_k_linear, q2_k_linear
    // serving-layout operators
    LinearInt4GroupedRowmajor = 32,
    LinearInt8WeightOnly = 33,
    LinearInt8Dynamic = 34,
    MoeFfnInt4 = 35,
    LinearInt4Block = 36,  // the int4 projection with a learned RMSNorm in front and / or a residual add behind, one node
};

struct BufferDecl {
    std::string name;
    uint32_t binding = 0;
    uint32_t access = VYB_ACCESS_READ_ONLY;
    uint32_t dtype = VYB_DT_U32;
    uint32_t count = 0;
    bool has_output_byte_range = false;
    uint64_t output_byte_begin = 0, output_byte_end = 0;
};

uint32_t dtype_size_bytes(uint32_t dtype);

// Operator parameters: the IR literals of the reference Program made explicit (the reference Program does not
// carry in_dim/out_dim/group_size as fields; the native facet needs them as an op spec).
struct OpParams {
    uint32_t u[12] = {0};
};

struct Program {
    std::string op_id;
    OpKind kind = OpKind::Linear4Bit;
    std::array<uint32_t, 3> workgroup{{1, 1, 1}};
    std::vector<BufferDecl> buffers;
    OpParams params;
    bool trap = false;
    std::string trap_message;

    std::vector<uint8_t> to_wire() const;   // canonical little-endian bytes ("VYBP" framing)
    static bool from_wire(const uint8_t* bytes, size_t len, Program* out, std::string* error);
    Digest fingerprint() const;
    const BufferDecl* buffer_by_binding(uint32_t binding) const;
};

// vyre_megakernel::Artifact: immutable compiled single-node graph; digest = blake3 of the framed bytes.
struct Artifact {
    Program program;
    std::vector<uint8_t> bytes;  // "VYBA" framing around the program wire
    Digest digest{};
};

// One emitted target module (vyre-megakernel/src/target.rs:236-249 EmittedTargetModule).
struct TargetModule {
    std::string entry_point;  // must be "main" (vyre-driver/src/materialize.rs:125-132)
    uint32_t node = 0;
    std::array<uint32_t, 3> workgroup{{1, 1, 1}};
    std::array<uint32_t, 3> grid{{1, 1, 1}};
    uint32_t dynamic_shared_bytes = 0;
    uint32_t kernel_variant = 0;
    std::vector<uint8_t> program_wire;
};

// vyre_megakernel::TargetPayload (envelope.rs:196-300): authenticated immutable bytes bound to an artifact.
struct Payload {
    Digest neutral_artifact{};
    std::string format;
    uint32_t format_version = 0;
    vyb_target_profile profile{};
    std::vector<TargetModule> modules;
    std::vector<uint8_t> bytes;  // full "VYBT" frame, what to_bytes()/from_bytes() exchange
    Digest digest{};             // blake3 over `bytes` without the trailing digest field

    void seal();  // (re)builds `bytes` and `digest` from the fields
    static bool from_bytes(const uint8_t* b, size_t len, Payload* out, std::string* error);
};

vyb_target_profile native_profile();
bool profile_equal(const vyb_target_profile& a, const vyb_target_profile& b);

// kernel variants recorded in the payload module
enum KernelVariant : uint32_t {
    KV_GENERIC = 0,
    KV_INT4_GEMV_TMA = 1,
    KV_INT4_PREFILL_TCGEN05 = 2,
    KV_INT8_GEMM_TCGEN05 = 3,
    KV_MOE_FUSED = 4,
    KV_AFFINE_GROUPED_OUTPUT_MAJOR = 5,  // the reference's own 4-bit layout, thread per output, 8 batch rows per weight
    KV_I4_MATVEC_WARP_ROWS = 6,          // i4x8 matvec, warp per row
    KV_K_QUANT_WORD_COLUMNS = 7,         // K-quant linear: thread per packed word column, k slices folded in fixed order
    KV_RMS_NORM_TREE = 8,                // RMSNorm rows of 2048 elements and more: sum of squares as a tree, not a chain
    KV_INT4_BLOCK_GEMV = 9,              // decode GEMV with the norm in its prologue and / or the residual add in its stores
};

uint32_t select_kernel_variant(const Program& p);

}  // namespace vyb

struct vyb_program {
    vyb::Program p;
};
struct vyb_artifact {
    vyb::Artifact a;
};
struct vyb_payload {
    vyb::Payload p;
};
